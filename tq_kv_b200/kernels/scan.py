"""Python entry point of the matrix-state recurrences (csrc/linear_scan.cu)."""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import torch

from ._lib import KernelError, check, core, need_contiguous, ptr, stream

SCAN_DECAY, SCAN_DELTA = 0, 1
MAX_KEY_WIDTH = 256


def linear_scan(proj: torch.Tensor, state: torch.Tensor, cu_seqlens: torch.Tensor, slots: torch.Tensor,
                out: torch.Tensor, *, n_seqs: int, heads: int, key_dim: int, value_dim: int, off_q: int, off_k: int,
                off_v: int, head_decay: Optional[torch.Tensor] = None, silu: bool = False,
                decay_logit: Optional[torch.Tensor] = None, off_a: int = 0, unit_eps: float = 1e-6,
                single_tokens: bool = False):
    """Walks each sequence's tokens of this step through a d x e float32 state per head and writes
    o_t = S_t^T q_t into out [T, heads * e] (float32).

    proj float32 [T, ld] holds, heads side by side, the query vectors from column off_q, the keys from off_k
    and the values from off_v.  With `head_decay` (float32 [heads]):  S_t = c_head S_{t-1} + k_t v_t^T, q/k/v
    first through silu if `silu`.  With `decay_logit` (float32 [T, heads * d]) and removal logits from column
    off_a of proj, the generalised delta rule:
        S_t = diag(w_t) S_{t-1} - (a_t * u_t)(u_t^T S_{t-1}) + k_t v_t^T,
        w = exp(-exp(-1/2) sigmoid(decay_logit)), a = sigmoid(removal logit), u = k / sqrt(|k|^2 + unit_eps).
    Unless `single_tokens`, the kernels work in place: afterwards proj holds silu(q | k | v) (first rule, with `silu`) or -(a * u) in
    place of the removal logits, and decay_logit holds w.  state float32 [slots, heads, d, e] is read at
    slots[b] before the first token and written after the last.  `single_tokens`: every sequence brings
    exactly one token (the kernel built for decoding runs)."""
    T, ld = proj.shape
    d, e = int(key_dim), int(value_dim)
    if proj.dtype != torch.float32 or out.dtype != torch.float32 or state.dtype != torch.float32:
        raise KernelError("linear_scan: projections, state and out must be float32")
    if tuple(state.shape[1:]) != (heads, d, e):
        raise KernelError(f"linear_scan: state has shape {tuple(state.shape)}, expected [slots, {heads}, {d}, {e}]")
    if tuple(out.shape) != (T, heads * e) or out.stride(1) != 1 or proj.stride(1) != 1:
        raise KernelError("linear_scan: out must be [T, heads * e]; rows contiguous")
    if not 0 < d <= MAX_KEY_WIDTH:
        raise KernelError(f"linear_scan: key width {d} is outside 1..{MAX_KEY_WIDTH}")
    if max(off_q, off_k) + heads * d > ld or off_v + heads * e > ld:
        raise KernelError("linear_scan: the projections' columns do not fit their rows")
    if (head_decay is None) == (decay_logit is None):
        raise KernelError("linear_scan: give either head_decay or decay_logit")
    if single_tokens and T != n_seqs:
        raise KernelError("linear_scan: single_tokens needs one token per sequence")
    need_contiguous(state=state, cu_seqlens=cu_seqlens, slots=slots, head_decay=head_decay)
    u = a = None
    ld_w = ld_u = 0
    if decay_logit is not None:
        if decay_logit.dtype != torch.float32 or tuple(decay_logit.shape) != (T, heads * d) or decay_logit.stride(1) != 1:
            raise KernelError("linear_scan: decay_logit must be float32 [T, heads * d]")
        if e != d or off_a + heads * d > ld:
            raise KernelError("linear_scan: the delta rule has square states; removal logits must fit the rows")
        mode, ld_w = SCAN_DELTA, decay_logit.stride(0)
        if not single_tokens:
            u = torch.empty((T, heads * d), dtype=torch.float32, device=proj.device)
            ld_u = u.stride(0)
        a = proj[:, off_a:]
    else:
        if head_decay.dtype != torch.float32 or head_decay.shape[0] != heads:
            raise KernelError("linear_scan: head_decay must be float32 [heads]")
        mode = SCAN_DECAY
    n_kernels = 1 if single_tokens else (2 if mode == SCAN_DELTA else (4 if silu else 1))
    check(core().tq_linear_scan(mode, ptr(proj[:, off_q:]), ptr(proj[:, off_k:]), ptr(proj[:, off_v:]), ptr(a),
                                proj.stride(0), ptr(decay_logit), ld_w, ptr(u), ld_u, ptr(head_decay), int(silu),
                                float(unit_eps), ptr(state), ptr(cu_seqlens), ptr(slots), int(n_seqs), T,
                                int(single_tokens), ptr(out), out.stride(0), heads, d, e, stream()),
          "linear_scan", n_kernels)
    return out


MAX_CONV_TAPS = 16
MAX_CONV_VECTOR = 256


def short_conv(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
               state: torch.Tensor, *, tok_seq: torch.Tensor, cu_seqlens: torch.Tensor, slots: torch.Tensor,
               n_seqs: int, regions: Sequence[tuple], silu: bool = True, single_tokens: bool = False,
               unit_eps: float = 1e-6, gate_raw: Optional[torch.Tensor] = None,
               beta_raw: Optional[torch.Tensor] = None, a_log: Optional[torch.Tensor] = None,
               dt_bias: Optional[torch.Tensor] = None, scalars: Optional[torch.Tensor] = None):
    """Causal convolution over time with one filter per channel, then silu (csrc/short_conv.cu):
    out[t, c] = act(bias[c] + sum_j weight[c, K-1-j] * x[t-j, c]).  x float32 [T, C] (may be a column slice),
    weight float32 [C, K], out float32 [T, >= C].  `state` float32 [slots, >= (K-1)*C] (may be a column slice of
    the per-sequence state) holds each sequence's last K-1 inputs, oldest first, and is brought up to date.
    `regions`: (first channel, channels, vector width, unit, scale) — each vector of a region with `unit` leaves
    as x * scale / sqrt(sum(x^2) + unit_eps).  With `gate_raw` float32 [T, H] the per-token scalars of a
    recurrence go to `scalars` float32 [T, H, 4]: g = exp(-exp(a_log) * softplus(gate_raw + dt_bias)), then
    sigmoid(beta_raw) if given, else the softplus itself."""
    T, C = x.shape
    K = weight.shape[1]
    if x.dtype != torch.float32 or out.dtype != torch.float32 or state.dtype != torch.float32 or weight.dtype != torch.float32:
        raise KernelError("short_conv: x, weight, out and state must be float32")
    if tuple(weight.shape) != (C, K) or not 1 <= K <= MAX_CONV_TAPS:
        raise KernelError(f"short_conv: weight must be [channels, taps <= {MAX_CONV_TAPS}]")
    if x.stride(1) != 1 or out.stride(1) != 1 or out.shape[0] != T or out.shape[1] < C:
        raise KernelError("short_conv: x and out must be contiguous along the row; out [T, >= C]")
    if state.dim() != 2 or state.stride(1) != 1 or state.shape[1] < (K - 1) * C:
        raise KernelError("short_conv: state must be [slots, >= (taps - 1) * channels]")
    if bias is not None and (bias.dtype != torch.float32 or bias.shape[0] != C):
        raise KernelError("short_conv: bias must be float32 [channels]")
    if single_tokens and T != n_seqs:
        raise KernelError("short_conv: single_tokens needs one token per sequence")
    regions = list(regions)
    if not 1 <= len(regions) <= 4:
        raise KernelError("short_conv: one to four regions")
    flat, scales = [], []
    for first, count, width, unit, scale in regions:
        if not 0 < width <= MAX_CONV_VECTOR or first < 0 or count <= 0 or first + count > C or (unit and count % width):
            raise KernelError(f"short_conv: region {(first, count, width, unit)} does not fit {C} channels "
                              f"(vectors of up to {MAX_CONV_VECTOR})")
        flat += [int(first), int(count), int(width), int(bool(unit))]
        scales.append(float(scale))
    reg = (ctypes.c_int * len(flat))(*flat)
    sc = (ctypes.c_float * len(scales))(*scales)
    H = ldg = ldb = 0
    if gate_raw is not None:
        H = gate_raw.shape[1]
        if (gate_raw.dtype != torch.float32 or gate_raw.shape[0] != T or gate_raw.stride(1) != 1 or a_log is None
                or dt_bias is None or scalars is None or a_log.shape[0] != H or dt_bias.shape[0] != H
                or a_log.dtype != torch.float32 or dt_bias.dtype != torch.float32
                or scalars.dtype != torch.float32 or tuple(scalars.shape) != (T, H, 4)):
            raise KernelError("short_conv: gate_raw float32 [T, H] needs a_log, dt_bias float32 [H] and scalars float32 [T, H, 4]")
        ldg = gate_raw.stride(0)
        if beta_raw is not None:
            if beta_raw.dtype != torch.float32 or tuple(beta_raw.shape) != (T, H) or beta_raw.stride(1) != 1:
                raise KernelError("short_conv: beta_raw must be float32 [T, H]")
            ldb = beta_raw.stride(0)
        need_contiguous(a_log=a_log, dt_bias=dt_bias, scalars=scalars)
    need_contiguous(weight=weight, bias=bias, tok_seq=tok_seq, cu_seqlens=cu_seqlens, slots=slots)
    n_kernels = 1 if single_tokens or K == 1 else 2
    check(core().tq_short_conv(ptr(x), x.stride(0), ptr(weight), ptr(bias), ptr(out), out.stride(0), ptr(state),
                               state.stride(0), ptr(tok_seq), ptr(cu_seqlens), ptr(slots), int(n_seqs), T, C, K,
                               int(silu), int(single_tokens), len(regions), reg, sc, float(unit_eps), ptr(gate_raw),
                               ldg, ptr(beta_raw), ldb, ptr(a_log), ptr(dt_bias), ptr(scalars), H, stream()),
          "short_conv", n_kernels)
    return out


def gated_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scalars: torch.Tensor, state: torch.Tensor,
               cu_seqlens: torch.Tensor, slots: torch.Tensor, out: torch.Tensor, *, n_seqs: int, heads: int,
               qk_heads: int, key_dim: int, value_dim: int, delta: bool, skip: Optional[torch.Tensor] = None,
               single_tokens: bool = False):
    """The matrix-state recurrences with one decay per head and token (csrc/linear_scan.cu).  q, k [T, qk_heads *
    d] and v [T, heads * e] are column slices of ONE float32 buffer (one row stride), ready for the recurrence;
    head h reads the q/k vectors of head h // (heads // qk_heads).  scalars float32 [T, heads, 4] holds g and a
    second number per token and head.  With `delta`:  S' = g S;  S = S' + k (beta (v - S'^T k))^T  (second = beta);
    else  S = g S + k (dt v)^T  (second = dt) and o += skip[head] * v if skip is given.  o = S^T q goes to out
    float32 [T, heads * e].  state float32 [slots, >= heads * d * e] (may be a column slice of the per-sequence
    state) is read before each sequence's first token and written after its last."""
    T = q.shape[0]
    d, e = int(key_dim), int(value_dim)
    for name, t, n in (("q", q, qk_heads * d), ("k", k, qk_heads * d), ("v", v, heads * e)):
        if t.dtype != torch.float32 or tuple(t.shape) != (T, n) or t.stride(1) != 1 or t.stride(0) != q.stride(0):
            raise KernelError(f"gated_scan: {name} must be float32 [T, {n}], a column slice of the buffer q lies in")
    if heads % qk_heads or not 0 < d <= MAX_KEY_WIDTH:
        raise KernelError(f"gated_scan: {heads} heads cannot share {qk_heads} key heads, or key width {d} is outside 1..{MAX_KEY_WIDTH}")
    if scalars.dtype != torch.float32 or tuple(scalars.shape) != (T, heads, 4) or not scalars.is_contiguous():
        raise KernelError("gated_scan: scalars must be float32 [T, heads, 4]")
    if state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1 or state.shape[1] < heads * d * e:
        raise KernelError("gated_scan: state must be float32 [slots, >= heads * d * e]")
    if out.dtype != torch.float32 or tuple(out.shape) != (T, heads * e) or out.stride(1) != 1:
        raise KernelError("gated_scan: out must be float32 [T, heads * e]")
    if skip is not None and (skip.dtype != torch.float32 or skip.shape[0] != heads):
        raise KernelError("gated_scan: skip must be float32 [heads]")
    if single_tokens and T != n_seqs:
        raise KernelError("gated_scan: single_tokens needs one token per sequence")
    need_contiguous(cu_seqlens=cu_seqlens, slots=slots, skip=skip)
    check(core().tq_gated_scan(int(bool(delta)), ptr(q), ptr(k), ptr(v), q.stride(0), ptr(scalars), ptr(skip),
                               heads // qk_heads, ptr(state), state.stride(0), ptr(cu_seqlens), ptr(slots), int(n_seqs),
                               T, int(single_tokens), ptr(out), out.stride(0), heads, d, e, stream()), "gated_scan")
    return out
