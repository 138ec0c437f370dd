"""Python entry point of the matrix-state recurrences (csrc/linear_scan.cu)."""
from __future__ import annotations

from typing import Optional

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
