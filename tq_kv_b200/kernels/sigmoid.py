"""Python entry points of the attention with sigmoid weights (csrc/sigmoid_attention.cu)."""
from __future__ import annotations

from typing import Optional

import torch

from ._lib import KernelError, check, core, dtype_code, need_contiguous, ptr, stream, tc_status_word

MAX_WIDTH = 256
NOT_SUPPORTED = 801      # cudaErrorNotSupported: the tensor-core kernel declines the shape
USE_TC_ATTENTION = True  # prompts in bfloat16 with keys and values 64 or 128 wide: the tcgen05 kernel


def rownorm_qkv_store(x: torch.Tensor, q_out: torch.Tensor, *, n_heads: int, n_kv_heads: int, key_dim: int,
                      value_dim: int, tok_pos, tok_seq, new_lens, q_weight: Optional[torch.Tensor] = None,
                      k_weight: Optional[torch.Tensor] = None, eps: float = 0.0, temp_coef: float = 0.0,
                      temp_every: int = 1, k_out=None, v_out=None, k_pages=None, v_pages=None, block_table=None,
                      table_width: int = 0, page_tokens: int = 64):
    """x float32 [T, >= nh*dk + nkv*dk + nkv*dv] holds q | k | v rows (biases already added).  q and k are each
    divided by the root mean square of their whole row and multiplied by q_weight / k_weight (float32, one
    entry per column; None: the row passes unchanged); q is then multiplied by
    1 + temp_coef * ln((pos + 1) // temp_every + 1).  q goes to q_out [T, nh*dk]; k and v go to k_out / v_out
    (if given) and into the paged cache (if given)."""
    T = x.shape[0]
    nq, nk, nv = n_heads * key_dim, n_kv_heads * key_dim, n_kv_heads * value_dim
    if x.dtype != torch.float32 or x.stride(1) != 1 or x.shape[1] < nq + nk + nv:
        raise KernelError("rownorm_qkv_store: x must be float32 [T, >= q + k + v columns]")
    if tuple(q_out.shape) != (T, nq):
        raise KernelError("rownorm_qkv_store: q_out must be [T, n_heads * key_dim]")
    for name, t, n in (("k_out", k_out, nk), ("v_out", v_out, nv)):
        if t is not None and (tuple(t.shape) != (T, n) or t.dtype != q_out.dtype):
            raise KernelError(f"rownorm_qkv_store: {name} must be [T, {n}] of q_out's dtype")
    for name, t, n in (("q_weight", q_weight, nq), ("k_weight", k_weight, nk)):
        if t is not None and (t.dtype != torch.float32 or t.shape[0] != n):
            raise KernelError(f"rownorm_qkv_store: {name} must be float32 [{n}]")
    if k_pages is not None:
        if (v_pages is None or block_table is None or k_pages.dtype != q_out.dtype or v_pages.dtype != q_out.dtype
                or tuple(k_pages.shape[1:]) != (n_kv_heads, page_tokens, key_dim)
                or tuple(v_pages.shape[1:]) != (n_kv_heads, page_tokens, value_dim)):
            raise KernelError("rownorm_qkv_store: cache pages do not fit the heads")
    if temp_every < 1:
        raise KernelError("rownorm_qkv_store: temp_every must be at least 1")
    need_contiguous(q_out=q_out, k_out=k_out, v_out=v_out, k_pages=k_pages, v_pages=v_pages, q_weight=q_weight,
                    k_weight=k_weight)
    check(core().tq_rownorm_qkv_store(
        ptr(x), x.stride(0), ptr(q_weight), ptr(k_weight), float(eps), float(temp_coef), int(temp_every), ptr(tok_pos),
        ptr(tok_seq), ptr(new_lens), ptr(block_table), table_width, page_tokens, ptr(q_out), ptr(k_out), ptr(v_out),
        ptr(k_pages), ptr(v_pages), dtype_code(q_out), T, n_heads, n_kv_heads, key_dim, value_dim, stream()),
        "rownorm_qkv_store")


def split_scratch_floats(n_tokens: int, n_heads: int, value_dim: int, n_splits: int) -> int:
    return n_tokens * n_heads * n_splits * value_dim if n_splits > 1 else 0


def sigmoid_attention(q: torch.Tensor, out: torch.Tensor, *, n_heads: int, n_kv_heads: int, key_dim: int,
                      value_dim: int, scale: float, tok_pos, tok_seq, cu_seqlens, start_pos,
                      bias: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                      k_packed=None, v_packed=None, k_pages=None, v_pages=None, block_table=None,
                      table_width: int = 0, page_tokens: int = 64, n_splits: int = 1,
                      scratch: Optional[torch.Tensor] = None):
    """out[t, h] = sigmoid(gate[t, h]) * sum over keys j <= pos(t) of
    sigmoid(q[t, h] . k_j * scale + bias[h, min(pos(t) - j, n_dist - 1)]) * v_j.
    q [T, nh*dk], out [T, nh*dv]; bias float32 [nh, n_dist] or None; gate float32 [T, nh] (may be a column slice)
    or None.  Keys and values come from the step's packed rows (every sequence then starts at position 0) or
    from the paged cache."""
    T = q.shape[0]
    if tuple(q.shape) != (T, n_heads * key_dim) or tuple(out.shape) != (T, n_heads * value_dim) or out.dtype != q.dtype:
        raise KernelError("sigmoid_attention: q must be [T, nh*dk] and out [T, nh*dv] of one dtype")
    if n_kv_heads <= 0 or n_heads % n_kv_heads:
        raise KernelError(f"sigmoid_attention: {n_heads} heads cannot share {n_kv_heads} key/value heads")
    if not (0 < key_dim <= MAX_WIDTH and 0 < value_dim <= MAX_WIDTH):
        raise KernelError(f"sigmoid_attention: widths {key_dim}, {value_dim} must be within 1..{MAX_WIDTH}")
    packed = k_packed is not None
    if packed:
        if (v_packed is None or k_packed.dtype != q.dtype or tuple(k_packed.shape) != (T, n_kv_heads * key_dim)
                or tuple(v_packed.shape) != (T, n_kv_heads * value_dim)):
            raise KernelError("sigmoid_attention: packed keys/values must be [T, nkv*dk] / [T, nkv*dv] of q's dtype")
    else:
        if k_pages is None or v_pages is None or block_table is None or k_pages.dtype != q.dtype:
            raise KernelError("sigmoid_attention: no key/value source of q's dtype was given")
        if (tuple(k_pages.shape[1:]) != (n_kv_heads, page_tokens, key_dim)
                or tuple(v_pages.shape[1:]) != (n_kv_heads, page_tokens, value_dim)):
            raise KernelError(f"sigmoid_attention: cache pages have shapes {tuple(k_pages.shape)}, {tuple(v_pages.shape)}")
    n_dist = 0
    if bias is not None:
        if bias.dtype != torch.float32 or bias.dim() != 2 or bias.shape[0] != n_heads:
            raise KernelError("sigmoid_attention: bias must be float32 [n_heads, distances]")
        n_dist = bias.shape[1]
    ldg = 0
    if gate is not None:
        if gate.dtype != torch.float32 or tuple(gate.shape) != (T, n_heads) or gate.stride(1) != 1:
            raise KernelError("sigmoid_attention: gate must be float32 [T, n_heads]")
        ldg = gate.stride(0)
    part = None
    if n_splits > 1:
        need = split_scratch_floats(T, n_heads, value_dim, n_splits)
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need:
            raise KernelError(f"sigmoid_attention: {n_splits} splits need {need} float32 of scratch")
        part = scratch
    need_contiguous(q=q, out=out, k_packed=k_packed, v_packed=v_packed, k_pages=k_pages, v_pages=v_pages,
                    block_table=block_table, bias=bias)
    n_seqs = cu_seqlens.shape[0] - 1
    if (USE_TC_ATTENTION and q.dtype == torch.bfloat16 and T > n_seqs and key_dim == value_dim
            and key_dim in (64, 128)):
        # prompts on the tcgen05 tensor cores: the softmax kernel's pipeline with sigmoid weights
        # (csrc/flash_prefill_tc.cu)
        st = core().tq_sigmoid_prefill_tc(
            ptr(q), ptr(k_packed), ptr(v_packed), ptr(k_pages), ptr(v_pages),
            0 if k_pages is None else k_pages.shape[0], ptr(block_table), table_width, page_tokens, ptr(cu_seqlens),
            ptr(start_pos), n_seqs, T, float(scale), ptr(bias), n_dist, ptr(gate), ldg, ptr(out), n_heads, n_kv_heads,
            key_dim, ptr(tc_status_word(q.device)), stream())
        if st != NOT_SUPPORTED:
            check(st, "sigmoid_prefill_tc")
            return out
    if USE_TC_ATTENTION and not packed and q.dtype == torch.bfloat16 and key_dim == value_dim:
        # the cache streamed once for all heads of a group (csrc/flash_decode.cu with sigmoid weights)
        st = core().tq_sigmoid_flash_decode(
            ptr(q), ptr(k_pages), ptr(v_pages), ptr(block_table), table_width, page_tokens, ptr(tok_pos), ptr(tok_seq),
            float(scale), ptr(bias), n_dist, ptr(gate), ldg, ptr(out), ptr(part), T, n_heads, n_kv_heads, key_dim,
            n_splits, stream())
        if st != NOT_SUPPORTED:
            check(st, "sigmoid_flash_decode")
            if n_splits > 1:
                check(core().tq_sigmoid_attention_sum(ptr(part), ptr(gate), ldg, ptr(out), dtype_code(out), T, n_heads,
                                                      value_dim, n_splits, stream()), "sigmoid_attention_sum")
            return out
    check(core().tq_sigmoid_attention(
        ptr(q), dtype_code(q), ptr(k_packed), ptr(v_packed), ptr(k_pages), ptr(v_pages), ptr(block_table), table_width,
        page_tokens, ptr(tok_pos), ptr(tok_seq), ptr(cu_seqlens), ptr(start_pos), float(scale), ptr(bias), n_dist,
        ptr(gate), ldg, ptr(out), ptr(part), T, n_heads, n_kv_heads, key_dim, value_dim, n_splits, stream()),
        "sigmoid_attention", 2 if n_splits > 1 else 1)
    return out
