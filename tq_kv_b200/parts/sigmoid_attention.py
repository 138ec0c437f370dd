"""Grouped-query attention whose weights are sigmoids, not a softmax.

With q (heads x key_dim), k (kv_heads x key_dim) and v (kv_heads x value_dim)
projected from the input (biases optional), the weight of key j for the query
at position i of head h is

    sigmoid(q_i . k_j * scale + table[bucket(i - j), h] + offset[h]),    j <= i,

and the weights are not normalised over the keys.  Options, all parameters:
  qk_norm "row"     q and k are each divided by the root mean square of their
                    whole row (all heads together) and multiplied by a weight
                    per entry, before the heads are split
  temp_coef, temp_every   q at position p is multiplied by
                    1 + temp_coef * ln(floor((p + 1) / temp_every) + 1)
  distance_bias     a learned table with B rows and a column per head, indexed
                    by the bucket of the distance n = i - j:  n itself below
                    B // 2, then min(B - 1, B//2 + floor(ln(n / (B//2)) /
                    ln(far / (B//2)) * (B - B//2)));  `scale` does not touch it
  head_offset       a learned constant per head added to every score
  head_gate         head h's result is multiplied by sigmoid(W_g x)_h
There is no rotation: positions enter through the bias and the temperature.

The table and the offset are folded at bind time into one float32 table per
head and distance (distances from `far` on share the last row), which the
kernels index with i - j.  Prompts from position 0 attend over the step's own
keys; everything else reads the paged cache (csrc/sigmoid_attention.cu).
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import kernels
from ..cache import KVRequest
from ..config import ConfigError
from ..kernels.sigmoid import split_scratch_floats
from .base import Mixer, Runtime, StepContext, WeightSpec, float32_vector


def distance_rows(rows: int, far: int, n_distances: int) -> torch.Tensor:
    """The table row for every distance 0 .. n_distances - 1 (int64): the distance itself below rows // 2, then
    min(rows - 1, rows // 2 + floor(ln(n / (rows // 2)) / ln(far / (rows // 2)) * (rows - rows // 2)))."""
    half = rows // 2
    out = []
    for n in range(n_distances):
        if n < half:
            out.append(n)
        elif half == 0 or far == half:                   # the formula divides by zero: everything beyond is the last row
            out.append(rows - 1 if n > half or half == 0 else half)
        else:
            b = half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half)))
            out.append(max(0, min(rows - 1, b)))
    return torch.tensor(out, dtype=torch.int64)


class SigmoidAttention(Mixer):
    takes_pending_norm = True           # x goes to kernels.linear only
    graph_capturable = True
    padded_rows_ok = True               # causal, and rows past a sequence's new length are not cached

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.heads, self.kv_heads = int(p["heads"]), int(p["kv_heads"])
        self.key_dim, self.value_dim = int(p["key_dim"]), int(p["value_dim"])
        if self.heads % self.kv_heads:
            raise ConfigError(f"{self.heads} heads cannot share {self.kv_heads} key/value heads")
        self.scale = float(p["scale"])
        self.qk_norm = p.get("qk_norm")
        if self.qk_norm not in (None, "row"):
            raise ConfigError(f"sigmoid attention: qk_norm '{self.qk_norm}' is not known (row or none)")
        self.eps = float(p.get("eps", 0.0))
        self.temp_coef = float(p.get("temp_coef", 0.0))
        self.temp_every = int(p.get("temp_every", 1))
        self.distance = p.get("distance_bias")          # {"rows": B or None, "far": D} or None
        self.head_offset = bool(p.get("head_offset", False))
        self.head_gate = bool(p.get("head_gate", False))
        self.qkv_bias = bool(p.get("qkv_bias", False))
        self.names = dict(p["names"])
        self.nq, self.nk, self.nv = self.heads * self.key_dim, self.kv_heads * self.key_dim, self.kv_heads * self.value_dim
        self.w_in = self.b_in = self.w_o = self.q_norm_w = self.k_norm_w = self.bias_table = None

    def _n(self, which: str) -> str:
        return self.prefix + self.names[which]

    def weight_specs(self):
        h = self.hidden
        specs = [WeightSpec(self._n("q"), (self.nq, h), "matrix"), WeightSpec(self._n("k"), (self.nk, h), "matrix"),
                 WeightSpec(self._n("v"), (self.nv, h), "matrix"),
                 WeightSpec(self._n("o"), (h, self.heads * self.value_dim), "matrix")]
        if self.qkv_bias:
            specs += [WeightSpec(self._n("q_bias"), (self.nq,), "bias"), WeightSpec(self._n("k_bias"), (self.nk,), "bias"),
                      WeightSpec(self._n("v_bias"), (self.nv,), "bias")]
        if self.qk_norm:
            specs += [WeightSpec(self._n("q_norm"), (self.nq,), "norm_scale"),
                      WeightSpec(self._n("k_norm"), (self.nk,), "norm_scale")]
        if self.distance is not None:
            rows = self.distance.get("rows")
            specs.append(WeightSpec(self._n("distance"), (-1 if rows is None else int(rows), self.heads), "bias"))
        if self.head_offset:
            specs.append(WeightSpec(self._n("offset"), (self.heads,), "bias"))
        if self.head_gate:
            specs.append(WeightSpec(self._n("gate"), (self.heads, h), "matrix"))
        return specs

    def bind(self, tensors, runtime: Runtime, shared=None):
        dev = runtime.device
        ws = [tensors[self._n(x)] for x in ("q", "k", "v")] + ([tensors[self._n("gate")]] if self.head_gate else [])
        if len({w.dtype for w in ws}) != 1:
            ws = [w.to(torch.float32) for w in ws]
        self.w_in = torch.cat(ws, dim=0).contiguous()          # q | k | v | gate rows: one product
        if self.qkv_bias:
            bias = torch.zeros(self.w_in.shape[0], dtype=torch.float32, device=dev)
            bias[:self.nq + self.nk + self.nv] = torch.cat(
                [float32_vector(tensors[self._n(x)]) for x in ("q_bias", "k_bias", "v_bias")])
            self.b_in = bias
        self.w_o = tensors[self._n("o")].contiguous()
        if self.qk_norm:
            self.q_norm_w = float32_vector(tensors[self._n("q_norm")])
            self.k_norm_w = float32_vector(tensors[self._n("k_norm")])
        table: Optional[torch.Tensor] = None
        if self.distance is not None:
            rel = float32_vector(tensors[self._n("distance")])                       # [B, heads]
            far = int(self.distance["far"])
            # from `far` on every distance has the last row (if the rows widen at all: far beyond the exact ones)
            n_dist = runtime.max_context if far <= rel.shape[0] // 2 else min(runtime.max_context, far + 1)
            n_dist = max(1, n_dist)
            rows = distance_rows(rel.shape[0], far, n_dist).to(dev)
            table = rel[rows].t().contiguous()                                       # [heads, n_dist]
        if self.head_offset:
            off = float32_vector(tensors[self._n("offset")]).reshape(self.heads, 1)
            table = off.contiguous() if table is None else (table + off).contiguous()
        self.bias_table = table

    def cache_request(self):
        return KVRequest(self.kv_heads, self.key_dim, None, self.value_dim)

    @staticmethod
    def _use_packed(start_pos, step_lens, owns_cache) -> bool:
        return owns_cache and all(s == 0 for s in start_pos) and any(n > 1 for n in step_lens)

    def forward(self, x, ctx: StepContext, residual):
        b, kv, dev = ctx.batch, ctx.kv, residual.device
        act = ctx.runtime.act_dtype
        proj = kernels.linear(x, self.w_in, bias=self.b_in, out_dtype=torch.float32)
        kernels.mark("qkv")
        T = proj.shape[0]
        owns = kv is not None and kv.writes
        packed = self._use_packed(b.host_start, b.host_lens, owns)
        q = torch.empty((T, self.nq), dtype=act, device=dev)
        k = torch.empty((T, self.nk), dtype=act, device=dev) if packed else None
        v = torch.empty((T, self.nv), dtype=act, device=dev) if packed else None
        kernels.rownorm_qkv_store(
            proj, q, n_heads=self.heads, n_kv_heads=self.kv_heads, key_dim=self.key_dim, value_dim=self.value_dim,
            tok_pos=b.tok_pos, tok_seq=b.tok_seq, new_lens=b.new_lens, q_weight=self.q_norm_w, k_weight=self.k_norm_w,
            eps=self.eps, temp_coef=self.temp_coef, temp_every=self.temp_every, k_out=k, v_out=v,
            k_pages=kv.k_pages if owns else None, v_pages=kv.v_pages if owns else None,
            block_table=kv.block_table if owns else None, table_width=kv.table_width if owns else 0,
            page_tokens=kv.page_tokens if kv is not None else 64)
        kernels.mark("rotary")
        out = torch.empty((T, self.heads * self.value_dim), dtype=act, device=dev)
        gate = proj[:, self.nq + self.nk + self.nv:] if self.head_gate else None
        common = dict(n_heads=self.heads, n_kv_heads=self.kv_heads, key_dim=self.key_dim, value_dim=self.value_dim,
                      scale=self.scale, tok_pos=b.tok_pos, tok_seq=b.tok_seq, cu_seqlens=b.cu_seqlens,
                      start_pos=b.start_pos, bias=self.bias_table, gate=gate)
        if packed:
            kernels.sigmoid_attention(q, out, k_packed=k, v_packed=v, **common)
        else:
            n_splits = kernels.plan_splits(T, self.kv_heads, b.max_new_len, ctx.runtime.sm_count)
            scratch = None
            if n_splits > 1:
                scratch = torch.empty(split_scratch_floats(T, self.heads, self.value_dim, n_splits),
                                      dtype=torch.float32, device=dev)
            kernels.sigmoid_attention(q, out, k_pages=kv.k_pages, v_pages=kv.v_pages, block_table=kv.block_table,
                                      table_width=kv.table_width, page_tokens=kv.page_tokens, n_splits=n_splits,
                                      scratch=scratch, **common)
        kernels.mark("attention")
        kernels.linear(out, self.w_o, out=residual, accumulate=True)
        kernels.mark("o")
