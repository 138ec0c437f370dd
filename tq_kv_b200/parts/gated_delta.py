"""A mixer with a matrix of memory per head, updated by the delta rule with one
decay and one write strength per head and token:

    q, k = unit(silu(conv(W_q h))), unit(silu(conv(W_k h)))     key_heads x key_dim; q also times query_scale
    v = silu(conv(W_v h))                                       heads x value_dim
    beta = sigmoid(W_b h),   g = exp(-exp(A_log) * softplus(W_a h + dt_bias))            per head
    S' = g S_{t-1};   u = beta (v - S'^T k);   S_t = S' + k u^T;   o_t = S_t^T q          (the read sees the write)
    out = W_o (rms_norm_per_head(o) * w * silu(W_g h))          w has value_dim entries, shared by the heads

conv is a short causal convolution over time per channel (no bias);
unit(x) = x / sqrt(sum(x^2) + unit_eps) per head; head h reads the q and k of
key head h // (heads / key_heads).  S starts at zero, is float32 and lives,
with the convolutions' last taps - 1 inputs, in the cache's per-sequence state
(csrc/short_conv.cu, csrc/linear_scan.cu).
"""
from __future__ import annotations

import torch

from .. import kernels
from ..cache import StateRequest
from ..config import ConfigError
from ..kernels.scan import MAX_CONV_TAPS, MAX_KEY_WIDTH
from .base import Mixer, Runtime, StepContext, WeightSpec, float32_vector
from .state_space import CONV_VECTOR


class GatedDeltaMixer(Mixer):
    graph_capturable = True             # slots and lengths are read on the device

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.heads, self.key_heads = int(p["heads"]), int(p["key_heads"])
        self.key_dim, self.value_dim, self.taps = int(p["key_dim"]), int(p["value_dim"]), int(p["taps"])
        self.eps, self.unit_eps = float(p["eps"]), float(p.get("unit_eps", 1e-6))
        self.query_scale = float(p.get("query_scale", 1.0))
        self.names = dict(p["names"])
        if self.heads % self.key_heads:
            raise ConfigError(f"{self.heads} heads cannot share {self.key_heads} key heads")
        if self.key_dim > MAX_KEY_WIDTH or not 1 <= self.taps <= MAX_CONV_TAPS:
            raise kernels.KernelError(f"gated delta rule: key width {self.key_dim} or {self.taps} taps exceed the kernels' limits")
        self.qk, self.vw = self.key_heads * self.key_dim, self.heads * self.value_dim
        self.conv_channels = 2 * self.qk + self.vw
        self.state_floats = self.heads * self.key_dim * self.value_dim
        self.w_in = self.conv_w = self.dt_bias = self.a_log = self.norm_w = self.w_o = None

    def _n(self, which: str) -> str:
        return self.prefix + self.names[which]

    def weight_specs(self):
        h, H = self.hidden, self.heads
        return [WeightSpec(self._n("q"), (self.qk, h), "matrix"), WeightSpec(self._n("k"), (self.qk, h), "matrix"),
                WeightSpec(self._n("v"), (self.vw, h), "matrix"),
                WeightSpec(self._n("q_conv"), (self.qk, self.taps), "conv"),
                WeightSpec(self._n("k_conv"), (self.qk, self.taps), "conv"),
                WeightSpec(self._n("v_conv"), (self.vw, self.taps), "conv"),
                WeightSpec(self._n("beta"), (H, h), "matrix"), WeightSpec(self._n("decay"), (H, h), "matrix"),
                WeightSpec(self._n("a_log"), (H,), "bias"), WeightSpec(self._n("dt_bias"), (H,), "bias"),
                WeightSpec(self._n("gate"), (self.vw, h), "matrix"),
                WeightSpec(self._n("norm"), (self.value_dim,), "norm_scale"),
                WeightSpec(self._n("out"), (h, self.vw), "matrix")]

    def bind(self, tensors, runtime: Runtime, shared=None):
        ws = [tensors[self._n(x)] for x in ("q", "k", "v", "decay", "beta", "gate")]
        if len({w.dtype for w in ws}) != 1:
            ws = [w.to(torch.float32) for w in ws]
        self.w_in = torch.cat(ws, dim=0).contiguous()          # q | k | v | decay logits | write logits | gate
        self.conv_w = torch.cat([float32_vector(tensors[self._n(x)]) for x in ("q_conv", "k_conv", "v_conv")],
                                dim=0).contiguous()
        self.dt_bias = float32_vector(tensors[self._n("dt_bias")])
        self.a_log = float32_vector(tensors[self._n("a_log")])
        self.norm_w = float32_vector(tensors[self._n("norm")]).repeat(self.heads).contiguous()
        self.w_o = tensors[self._n("out")].contiguous()

    def state_request(self):
        return StateRequest((self.state_floats + (self.taps - 1) * self.conv_channels,), torch.float32)

    def forward(self, x, ctx: StepContext, residual):
        b, dev = ctx.batch, residual.device
        act = ctx.runtime.act_dtype
        qk, vw, C, H = self.qk, self.vw, self.conv_channels, self.heads
        proj = kernels.linear(x, self.w_in, out_dtype=torch.float32)
        kernels.mark("qkv")
        T = proj.shape[0]
        single = b.single_tokens
        cv = torch.empty((T, C), dtype=torch.float32, device=dev)
        scal = torch.empty((T, H, 4), dtype=torch.float32, device=dev)
        kernels.short_conv(proj[:, :C], self.conv_w, None, cv, ctx.state[:, self.state_floats:],
                           tok_seq=b.tok_seq, cu_seqlens=b.cu_seqlens, slots=b.slots, n_seqs=b.n_seqs,
                           regions=[(0, qk, self.key_dim, True, self.query_scale), (qk, qk, self.key_dim, True, 1.0),
                                    (2 * qk, vw, min(vw, CONV_VECTOR), False, 1.0)],
                           silu=True, single_tokens=single, unit_eps=self.unit_eps, gate_raw=proj[:, C:C + H],
                           beta_raw=proj[:, C + H:C + 2 * H], a_log=self.a_log, dt_bias=self.dt_bias, scalars=scal)
        kernels.mark("conv")
        o = torch.empty((T, vw), dtype=torch.float32, device=dev)
        kernels.gated_scan(cv[:, :qk], cv[:, qk:2 * qk], cv[:, 2 * qk:], scal, ctx.state[:, :self.state_floats],
                           b.cu_seqlens, b.slots, o, n_seqs=b.n_seqs, heads=H, qk_heads=self.key_heads,
                           key_dim=self.key_dim, value_dim=self.value_dim, delta=True, single_tokens=single)
        kernels.mark("scan")
        y = torch.empty((T, vw), dtype=act, device=dev)
        kernels.group_rmsnorm(o, self.norm_w, self.eps, y, groups=H, gate=proj[:, C + 2 * H:], gate_mode=kernels.GATE_SILU)
        kernels.mark("norms")
        kernels.linear(y, self.w_o, out=residual, accumulate=True)
        kernels.mark("o")
