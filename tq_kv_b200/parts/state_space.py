"""A mixer with a matrix of memory per head that fades by a decay computed per
token (selective state space, in its form with one scalar decay per head):

    [z | x B C | dt] = W_in h                      z, x: heads x value_dim; B, C: groups x state; dt: heads
    x B C <- silu(causal_conv(x B C) + bias)       a short convolution over time per channel
    dt = softplus(dt + dt_bias),   g = exp(-exp(A_log) * dt)            per head
    S_t = g S_{t-1} + dt * B_t x_t^T   (state x value_dim),   y_t = S_t^T C_t + D_head * x_t
    out = W_o (rms_norm_in_groups(y * silu(z)) * w)                     the gate comes before the norm

Head h reads the B and C of group h // (heads / groups).  S starts at zero, is
float32 and lives, with the convolution's last taps - 1 inputs, in the cache's
per-sequence state: a prompt, a portion of a prompt and a decoded token run
the same kernels (csrc/short_conv.cu, csrc/linear_scan.cu).
"""
from __future__ import annotations

import torch

from .. import kernels
from ..cache import StateRequest
from ..config import ConfigError
from ..kernels.scan import MAX_CONV_TAPS, MAX_KEY_WIDTH
from .base import Mixer, Runtime, StepContext, WeightSpec, float32_vector

CONV_VECTOR = 128          # channels a warp of the convolution kernel takes where no vector is normed


class StateSpaceMixer(Mixer):
    graph_capturable = True             # slots and lengths are read on the device

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.heads, self.value_dim, self.n_state = int(p["heads"]), int(p["value_dim"]), int(p["state"])
        self.groups, self.norm_groups, self.taps = int(p["groups"]), int(p["norm_groups"]), int(p["taps"])
        self.eps = float(p["eps"])
        self.names = dict(p["names"])
        self.inner = self.heads * self.value_dim
        self.bc = self.groups * self.n_state
        self.conv_channels = self.inner + 2 * self.bc
        if self.heads % self.groups or self.inner % self.norm_groups:
            raise ConfigError("state-space mixer: heads must divide into groups, the inner width into norm groups")
        if self.n_state > MAX_KEY_WIDTH or not 1 <= self.taps <= MAX_CONV_TAPS:
            raise kernels.KernelError(f"state-space mixer: state {self.n_state} or {self.taps} taps exceed the kernels' limits")
        self.state_floats = self.heads * self.n_state * self.value_dim
        self.w_in = self.conv_w = self.conv_b = self.dt_bias = self.a_log = self.skip = self.norm_w = self.w_o = None

    def _n(self, which: str) -> str:
        return self.prefix + self.names[which]

    def weight_specs(self):
        h, c = self.hidden, self.conv_channels
        return [WeightSpec(self._n("in"), (2 * self.inner + 2 * self.bc + self.heads, h), "matrix"),
                WeightSpec(self._n("conv"), (c, self.taps), "conv"),
                WeightSpec(self._n("conv_bias"), (c,), "bias"),
                WeightSpec(self._n("dt_bias"), (self.heads,), "bias"),
                WeightSpec(self._n("a_log"), (self.heads,), "bias"),
                WeightSpec(self._n("skip"), (self.heads,), "norm_scale"),
                WeightSpec(self._n("norm"), (self.inner,), "norm_scale"),
                WeightSpec(self._n("out"), (h, self.inner), "matrix")]

    def bind(self, tensors, runtime: Runtime, shared=None):
        self.w_in = tensors[self._n("in")].contiguous()
        self.conv_w = float32_vector(tensors[self._n("conv")])
        self.conv_b = float32_vector(tensors[self._n("conv_bias")])
        self.dt_bias = float32_vector(tensors[self._n("dt_bias")])
        self.a_log = float32_vector(tensors[self._n("a_log")])
        self.skip = float32_vector(tensors[self._n("skip")])
        self.norm_w = float32_vector(tensors[self._n("norm")])
        self.w_o = tensors[self._n("out")].contiguous()

    def state_request(self):
        return StateRequest((self.state_floats + (self.taps - 1) * self.conv_channels,), torch.float32)

    def forward(self, x, ctx: StepContext, residual):
        b, dev = ctx.batch, residual.device
        act = ctx.runtime.act_dtype
        inner, bc, C, H = self.inner, self.bc, self.conv_channels, self.heads
        proj = kernels.linear(x, self.w_in, out_dtype=torch.float32)
        kernels.mark("qkv")
        T = proj.shape[0]
        single = b.single_tokens
        cv = torch.empty((T, C), dtype=torch.float32, device=dev)
        scal = torch.empty((T, H, 4), dtype=torch.float32, device=dev)
        kernels.short_conv(proj[:, inner:inner + C], self.conv_w, self.conv_b, cv, ctx.state[:, self.state_floats:],
                           tok_seq=b.tok_seq, cu_seqlens=b.cu_seqlens, slots=b.slots, n_seqs=b.n_seqs,
                           regions=[(0, C, min(C, CONV_VECTOR), False, 1.0)], silu=True, single_tokens=single,
                           gate_raw=proj[:, inner + C:], a_log=self.a_log, dt_bias=self.dt_bias, scalars=scal)
        kernels.mark("conv")
        o = torch.empty((T, inner), dtype=torch.float32, device=dev)
        kernels.gated_scan(cv[:, inner + bc:], cv[:, inner:inner + bc], cv[:, :inner], scal,
                           ctx.state[:, :self.state_floats], b.cu_seqlens, b.slots, o, n_seqs=b.n_seqs, heads=H,
                           qk_heads=self.groups, key_dim=self.n_state, value_dim=self.value_dim, delta=False,
                           skip=self.skip, single_tokens=single)
        kernels.mark("scan")
        y = torch.empty((T, inner), dtype=act, device=dev)
        kernels.group_rmsnorm(o, self.norm_w, self.eps, y, groups=self.norm_groups, gate=proj[:, :inner],
                              gate_mode=kernels.GATE_SILU_FIRST)
        kernels.mark("norms")
        kernels.linear(y, self.w_o, out=residual, accumulate=True)
        kernels.mark("o")
