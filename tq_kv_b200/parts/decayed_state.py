"""A mixer with a matrix of memory per head that fades by a constant factor
per head (linear attention with decay):

    S_t = decay_head * S_{t-1} + k_t v_t^T,     o_t = S_t^T q_t

with q, k (heads x key_dim) and v (heads x value_dim) projections of the input
passed through an activation (silu, or none).  The heads of a token side by
side are RMS-normed together with a weight, multiplied by sigmoid(W_g x) and
projected.  S starts at zero, is float32 and lives in the cache's per-sequence
state.  The scan kernel is the one of the delta rule (csrc/linear_scan.cu).
"""
from __future__ import annotations

import torch

from .. import kernels
from ..cache import StateRequest
from ..config import ConfigError
from .base import Mixer, Runtime, StepContext, WeightSpec, float32_vector


class DecayedStateMixer(Mixer):
    takes_pending_norm = True           # x goes to kernels.linear only
    graph_capturable = True

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.heads, self.key_dim, self.value_dim = int(p["heads"]), int(p["key_dim"]), int(p["value_dim"])
        self.decay = [float(x) for x in p["decay"]]
        if len(self.decay) != self.heads:
            raise ConfigError(f"{len(self.decay)} decays for {self.heads} heads")
        self.activation = p.get("activation", "silu")
        if self.activation not in ("silu", None):
            raise ConfigError(f"decayed-state mixer: activation '{self.activation}' is not known (silu or none)")
        self.eps = float(p["eps"])
        self.names = dict(p["names"])
        self.qk, self.vw = self.heads * self.key_dim, self.heads * self.value_dim
        self.w_in = self.norm_w = self.w_o = self.decay_t = None

    def _n(self, which: str) -> str:
        return self.prefix + self.names[which]

    def weight_specs(self):
        h = self.hidden
        return [WeightSpec(self._n("q"), (self.qk, h), "matrix"), WeightSpec(self._n("k"), (self.qk, h), "matrix"),
                WeightSpec(self._n("v"), (self.vw, h), "matrix"), WeightSpec(self._n("gate"), (self.vw, h), "matrix"),
                WeightSpec(self._n("norm"), (self.vw,), "norm_scale"), WeightSpec(self._n("out"), (h, self.vw), "matrix")]

    def bind(self, tensors, runtime: Runtime, shared=None):
        ws = [tensors[self._n(x)] for x in ("q", "k", "v", "gate")]
        if len({w.dtype for w in ws}) != 1:
            ws = [w.to(torch.float32) for w in ws]
        self.w_in = torch.cat(ws, dim=0).contiguous()
        self.norm_w = float32_vector(tensors[self._n("norm")])
        self.w_o = tensors[self._n("out")].contiguous()
        self.decay_t = torch.tensor(self.decay, dtype=torch.float32, device=runtime.device)

    def state_request(self):
        return StateRequest((self.heads, self.key_dim, self.value_dim), torch.float32)

    def forward(self, x, ctx: StepContext, residual):
        b, dev = ctx.batch, residual.device
        act = ctx.runtime.act_dtype
        proj = kernels.linear(x, self.w_in, out_dtype=torch.float32)
        kernels.mark("qkv")
        T = proj.shape[0]
        o = torch.empty((T, self.vw), dtype=torch.float32, device=dev)
        kernels.linear_scan(proj, ctx.state, b.cu_seqlens, b.slots, o, n_seqs=b.n_seqs, heads=self.heads,
                            key_dim=self.key_dim, value_dim=self.value_dim, off_q=0, off_k=self.qk, off_v=2 * self.qk,
                            head_decay=self.decay_t, silu=self.activation == "silu", single_tokens=b.single_tokens)
        kernels.mark("scan")
        y = torch.empty((T, self.vw), dtype=act, device=dev)
        kernels.group_rmsnorm(o, self.norm_w, self.eps, y, groups=1, gate=proj[:, 2 * self.qk + self.vw:])
        kernels.mark("norms")
        kernels.linear(y, self.w_o, out=residual, accumulate=True)
        kernels.mark("o")
