"""A mixer with a matrix of memory per head, updated by the generalised delta
rule.  Per head, with r, k, v of `dim` values each (projections of the input):

    w = exp(-exp(-1/2) * sigmoid(W_out tanh(W_in x) + b_w))     decay per key channel
    a = sigmoid(W_a x + b_a)                                    removal rate per key channel
    u = k / sqrt(|k|^2 + unit_eps)                              the unit key
    S_t = diag(w) S_{t-1} - (a * u)(u^T S_{t-1}) + k v^T        (both terms read the old state)
    o_t = S_t^T r

Each head's o is divided by its root mean square, the heads side by side are
multiplied by a weight and by sigmoid(W_g x), and projected.  S starts at
zero, is float32 and lives in the cache's per-sequence state, so a prompt, a
portion of a prompt and a decoded token run the same kernels.

All projections of x are one product (read | key | value | gate | removal |
decay-in rows of one weight, float32 result); everything that enters the
recurrence is made from that result in float32 inside the scan kernel
(csrc/linear_scan.cu).
"""
from __future__ import annotations

import torch

from .. import kernels
from ..cache import StateRequest
from ..kernels.scan import MAX_KEY_WIDTH
from .base import Mixer, Runtime, StepContext, WeightSpec, float32_vector

# below this inner width the decay's second product runs on the float32 kernels (the tensor-core ones want
# whole tiles of K)
_MIN_TC_RANK = 64


class DeltaRuleMixer(Mixer):
    takes_pending_norm = True           # x goes to kernels.linear only
    graph_capturable = True             # slots and lengths are read on the device

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.heads, self.dim = int(p["heads"]), int(p["dim"])
        self.rank = p.get("rank")                      # None: the checkpoint's shapes say
        self.eps = float(p["eps"])
        self.unit_eps = float(p.get("unit_eps", 1e-6))
        self.names = dict(p["names"])
        self.inner = self.heads * self.dim
        if self.dim > MAX_KEY_WIDTH:
            raise kernels.KernelError(f"delta rule: head width {self.dim} exceeds the scan kernel's limit")
        self.w_in = self.b_in = self.w_decay = self.b_decay = self.norm_w = self.w_o = None

    def _n(self, which: str) -> str:
        return self.prefix + self.names[which]

    def weight_specs(self):
        n, h, r = self.inner, self.hidden, -1 if self.rank is None else int(self.rank)
        return [WeightSpec(self._n(x), (n, h), "matrix") for x in ("read", "key", "value", "gate", "remove")] + [
            WeightSpec(self._n("remove_bias"), (n,), "bias"),
            WeightSpec(self._n("decay_in"), (r, h), "matrix"),
            WeightSpec(self._n("decay_out"), (n, r), "matrix"),
            WeightSpec(self._n("decay_bias"), (n,), "bias"),
            WeightSpec(self._n("norm"), (n,), "norm_scale"),
            WeightSpec(self._n("out"), (h, n), "matrix"),
        ]

    def bind(self, tensors, runtime: Runtime, shared=None):
        ws = [tensors[self._n(x)] for x in ("read", "key", "value", "gate", "remove", "decay_in")]
        if len({w.dtype for w in ws}) != 1:
            ws = [w.to(torch.float32) for w in ws]
        self.w_in = torch.cat(ws, dim=0).contiguous()          # one product for everything that reads x
        self.rank = int(ws[-1].shape[0])
        n = self.inner
        bias = torch.zeros(self.w_in.shape[0], dtype=torch.float32, device=self.w_in.device)
        bias[4 * n:5 * n] = float32_vector(tensors[self._n("remove_bias")])
        self.b_in = bias
        w2 = tensors[self._n("decay_out")]
        if tuple(w2.shape) != (n, self.rank):
            raise kernels.KernelError(f"delta rule: {self._n('decay_out')} has shape {tuple(w2.shape)}, "
                                      f"expected {(n, self.rank)}")
        self.decay_in_float32 = self.rank < _MIN_TC_RANK or self.rank % 8 != 0
        self.w_decay = (w2.to(torch.float32) if self.decay_in_float32 else w2).contiguous()
        self.b_decay = float32_vector(tensors[self._n("decay_bias")])
        self.norm_w = float32_vector(tensors[self._n("norm")])
        self.w_o = tensors[self._n("out")].contiguous()

    def state_request(self):
        return StateRequest((self.heads, self.dim, self.dim), torch.float32)

    def forward(self, x, ctx: StepContext, residual):
        b, n, dev = ctx.batch, self.inner, residual.device
        act = ctx.runtime.act_dtype
        proj = kernels.linear(x, self.w_in, bias=self.b_in, out_dtype=torch.float32)
        kernels.mark("qkv")
        T = proj.shape[0]
        low = torch.empty((T, self.rank), dtype=torch.float32 if self.decay_in_float32 else act, device=dev)
        kernels.tanh_rows(proj[:, 5 * n:], low)
        decay_logit = kernels.linear(low, self.w_decay, bias=self.b_decay, out_dtype=torch.float32)
        kernels.mark("decay")
        o = torch.empty((T, n), dtype=torch.float32, device=dev)
        kernels.linear_scan(proj, ctx.state, b.cu_seqlens, b.slots, o, n_seqs=b.n_seqs, heads=self.heads,
                            key_dim=self.dim, value_dim=self.dim, off_q=0, off_k=n, off_v=2 * n, off_a=4 * n,
                            decay_logit=decay_logit, unit_eps=self.unit_eps, single_tokens=b.single_tokens)
        kernels.mark("scan")
        y = torch.empty((T, n), dtype=act, device=dev)
        kernels.group_rmsnorm(o, self.norm_w, self.eps, y, groups=self.heads, gate=proj[:, 3 * n:4 * n])
        kernels.mark("norms")
        kernels.linear(y, self.w_o, out=residual, accumulate=True)
        kernels.mark("o")
