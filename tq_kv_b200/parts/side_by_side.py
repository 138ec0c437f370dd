"""Several mixers side by side on the same input.  Each branch's result is
RMS-normed over the model width with a weight of its own; the block's
residual stream gets `scale` times their sum (0.5 for the mean of two).

A branch is any registered mixer; what it asks of the cache is passed on: at
most one branch may ask for keys and values and at most one for per-sequence
state (a schedule entry owns one cache group and one state tensor).
"""
from __future__ import annotations

import torch

from .. import kernels
from ..config import ConfigError
from .base import Mixer, Runtime, StepContext, WeightSpec, float32_vector
from .registry import make_part


class SideBySideMixer(Mixer):
    takes_pending_norm = True           # (run once here: the branches share its result)
    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.width = int(p["width"])
        self.eps = float(p["eps"])
        self.scale = float(p.get("scale", 1.0))
        self.branches = [make_part(b["part"]) for b in p["branches"]]
        self.norm_names = [b["out_norm"] for b in p["branches"]]
        if not 1 <= len(self.branches) <= 4:
            raise ConfigError("a side-by-side mixer has one to four branches")
        if sum(b.cache_request() is not None for b in self.branches) > 1 \
                or sum(b.state_request() is not None for b in self.branches) > 1:
            raise ConfigError("a side-by-side mixer can hold one branch with keys and values and one with state")
        self.norm_w: list = []

    @property
    def graph_capturable(self):
        return all(getattr(b, "graph_capturable", True) for b in self.branches)

    @property
    def padded_rows_ok(self):
        return all(getattr(b, "padded_rows_ok", False) for b in self.branches)

    def weight_specs(self):
        specs = [ws for b in self.branches for ws in b.weight_specs()]
        return specs + [WeightSpec(n, (self.width,), "norm_scale") for n in self.norm_names]

    def ignored_weights(self):
        return [n for b in self.branches for n in b.ignored_weights()]

    def bind(self, tensors, runtime: Runtime, shared=None):
        for b in self.branches:
            b.bind(tensors, runtime, shared)
        self.norm_w = [float32_vector(tensors[n]) for n in self.norm_names]

    def cache_request(self):
        for b in self.branches:
            r = b.cache_request()
            if r is not None:
                return r
        return None

    def state_request(self):
        for b in self.branches:
            r = b.state_request()
            if r is not None:
                return r
        return None

    def check_step(self, start_pos, step_lens, owns_cache):
        for b in self.branches:
            b.check_step(start_pos, step_lens, owns_cache)

    def forward(self, x, ctx: StepContext, residual):
        if isinstance(x, kernels.PendingNorm):
            x = x.materialize()
        outs = []
        for b in self.branches:
            y = torch.zeros_like(residual)          # a branch adds its result into what it is given
            b.forward(x, ctx, y)
            outs.append(y)
        kernels.add_normed(residual, list(zip(outs, self.norm_w)), self.eps, self.scale)
        kernels.mark("norms")
