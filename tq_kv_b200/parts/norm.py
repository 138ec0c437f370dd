"""RMS norm.  Reference: src/models/turbo_generic.rs:41-51 — computed in
float32: x / sqrt(mean(x^2) + eps) * weight; no bias, no `1 + weight`.  A model that stores its norm weights as
the distance from one says so with `weight_offset` (1.0): the offset is added once, in float32, when the
weights are bound."""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from ..config import ConfigError
from .base import Norm, Runtime, WeightSpec, float32_vector


class RMSNorm(Norm):
    padded_rows_ok = True               # row by row

    def __init__(self, spec):
        super().__init__(spec)
        self.width = int(self.params["width"])
        self.eps = float(self.params["eps"])
        self.weight_name = self.params.get("weight_name") or self.prefix + "weight"
        self.weight_offset = float(self.params.get("weight_offset", 0.0))
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self):
        # (stored as the distance from one: random weights are then drawn around zero)
        return [WeightSpec(self.weight_name, (self.width,), "norm_offset" if self.weight_offset else "norm_scale")]

    def bind(self, tensors, runtime: Runtime, shared=None):
        self.weight = float32_vector(tensors[self.weight_name])
        if self.weight_offset != 0.0:
            self.weight = (self.weight + self.weight_offset).contiguous()

    def forward(self, x, out_dtype, rows=None):
        n = x.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n, self.width), dtype=out_dtype, device=x.device)
        return kernels.rmsnorm(x, self.weight, self.eps, out, rows)

    def pending(self, x, out_dtype):
        """The norm of all rows of x as a `kernels.PendingNorm`: a part that
        feeds it to `kernels.linear` lets the product fold the norm in where
        it can (else the norm runs then, as a kernel of its own)."""
        return kernels.PendingNorm(x, self.weight, self.eps, out_dtype)


class GroupRMSNorm(RMSNorm):
    """RMS norm in groups: the row is cut into `groups` equal consecutive
    parts, each divided by its own sqrt(mean(part^2) + eps); then the whole row
    times the weight.  One group is the plain norm."""
    def __init__(self, spec):
        super().__init__(spec)
        self.groups = int(self.params.get("groups", 1))
        if self.groups < 1 or self.width % self.groups:
            raise ConfigError(f"a norm over {self.width} values cannot be cut into {self.groups} equal groups")
        if self.groups > 1:
            self.pending = None             # the products fold in the plain norm only

    def forward(self, x, out_dtype, rows=None):
        n = x.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n, self.width), dtype=out_dtype, device=x.device)
        return kernels.group_rmsnorm(x, self.weight, self.eps, out, groups=self.groups, rows=rows)
