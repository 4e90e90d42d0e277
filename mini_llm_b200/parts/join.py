"""Joins: how a branch's result reaches the residual stream when that is more than a sum.

``NormScaleJoin``: x += rms_norm(y, w) * s, the branch's result normed once more (plain weights, eps inside the
root) and multiplied column by column by a learned scale before it is added; all 32-bit, one kernel.
"""
from __future__ import annotations

from .base import Join, ParamSpec, register_part


class NormScaleJoin(Join):
    def __init__(self, hidden_size: int, eps: float, scaled: bool = True):
        self.hidden_size = int(hidden_size)
        self.eps = float(eps)
        self.scaled = bool(scaled)
        self.scale = None

    def param_specs(self):
        p = {"weight": ParamSpec((self.hidden_size,), "vector")}
        if self.scaled:
            p["scale"] = ParamSpec((self.hidden_size,), "vector")
        return p

    def forward(self, y, x, ctx):
        self.rt.ops.norm_scale_add(y, self.weight, self.scale, x, self.eps)


register_part("join", "norm_scale", NormScaleJoin)
