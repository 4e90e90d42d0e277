"""LayerNorm with its eps as a parameter.

Formula as the reference computes it (src/kernels/layernorm.cu:32-49): mean,
biased variance of the centred values, (x-mean)*rsqrt(var+eps)*gamma+beta, all
in 32-bit; the reference kernel is fixed to 768 columns (:12), this one takes
any width.
"""
from __future__ import annotations

from .base import Norm, ParamSpec, register_part


class LayerNorm(Norm):
    supports_lazy = True

    def __init__(self, hidden_size: int, eps: float):
        self.hidden_size = int(hidden_size)
        self.eps = float(eps)

    def param_specs(self):
        return {"weight": ParamSpec((self.hidden_size,), "vector"),
                "bias": ParamSpec((self.hidden_size,), "vector")}

    def forward(self, x, ctx, rows=None, lazy=False):
        """``lazy``: the consumer is a product that can fuse the norm into its loads; it gets
        a NormedInput instead of a tensor (and may still ask for the tensor)."""
        if lazy:
            return self.rt.ops.NormedInput(x, self.weight, self.bias, self.eps, rows, ctx.ws, self.rt.act_dtype)
        n = x.shape[0] if rows is None else rows.shape[0]
        out = ctx.ws.buf("norm_out", n, self.hidden_size, self.rt.act_dtype)
        self.rt.ops.layernorm(x, self.weight, self.bias, self.eps, out, rows=rows)
        return out


register_part("norm", "layernorm", LayerNorm)


class RMSNorm(Norm):
    """y = x / sqrt(mean(x^2) + eps) * (w + 1) for weights stored around zero (``unit_offset``), or * w for
    plain weights; eps inside the root, all 32-bit.  ``forward_pair`` norms the same rows with two weight
    vectors (this norm's and ``other``'s) from one sum of squares: the two branches of a parallel block.  With
    ``lazy=True`` a product that can take the norm into its loads gets it unevaluated (few rows: decode steps)."""

    supports_lazy = True
    # A product that takes the norm into its loads norms its rows again in every CTA.  Measured in decode steps of 8
    # requests: at widths 768 and 1024 that is as fast as a norm kernel of its own or a little faster (one launch less
    # per product), at width 2048 it is 10 % slower (0.327 against 0.297 ms per step), so wider rows are normed first.
    LAZY_MAX_ROWS, LAZY_MAX_WIDTH = 16, 1024

    def __init__(self, hidden_size: int, eps: float, unit_offset: bool = False):
        self.hidden_size = int(hidden_size)
        self.eps = float(eps)
        self.unit_offset = bool(unit_offset)

    def lazy_pays(self, n_rows: int) -> bool:
        return n_rows <= self.LAZY_MAX_ROWS and self.hidden_size <= self.LAZY_MAX_WIDTH

    def param_specs(self):
        return {"weight": ParamSpec((self.hidden_size,), "vector")}

    def bind(self, params, rt) -> None:
        import torch
        super().bind(params, rt)
        if "weight" in params:       # what the fused products multiply and add: w + 1 (or w), and nothing
            self.gamma = (self.weight + 1.0).contiguous() if self.unit_offset else self.weight
            self.zero_beta = torch.zeros_like(self.weight)

    def forward(self, x, ctx, rows=None, lazy=False, name="norm_out"):
        if lazy and self.lazy_pays(x.shape[0] if rows is None else rows.shape[0]):
            return self.rt.ops.NormedInput(x, self.gamma, self.zero_beta, self.eps, rows, ctx.ws, self.rt.act_dtype,
                                           rms=True, buf=name)
        n = x.shape[0] if rows is None else rows.shape[0]
        out = ctx.ws.buf(name, n, self.hidden_size, self.rt.act_dtype)
        self.rt.ops.rmsnorm(x, self.weight, self.eps, out, rows=rows, unit_offset=self.unit_offset)
        return out

    def pairs_with(self, other) -> bool:
        return (isinstance(other, RMSNorm) and other.hidden_size == self.hidden_size and other.eps == self.eps
                and other.unit_offset == self.unit_offset)

    def forward_pair(self, other, x, ctx):
        n = x.shape[0]
        out1 = ctx.ws.buf("norm_out", n, self.hidden_size, self.rt.act_dtype)
        out2 = ctx.ws.buf("norm_out_b", n, self.hidden_size, self.rt.act_dtype)
        self.rt.ops.rmsnorm(x, self.weight, self.eps, out1, unit_offset=self.unit_offset, weight2=other.weight, out2=out2)
        return out1, out2


register_part("norm", "rmsnorm", RMSNorm)
