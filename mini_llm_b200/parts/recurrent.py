"""Recurrent mixers: a fixed-size state per request instead of a growing cache.

``GatedLinearRecurrence`` is linear attention in which one gate decides both
what is forgotten and what is written.  Per head, with q_t = silu(W_q h_t),
v_t = W_v h_t and the forget gate f_t = l + (1 - l) * sigmoid(W_f h_t + b)
(l a learned lower bound per channel, kept as given):

    S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T        S in R^(dim x vdim), S_(-1) = 0
    o_t = S_t^T q_t

(there is no key: 1 - f_t takes its place, and no further scale).  Each head's
o_t is RMS-normed over its vdim channels with a plain weight shared by the
heads, the heads are joined and projected by W_o.  The state, the gate and its
complement, the update, o_t and the norm are 32-bit on both paths; the state
lives in the request's slot of the cache manager's state arena, zero at
admission, and is carried from step to step.
"""
from __future__ import annotations

from ..cache.manager import StateNeed
from .base import ParamSpec, register_part
from .projected import ProjectedMixer

# what csrc/gated_recurrence.cu takes: a head's state column is kept in registers, 64 rows per thread
_ROWS_PER_THREAD = 64
_MAX_THREADS = 512


class GatedLinearRecurrence(ProjectedMixer):
    in_names = ("q_weight", "f_weight", "v_weight")
    out_name = "out_weight"

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, v_head_dim: int, norm_eps: float):
        self.hidden_size, self.num_heads = int(hidden_size), int(num_heads)
        self.head_dim, self.v_head_dim = int(head_dim), int(v_head_dim)
        self.norm_eps = float(norm_eps)
        self.k_size = self.num_heads * self.head_dim
        self.v_size = self.num_heads * self.v_head_dim

    def param_specs(self):
        return {"q_weight": ParamSpec((self.k_size, self.hidden_size), "matrix"),
                "f_weight": ParamSpec((self.k_size, self.hidden_size), "matrix"),
                "f_bias": ParamSpec((self.k_size,), "vector"),
                "lower": ParamSpec((self.k_size,), "vector"),
                "v_weight": ParamSpec((self.v_size, self.hidden_size), "matrix"),
                "norm_weight": ParamSpec((self.v_head_dim,), "vector"),
                "out_weight": ParamSpec((self.hidden_size, self.v_size), "matrix")}

    def kernel_limits(self, dtype: str):
        groups = -(-self.head_dim // _ROWS_PER_THREAD)
        threads = groups * (-(-self.v_head_dim // 32) * 32)
        if threads > _MAX_THREADS:
            return [f"gated linear recurrence: a state of {self.head_dim} x {self.v_head_dim} per head needs {threads} "
                    f"threads of one CTA; the kernel has {_MAX_THREADS}"]
        return []

    def cache_need(self):
        return StateNeed((self.num_heads, self.head_dim, self.v_head_dim), "float32")

    def core(self, proj, ctx, cache, out, out_scale: float = 1.0) -> None:
        K = self.k_size
        self.rt.ops.gated_recurrence(proj[:, :K], proj[:, K:2 * K], proj[:, 2 * K:], self.f_bias, self.lower,
                                     self.norm_weight, self.norm_eps, cache.state, ctx, out, heads=self.num_heads,
                                     out_scale=out_scale, write_state=cache.write)


register_part("mixer", "gated_linear_recurrence", GatedLinearRecurrence)
