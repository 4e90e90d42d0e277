"""State-space mixers: a fixed-size state per request, carried from token to token.

``Mamba2Mixer`` (state-space duality).  With inner = heads * vdim, N state rows and G groups, W_in h is
[z: inner | x: inner | B: G*N | C: G*N | dt: heads].  x, B and C pass a causal convolution per channel (weights
[channels, taps], the last column the current token's, zeros before the start of a sequence, a bias) and silu.
dt <- softplus(dt + dt_bias).  Per head h (group floor(h / (heads / G))), with a state S [N, vdim] that starts at zero:

    S_t = exp(-exp(A_log_h) dt_t) S_(t-1) + dt_t B_t x_t^T        y_t = S_t^T C_t + D_h x_t

The joined y is multiplied by silu(z), RMS-normed in ``norm_groups`` equal parts (each by its own root mean square),
multiplied by a weight, and projected by W_o.  The request's state holds S of every head and the last taps - 1 inputs
of the convolution, both 32-bit, in one row of the cache manager's state arena; dt, the decay and the recurrence are
32-bit whatever the engine's dtype.
"""
from __future__ import annotations

from ..cache.manager import StateNeed
from .base import ParamSpec, register_part
from .projected import ProjectedMixer


class Mamba2Mixer(ProjectedMixer):
    in_names = ("in_proj",)
    out_name = "out_weight"

    def __init__(self, hidden_size: int, num_heads: int, v_head_dim: int, state_size: int, groups: int, conv_taps: int,
                 norm_groups: int, norm_eps: float):
        self.hidden_size, self.num_heads, self.v_head_dim = int(hidden_size), int(num_heads), int(v_head_dim)
        self.state_size, self.groups, self.conv_taps = int(state_size), int(groups), int(conv_taps)
        self.norm_groups, self.norm_eps = int(norm_groups), float(norm_eps)
        self.inner = self.num_heads * self.v_head_dim
        self.channels = self.inner + 2 * self.groups * self.state_size
        if self.num_heads % self.groups:
            raise ValueError(f"mamba2: {self.num_heads} heads in {self.groups} groups")
        if self.inner % self.norm_groups:
            raise ValueError(f"mamba2: {self.inner} columns in {self.norm_groups} norm groups")
        self.ssm_floats = self.num_heads * self.state_size * self.v_head_dim
        self.state_floats = self.ssm_floats + (self.conv_taps - 1) * self.channels

    def param_specs(self):
        Hm = self.num_heads
        return {"in_proj": ParamSpec((2 * self.inner + 2 * self.groups * self.state_size + Hm, self.hidden_size), "matrix"),
                "conv_weight": ParamSpec((self.channels, self.conv_taps), "vector"),
                "conv_bias": ParamSpec((self.channels,), "vector"),
                "dt_bias": ParamSpec((Hm,), "vector"),
                "A_log": ParamSpec((Hm,), "vector"),
                "D": ParamSpec((Hm,), "vector"),
                "norm_weight": ParamSpec((self.inner,), "vector"),
                "out_weight": ParamSpec((self.hidden_size, self.inner), "matrix")}

    def kernel_limits(self, dtype: str):
        from .. import ops
        out = []
        if self.state_size > ops.SSD_MAX_STATE_ROWS:
            out.append(f"mamba2: a state of {self.state_size} rows per head; the kernel takes {ops.SSD_MAX_STATE_ROWS}")
        if not (1 <= self.conv_taps <= ops.SSD_MAX_TAPS):
            out.append(f"mamba2: a convolution of {self.conv_taps} taps; the kernel takes 1 to {ops.SSD_MAX_TAPS}")
        return out

    def cache_need(self):
        return StateNeed((self.state_floats,), "float32")

    def core(self, proj, ctx, cache, out, out_scale: float = 1.0) -> None:
        import torch
        if out_scale != 1.0:
            raise NotImplementedError("mamba2 takes no branch factor")
        ops = self.rt.ops
        T = proj.shape[0]
        xbc = ctx.ws.buf("ssd_xbc", T, self.channels, torch.float32)
        ops.ssd_conv(proj, self.inner, self.conv_weight, self.conv_bias, cache.state, self.ssm_floats, ctx, xbc,
                     write_state=cache.write)
        y = ctx.ws.buf("ssd_y", T, self.inner, torch.float32)
        ops.ssd_scan(xbc, proj, self.inner + self.channels, self.dt_bias, self.A_log, self.D, cache.state, ctx, y,
                     heads=self.num_heads, vdim=self.v_head_dim, state_rows=self.state_size, groups=self.groups,
                     write_state=cache.write)
        ops.gated_group_norm(y, proj[:, :self.inner], self.norm_weight, out, self.norm_groups, self.norm_eps)


register_part("mixer", "mamba2", Mamba2Mixer)
