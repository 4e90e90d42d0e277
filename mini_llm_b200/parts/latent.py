"""Attention over a compressed (latent) key/value cache.

Per token the layer keeps one row for all heads: the latent c = rms_norm(W_dkv h [:R]) (plain weight) and one
rotated key part k_r = rot(W_dkv h [R:]) of dr columns.  A head's key is [W_uk c | k_r], its value W_uv c, its query
[q_n | rot(q_r)] from W_q h, the score (q_n . W_uk c + q_r . k_r) * scale, causal, ordinary softmax.  The joined
heads are multiplied by sigmoid(W_g h) and projected by W_o.

The up-projections are never applied to cached tokens: with qa = W_uk^T q_n the score is (qa . c + q_r . k_r) * scale
and the head's output W_uv (sum_j p_j c_j), so attention runs over the cache rows as they are (one key/value head
whose value is the first R columns of its key) and W_uk, W_uv are two small per-head products on the step's own
tokens, before and after.  A layer with ``own_kv=False`` has no W_dkv: the schedule gives it another layer's cache
(``ScheduleEntry.cache_of``), whose rows it reads with its own W_uk, W_uv and queries.

Rotation: ``parts.rotary.rotary_table`` (YaRN scaling optional) on the first ``rot_dims`` of the dr columns.
32-bit: the latent's norm, angles, cos/sin, the absorbed query, scores, softmax, the weighted sum.
"""
from __future__ import annotations

from typing import Optional

from ..cache.manager import PagedNeed
from .base import ParamSpec, register_part
from .projected import ProjectedMixer
from .rotary import rotary_table


class LatentAttention(ProjectedMixer):
    out_name = "out_weight"

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, rot_dim: int, v_head_dim: int, kv_rank: int,
                 scale: float, norm_eps: float, rot_dims: Optional[int] = None, rot_base: float = 10000.0,
                 rot_scaling: Optional[dict] = None, own_kv: bool = True, gated: bool = True):
        self.hidden_size, self.num_heads = int(hidden_size), int(num_heads)
        self.head_dim, self.rot_dim, self.v_head_dim, self.kv_rank = int(head_dim), int(rot_dim), int(v_head_dim), int(kv_rank)
        self.scale, self.norm_eps = float(scale), float(norm_eps)
        self.rot_dims = self.rot_dim if rot_dims is None else int(rot_dims)
        self.rot_base, self.rot_scaling = float(rot_base), rot_scaling
        self.own_kv, self.gated = bool(own_kv), bool(gated)
        if self.rot_dims > self.rot_dim or self.rot_dims % 2:
            raise ValueError(f"latent attention: {self.rot_dims} rotated dimensions of {self.rot_dim}")
        self.q_size = self.num_heads * (self.head_dim + self.rot_dim)
        self.o_size = self.num_heads * self.v_head_dim
        self.key_dim = self.kv_rank + self.rot_dim
        self.row = -(-self.key_dim // 8) * 8            # a cache row: padded to 16-byte pieces, the padding zero
        self.in_names = tuple(n for n, on in (("q_weight", True), ("dkv_weight", self.own_kv), ("g_weight", self.gated)) if on)
        self.dkv_norm = None

    def param_specs(self):
        D, H, R = self.hidden_size, self.num_heads, self.kv_rank
        p = {"q_weight": ParamSpec((self.q_size, D), "matrix"),
             "uk_weight": ParamSpec((H * self.head_dim, R), "matrix"),
             "uv_weight": ParamSpec((self.o_size, R), "matrix"),
             "out_weight": ParamSpec((D, self.o_size), "matrix")}
        if self.own_kv:
            p["dkv_weight"] = ParamSpec((self.key_dim, D), "matrix")
            p["dkv_norm"] = ParamSpec((R,), "vector")
        if self.gated:
            p["g_weight"] = ParamSpec((self.o_size, D), "matrix")
        return p

    def kernel_limits(self, dtype: str):
        from .. import ops
        out = []
        if self.kv_rank > ops.LATENT_MAX_RANK or self.key_dim > ops.LATENT_MAX_KEY:
            out.append(f"latent attention: a latent of {self.kv_rank} with {self.rot_dim} rotated columns; the kernel takes "
                       f"latents up to {ops.LATENT_MAX_RANK} and rows up to {ops.LATENT_MAX_KEY}")
        return out

    def cache_need(self):
        if not self.own_kv:
            return None
        return PagedNeed(kv_heads=1, head_dim=self.row, values_in_keys=True)

    def bind(self, params, rt) -> None:
        import torch
        super().bind(params, rt)
        if not params:
            return
        H, dn, dv, R = self.num_heads, self.head_dim, self.v_head_dim, self.kv_rank
        # per head: [R, dn] (the transposed up-projection of keys, for the absorbed query) and [dv, R]
        self.uk_t = self.uk_weight.view(H, dn, R).transpose(1, 2).contiguous()
        self.uv = self.uv_weight.view(H, dv, R)
        freq, self.mscale = rotary_table(self.rot_dims, self.rot_base, self.rot_scaling)
        self.freq = torch.tensor(freq, dtype=torch.float64).to(torch.float32).to(rt.device)
        self.uk_weight = None

    def core(self, proj, ctx, cache, out, out_scale: float = 1.0) -> None:
        import torch
        if out_scale != 1.0:
            raise NotImplementedError("latent attention takes no branch factor")
        if cache.k_pages is None:
            raise RuntimeError("latent attention: the layer has no cache (a layer without W_dkv must be given another layer's)")
        ops = self.rt.ops
        T = proj.shape[0]
        H, R, dk = self.num_heads, self.kv_rank, self.key_dim
        gv = ctx.groups[cache.group]
        qa = ctx.ws.buf("latent_q", T, H * dk, torch.float32)
        write = self.own_kv and cache.write
        ops.latent_prepare(proj, 0, self.q_size if self.own_kv else None, ctx, gv.slot_mapping, self.freq, self.mscale,
                           self.dkv_norm, self.norm_eps, cache.k_pages, qa, heads=H, dim=self.head_dim, rot_dim=self.rot_dim,
                           rank=R, rot_dims=self.rot_dims, write=write)
        ops.headwise_linear(proj[:, :self.q_size], self.head_dim + self.rot_dim, self.uk_t, qa, dk)
        ol = ctx.ws.buf("latent_o", T, H * R, torch.float32)
        ops.latent_attention(qa, cache.k_pages, gv.block_table, ctx, ol, heads=H, rank=R, scale=self.scale)
        g0 = self.q_size + (self.key_dim if self.own_kv else 0)
        ops.headwise_linear(ol, R, self.uv, out, self.v_head_dim,
                            gate=proj[:, g0:g0 + self.o_size] if self.gated else None)


register_part("mixer", "latent_attention", LatentAttention)
