"""Falisun: configuration -> model description.

A decoder without a position table (positions enter through the rotation inside the attention layers), a 32-bit
residual stream, and layers x <- x + s1 * norm1b(mixer(norm1(x))), x <- x + s2 * norm2b(ff(norm2(x))): RMS norms with
plain weights before and after each branch and a learned scale per column on the normed result (arrangement
"sandwich" with "norm_scale" joins).  The mixer of a layer is attention over a cache of latents
(``parts.latent.LatentAttention``; a layer may read the cached rows of an earlier layer instead of making its own)
or a Mamba-2 state-space mixer (``parts.ssm.Mamba2Mixer``); the feed-forward is a mixture of gated experts with a
group-limited router and a shared expert (``parts.moe.MoEFeedForward``), or absent.  The head is the embedding table.

Tensor names: embed, final.norm; l<i>.{norm1,norm1b,norm2,norm2b,ls1,ls2};
l<i>.mix.{q,dkv,dkv.norm,uk,uv,g,o} or l<i>.mix.{in,conv,conv.b,dt_bias,A_log,D,norm,o};
l<i>.mlp.router, l<i>.mlp.e<k>.{gate,up,down}, l<i>.mlp.shared.{gate,up,down}; matrices are stored [out, in].
"""
from __future__ import annotations

import math

from ..config.base import register_architecture
from ..config.falisun import FalisunConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, WeightRef


def build_falisun_spec(cfg: FalisunConfig) -> ModelSpec:
    D = cfg.width
    std = 1.0 / math.sqrt(D)

    def norm(name):
        return PartSpec("rmsnorm", dict(hidden_size=D, eps=cfg.norm_eps, unit_offset=False),
                        {"weight": WeightRef((name,), init=("uniform", 0.5, 1.5))})

    def join(norm_name, scale_name):
        return PartSpec("norm_scale", dict(hidden_size=D, eps=cfg.norm_eps, scaled=True),
                        {"weight": WeightRef((norm_name,), init=("uniform", 0.5, 1.5)),
                         "scale": WeightRef((scale_name,), init=("uniform", 0.2, 1.0))})

    layers, schedule, ignored = [], [], []
    for i, lay in enumerate(cfg.layers):
        p = f"l{i}."
        m = p + "mix."
        s = lay.mixer
        if lay.type == "latent_attention":
            own = s.kv_from is None
            weights = {"q_weight": WeightRef((m + "q",), init=("normal", std)),
                       "uk_weight": WeightRef((m + "uk",), init=("normal", 1.0 / math.sqrt(s.kv_rank))),
                       "uv_weight": WeightRef((m + "uv",), init=("normal", 1.0 / math.sqrt(s.kv_rank))),
                       "g_weight": WeightRef((m + "g",), init=("normal", std)),
                       "out_weight": WeightRef((m + "o",), init=("normal", 1.0 / math.sqrt(s.heads * s.vdim)))}
            if own:
                weights["dkv_weight"] = WeightRef((m + "dkv",), init=("normal", std))
                weights["dkv_norm"] = WeightRef((m + "dkv.norm",), init=("uniform", 0.5, 1.5))
            mixer = PartSpec("latent_attention",
                             dict(hidden_size=D, num_heads=s.heads, head_dim=s.dim, rot_dim=s.rot_dim, v_head_dim=s.vdim,
                                  kv_rank=s.kv_rank, scale=s.scale, norm_eps=cfg.norm_eps, rot_dims=s.rot_dims,
                                  rot_base=s.rot_base, rot_scaling=s.rot_scaling, own_kv=own, gated=True), weights)
            schedule.append(ScheduleEntry(i, cache_of=i if own else s.kv_from))
        else:
            inner = s.heads * s.vdim
            mixer = PartSpec("mamba2",
                             dict(hidden_size=D, num_heads=s.heads, v_head_dim=s.vdim, state_size=s.state, groups=s.groups,
                                  conv_taps=s.conv, norm_groups=s.norm_groups, norm_eps=cfg.norm_eps),
                             {"in_proj": WeightRef((m + "in",), init=("normal", std)),
                              "conv_weight": WeightRef((m + "conv",), init=("normal", 0.5)),
                              "conv_bias": WeightRef((m + "conv.b",), init=("normal", 0.1)),
                              "dt_bias": WeightRef((m + "dt_bias",), init=("uniform", -3.0, 0.0)),
                              "A_log": WeightRef((m + "A_log",), init=("uniform", -1.0, 1.0)),
                              "D": WeightRef((m + "D",), init=("uniform", 0.5, 1.5)),
                              "norm_weight": WeightRef((m + "norm",), init=("uniform", 0.5, 1.5)),
                              "out_weight": WeightRef((m + "o",), init=("normal", 1.0 / math.sqrt(inner)))})
            schedule.append(ScheduleEntry(i))
        ff = ff_norm = ff_join = None
        if lay.mlp is not None:
            f = lay.mlp
            w = {"router": WeightRef((p + "mlp.router",), init=("normal", 2.0 * std))}
            for e in range(f.experts):
                w[f"expert{e}.gate"] = WeightRef((f"{p}mlp.e{e}.gate",), init=("normal", std))
                w[f"expert{e}.up"] = WeightRef((f"{p}mlp.e{e}.up",), init=("normal", std))
                w[f"expert{e}.down"] = WeightRef((f"{p}mlp.e{e}.down",), init=("normal", 1.0 / math.sqrt(f.expert_ff)))
            if f.shared_ff is not None:
                w["shared.gate"] = WeightRef((p + "mlp.shared.gate",), init=("normal", std))
                w["shared.up"] = WeightRef((p + "mlp.shared.up",), init=("normal", std))
                w["shared.down"] = WeightRef((p + "mlp.shared.down",), init=("normal", 1.0 / math.sqrt(f.shared_ff)))
            ff = PartSpec("moe", dict(hidden_size=D, num_experts=f.experts, top=f.top, expert_size=f.expert_ff,
                                      groups=f.groups, keep=f.keep, shared_size=f.shared_ff, activation="silu"), w)
            ff_norm = norm(p + "norm2")
            ff_join = join(p + "norm2b", p + "ls2")
        else:
            ignored.append(rf"^l{i}\.(norm2|norm2b|ls2)$")     # a layer without a feed-forward has no use for them
        layers.append(LayerSpec(mixer=mixer, ff=ff, mixer_norm=norm(p + "norm1"), ff_norm=ff_norm, arrangement="sandwich",
                                mixer_join=join(p + "norm1b", p + "ls1"), ff_join=ff_join))
    return ModelSpec(hidden_size=D, vocab_size=cfg.vocab,
                     embedding=PartSpec("token", dict(hidden_size=D, vocab_size=cfg.vocab),
                                        {"table": WeightRef(("embed",), init=("normal", 1.0))}),
                     positions=PartSpec("none", {}, {}),
                     layers=layers, final_norm=norm("final.norm"),
                     head=PartSpec("tied", dict(hidden_size=D, vocab_size=cfg.vocab), {}),
                     schedule=schedule, max_positions=cfg.max_positions, eos_token_id=cfg.eos_token_id,
                     ignored_tensors=ignored)


register_architecture("Falisun", FalisunConfig, build_falisun_spec, replace=True)
