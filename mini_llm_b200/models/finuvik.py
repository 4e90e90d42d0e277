"""Finuvik: configuration -> model description.

A decoder with a learned position table added to the token embedding, a 32-bit
residual stream and parallel blocks, x += mixer(norm1(x)) + ff(norm2(x)), whose
two RMS norms (weights stored around zero) read the same x.  The mixer is two
branches on the same input, added with fixed factors: softmax attention with
grouped key/value heads of their own sizes, a query temperature and a
logarithmic distance penalty (``parts.attention.DistanceBiasAttention``), and
a gated linear recurrence with a matrix state per head
(``parts.recurrent.GatedLinearRecurrence``).  The feed-forward is gated with
ReLU, or absent.  A layer may use another layer's tensors (``weights_of``)
while keeping its own cache and state: it becomes another run of that layer
in the schedule, with a private cache.  The head is a matrix of its own.

Tensor names: embed, pos, final.norm, head; l<i>.norm1, l<i>.norm2,
l<i>.mix.left.{q,k,v,o,r1,r2}, l<i>.mix.right.{q,f,f.b,lower,v,norm,o},
l<i>.mlp.{gate,up,down}; matrices are stored [out, in].
"""
from __future__ import annotations

import math

from ..config.base import register_architecture
from ..config.finuvik import FinuvikConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, WeightRef

FF_ACTIVATION = "relu"      # fixed by the design


def build_finuvik_spec(cfg: FinuvikConfig) -> ModelSpec:
    D = cfg.width
    std = 1.0 / math.sqrt(D)

    def norm(name):
        return PartSpec("rmsnorm", dict(hidden_size=D, eps=cfg.norm_eps, unit_offset=True),
                        {"weight": WeightRef((name,), init=("normal", 0.1))})

    layers, index_of, schedule, ignored = [], {}, [], []
    for i, lay in enumerate(cfg.layers):
        if cfg.weight_layer(i) != i:
            continue
        p = f"l{i}."
        L, R = lay.left, lay.right
        left = dict(name="left", kind="distance_bias_attention",
                    params=dict(hidden_size=D, num_heads=L.heads, num_kv_heads=L.kv_heads, head_dim=L.dim,
                                v_head_dim=L.vdim, scale=L.scale, max_positions=cfg.max_positions,
                                q_temp_coef=L.q_temp_coef, q_temp_every=L.q_temp_every, log_distance_bias=True))
        right = dict(name="right", kind="gated_linear_recurrence",
                     params=dict(hidden_size=D, num_heads=R.heads, head_dim=R.dim, v_head_dim=R.vdim,
                                 norm_eps=cfg.norm_eps))
        m = p + "mix."
        mixer = PartSpec(
            "parallel", dict(branches=[left, right], scales=[lay.left_scale, lay.right_scale]),
            {"left.q_weight": WeightRef((m + "left.q",), init=("normal", std)),
             "left.k_weight": WeightRef((m + "left.k",), init=("normal", std)),
             "left.v_weight": WeightRef((m + "left.v",), init=("normal", std)),
             "left.r1": WeightRef((m + "left.r1",), init=("uniform", 0.2, 1.0)),
             "left.r2": WeightRef((m + "left.r2",), init=("uniform", 0.05, 0.5)),
             "left.out_weight": WeightRef((m + "left.o",), init=("normal", 1.0 / math.sqrt(L.heads * L.vdim))),
             "right.q_weight": WeightRef((m + "right.q",), init=("normal", std)),
             "right.f_weight": WeightRef((m + "right.f",), init=("normal", std)),
             "right.f_bias": WeightRef((m + "right.f.b",), init=("normal", 1.0)),
             "right.lower": WeightRef((m + "right.lower",), init=("uniform", 0.0, 0.9)),
             "right.v_weight": WeightRef((m + "right.v",), init=("normal", std)),
             "right.norm_weight": WeightRef((m + "right.norm",), init=("uniform", 0.5, 1.5)),
             "right.out_weight": WeightRef((m + "right.o",), init=("normal", 1.0 / math.sqrt(R.heads * R.vdim)))})
        ff = ff_norm = None
        if lay.ff is not None:
            ff = PartSpec("gated_mlp", dict(hidden_size=D, inner_size=lay.ff, activation=FF_ACTIVATION),
                          {"gate_weight": WeightRef((p + "mlp.gate",), init=("normal", std)),
                           "up_weight": WeightRef((p + "mlp.up",), init=("normal", std)),
                           "down_weight": WeightRef((p + "mlp.down",), init=("normal", 1.0 / math.sqrt(lay.ff)))})
            ff_norm = norm(p + "norm2")
        else:
            ignored.append(rf"^l{i}\.norm2$")       # a layer without a feed-forward has no use for a second norm
        index_of[i] = len(layers)
        layers.append(LayerSpec(mixer=mixer, ff=ff, mixer_norm=norm(p + "norm1"), ff_norm=ff_norm, arrangement="parallel"))
    for i in range(len(cfg.layers)):
        j = cfg.weight_layer(i)
        schedule.append(ScheduleEntry(index_of[j], private_cache=(j != i)))
    return ModelSpec(hidden_size=D, vocab_size=cfg.vocab,
                     embedding=PartSpec("token", dict(hidden_size=D, vocab_size=cfg.vocab),
                                        {"table": WeightRef(("embed",), init=("normal", 1.0))}),
                     positions=PartSpec("learned", dict(hidden_size=D, max_positions=cfg.max_positions),
                                        {"table": WeightRef(("pos",), init=("normal", 0.3))}),
                     layers=layers, final_norm=norm("final.norm"),
                     head=PartSpec("linear", dict(hidden_size=D, vocab_size=cfg.vocab),
                                   {"weight": WeightRef(("head",), init=("normal", std))}),
                     schedule=schedule, max_positions=cfg.max_positions, eos_token_id=cfg.eos_token_id,
                     ignored_tensors=ignored)


register_architecture("Finuvik", FinuvikConfig, build_finuvik_spec, replace=True)
