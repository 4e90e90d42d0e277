"""Small Falisun configurations and weights for the tests: two models that differ from each other in every size and
option, with weights that make faults show."""
from __future__ import annotations

import math

import torch


def latent(heads, dim, rot_dim, vdim, kv_rank, scale, base=10000.0, dims=None, scaling=None, kv_from=None):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, scale=scale,
             rot=dict(base=base, dims=rot_dim if dims is None else dims, scaling=scaling))
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def mamba(heads, vdim, state, groups, conv, norm_groups):
    return dict(heads=heads, vdim=vdim, state=state, groups=groups, conv=conv, norm_groups=norm_groups)


def moe(experts, top, ff, groups=None, shared=None):
    router = dict(experts=experts, top=top)
    if groups is not None:
        router["groups"] = dict(count=groups[0], keep=groups[1])
    return dict(kind="moe", router=router, expert=dict(ff=ff), shared=dict(ff=shared) if shared else None)


def layer(kind, mixer, mlp):
    return dict(type=kind, mixer=mixer, mlp=mlp)


def config(width, vocab, eps, layers):
    return dict(architecture="Falisun", width=width, vocab=vocab, norm=dict(eps=eps), layers=layers)


YARN_P = dict(factor=4.0, original=32, fast=8.0, slow=1.0)
# P: attention first; three heads; a latent of 40 (no multiple of 32) with 8 rotated columns under YaRN whose original
# context (32) the prompts pass; a Mamba-2 layer without feed-forward whose state has 20 rows (no multiple of 8) and heads
# of 12 columns, one norm group, four taps; a layer that reads layer 0's rows with five heads of other sizes and a router
# without groups, one expert per token and no shared expert; a Mamba-2 layer with one group and two taps.
CFG_P = config(64, 97, 1e-6, [
    layer("latent_attention", latent(3, 16, 8, 24, 40, 0.3, base=100.0, scaling=YARN_P), moe(6, 2, 24, groups=(3, 2), shared=40)),
    layer("mamba2", mamba(4, 12, 20, 2, 4, 1), None),
    layer("latent_attention", latent(5, 8, 8, 16, 40, 0.45, base=100.0, scaling=YARN_P, kv_from=0), moe(4, 1, 16)),
    layer("mamba2", mamba(2, 40, 8, 1, 2, 2), moe(3, 3, 8, shared=8)),
])
# Q: Mamba-2 first (six heads in three groups, three norm groups); ten attention heads (two blocks of the attention
# kernel) over a latent of 136, only 8 of the 16 rotated columns turn, no frequency scaling; a layer that reads those rows;
# a last attention layer with a cache of its own of another row size (a second cache group), one head, no rotation at all.
CFG_Q = config(96, 211, 1e-5, [
    layer("mamba2", mamba(6, 16, 64, 3, 3, 3), moe(8, 3, 40, groups=(2, 1), shared=24)),
    layer("latent_attention", latent(10, 24, 16, 8, 136, 0.2, dims=8), None),
    layer("latent_attention", latent(2, 40, 16, 56, 136, 0.25, dims=8, kv_from=1), moe(5, 2, 24, groups=(5, 3))),
    layer("latent_attention", latent(1, 32, 4, 32, 24, 0.35, dims=0), moe(2, 1, 64, shared=16)),
])
CONFIGS = {"P": CFG_P, "Q": CFG_Q}
PAGE = {"P": 8, "Q": 16}


def make_tensors(cfg, seed):
    """Projections large enough for a peaked softmax (single keys carry weight), decays between fast and very slow,
    step sizes from small to large, norm weights and layer scales away from 0 and 1, routers that decide clearly."""
    g = torch.Generator().manual_seed(seed)
    D = cfg["width"]

    def normal(*shape, std):
        return torch.empty(*shape).normal_(0.0, std, generator=g)

    def uniform(*shape, lo, hi):
        return torch.empty(*shape).uniform_(lo, hi, generator=g)

    t = {"embed": normal(cfg["vocab"], D, std=0.8), "final.norm": uniform(D, lo=0.5, hi=1.5)}
    for i, lay in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lay["mixer"]
        for n in ("norm1", "norm1b"):
            t[p + n] = uniform(D, lo=0.5, hi=1.5)
        t[p + "ls1"] = uniform(D, lo=0.3, hi=1.2)
        if lay["type"] == "latent_attention":
            H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            t[p + "mix.q"] = normal(H * (dn + dr), D, std=2.0 / math.sqrt(D))
            if m.get("kv_from") is None:
                t[p + "mix.dkv"] = normal(R + dr, D, std=1.5 / math.sqrt(D))
                t[p + "mix.dkv.norm"] = uniform(R, lo=0.5, hi=1.5)
            t[p + "mix.uk"] = normal(H * dn, R, std=1.5 / math.sqrt(R))
            t[p + "mix.uv"] = normal(H * dv, R, std=1.0 / math.sqrt(R))
            t[p + "mix.g"] = normal(H * dv, D, std=1.5 / math.sqrt(D))
            t[p + "mix.o"] = normal(D, H * dv, std=1.0 / math.sqrt(H * dv))
        else:
            Hm, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
            inner, C = Hm * P, Hm * P + 2 * G * N
            t[p + "mix.in"] = normal(2 * inner + 2 * G * N + Hm, D, std=1.2 / math.sqrt(D))
            t[p + "mix.conv"] = normal(C, m["conv"], std=0.6)
            t[p + "mix.conv.b"] = normal(C, std=0.2)
            t[p + "mix.dt_bias"] = uniform(Hm, lo=-4.0, hi=1.0)
            t[p + "mix.A_log"] = uniform(Hm, lo=-3.0, hi=1.5)
            t[p + "mix.D"] = uniform(Hm, lo=0.3, hi=1.5)
            t[p + "mix.norm"] = uniform(inner, lo=0.5, hi=1.5)
            t[p + "mix.o"] = normal(D, inner, std=1.0 / math.sqrt(inner))
        f = lay.get("mlp")
        if f:
            for n in ("norm2", "norm2b"):
                t[p + n] = uniform(D, lo=0.5, hi=1.5)
            t[p + "ls2"] = uniform(D, lo=0.3, hi=1.2)
            t[p + "mlp.router"] = normal(f["router"]["experts"], D, std=3.0 / math.sqrt(D))
            names = [f"e{e}" for e in range(f["router"]["experts"])]
            sizes = [f["expert"]["ff"]] * len(names)
            if f.get("shared"):
                names.append("shared")
                sizes.append(f["shared"]["ff"])
            for n, F in zip(names, sizes):
                t[f"{p}mlp.{n}.gate"] = normal(F, D, std=1.2 / math.sqrt(D))
                t[f"{p}mlp.{n}.up"] = normal(F, D, std=1.2 / math.sqrt(D))
                t[f"{p}mlp.{n}.down"] = normal(D, F, std=1.0 / math.sqrt(F))
    return {k: v.to(torch.bfloat16).float() for k, v in t.items()}
