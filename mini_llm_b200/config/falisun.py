"""FalisunConfig: the keys of a Falisun config.json, typed and checked.

A Falisun model is a list of layers.  Every entry names its mixer ("latent_attention" or "mamba2") with that
mixer's sizes and constants, and its feed-forward (a mixture of experts) or none.  Nothing is assumed equal
between layers: every size is read per entry.  A latent-attention layer may name another layer whose cached
latents it reads instead of making its own (``kv_from``).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .base import ConfigError, ModelConfig
from .finuvik import _int, _num

LAYER_TYPES = ("latent_attention", "mamba2")
FF_KINDS = ("moe",)


@dataclass
class LatentAttentionSizes:
    heads: int
    dim: int                  # unrotated query/key columns per head
    rot_dim: int              # rotated query/key columns per head (the key's are shared by all heads)
    vdim: int                 # value columns per head
    kv_rank: int              # size of the cached latent
    scale: float              # factor on the scores, as given
    rot_dims: int             # how many of the rot_dim columns turn
    rot_base: float
    rot_scaling: Optional[Dict[str, float]] = None     # YaRN: factor, original, fast, slow
    kv_from: Optional[int] = None                      # the layer whose cached rows this one reads


@dataclass
class Mamba2Sizes:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int                 # taps of the short convolution
    norm_groups: int


@dataclass
class MoESizes:
    experts: int
    top: int
    expert_ff: int
    groups: int = 1
    keep: int = 1
    shared_ff: Optional[int] = None


@dataclass
class FalisunLayer:
    type: str
    mixer: Any
    mlp: Optional[MoESizes] = None


@dataclass
class FalisunConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    norm_eps: float = 1e-5
    layers: List[FalisunLayer] = field(default_factory=list)
    eos_token_id: Optional[int] = None
    max_positions: Optional[int] = None
    raw: Dict[str, Any] = field(default_factory=dict, repr=False)

    @staticmethod
    def _latent(m: dict, where: str, n_layers: int, index: int) -> LatentAttentionSizes:
        rot = m.get("rot")
        if not isinstance(rot, dict):
            raise ConfigError(f"config.json: {where}.rot must be an object with 'base' and 'dims'")
        rot_dim = _int(m, "rot_dim", where, minimum=0)
        dims = _int(rot, "dims", where + ".rot", minimum=0)
        if dims % 2 or dims > rot_dim:
            raise ConfigError(f"config.json: {where}.rot.dims={dims} must be even and at most rot_dim={rot_dim}")
        scaling = rot.get("scaling")
        if scaling is not None:
            if not isinstance(scaling, dict):
                raise ConfigError(f"config.json: {where}.rot.scaling must be an object or null")
            scaling = {k: _num(scaling, k, where + ".rot.scaling") for k in ("factor", "original", "fast", "slow")}
            if scaling["factor"] <= 0 or scaling["original"] <= 0 or scaling["fast"] <= 0 or scaling["slow"] <= 0:
                raise ConfigError(f"config.json: {where}.rot.scaling: factor, original, fast and slow must be positive")
        base = _num(rot, "base", where + ".rot")
        if base <= 1.0 and dims:
            raise ConfigError(f"config.json: {where}.rot.base must be greater than 1")
        src = m.get("kv_from")
        if src is not None:
            src = _int(m, "kv_from", where, minimum=0)
            if src >= n_layers or src == index:
                raise ConfigError(f"config.json: {where}.kv_from={src} names no other layer of the {n_layers}")
        return LatentAttentionSizes(heads=_int(m, "heads", where), dim=_int(m, "dim", where), rot_dim=rot_dim,
                                    vdim=_int(m, "vdim", where), kv_rank=_int(m, "kv_rank", where),
                                    scale=_num(m, "scale", where), rot_dims=dims, rot_base=base, rot_scaling=scaling,
                                    kv_from=src)

    @staticmethod
    def _mamba(m: dict, where: str) -> Mamba2Sizes:
        s = Mamba2Sizes(heads=_int(m, "heads", where), vdim=_int(m, "vdim", where), state=_int(m, "state", where),
                        groups=_int(m, "groups", where), conv=_int(m, "conv", where),
                        norm_groups=_int(m, "norm_groups", where))
        if s.heads % s.groups:
            raise ConfigError(f"config.json: {where}: heads={s.heads} is not a multiple of groups={s.groups}")
        if (s.heads * s.vdim) % s.norm_groups:
            raise ConfigError(f"config.json: {where}: heads * vdim = {s.heads * s.vdim} is not a multiple of "
                              f"norm_groups={s.norm_groups}")
        return s

    @staticmethod
    def _moe(mlp: dict, where: str) -> MoESizes:
        if mlp.get("kind") not in FF_KINDS:
            raise ConfigError(f"config.json: {where}.kind must be one of {FF_KINDS}, got {mlp.get('kind')!r}")
        r, ex = mlp.get("router"), mlp.get("expert")
        if not isinstance(r, dict) or not isinstance(ex, dict):
            raise ConfigError(f"config.json: {where} must have 'router' and 'expert' objects")
        experts, top = _int(r, "experts", where + ".router"), _int(r, "top", where + ".router")
        groups, keep = 1, 1
        g = r.get("groups")
        if g is not None:
            if not isinstance(g, dict):
                raise ConfigError(f"config.json: {where}.router.groups must be an object or null")
            groups, keep = _int(g, "count", where + ".router.groups"), _int(g, "keep", where + ".router.groups")
        if experts % groups or keep > groups:
            raise ConfigError(f"config.json: {where}.router: {experts} experts in {groups} groups, {keep} kept")
        if top > keep * (experts // groups):
            raise ConfigError(f"config.json: {where}.router: top={top} exceeds the {keep * (experts // groups)} experts of "
                              f"the kept groups")
        shared = mlp.get("shared")
        if shared is not None and not isinstance(shared, dict):
            raise ConfigError(f"config.json: {where}.shared must be an object or null")
        return MoESizes(experts=experts, top=top, expert_ff=_int(ex, "ff", where + ".expert"), groups=groups, keep=keep,
                        shared_ff=_int(shared, "ff", where + ".shared") if shared is not None else None)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "FalisunConfig":
        for key in ("vocab", "width", "norm", "layers"):
            if d.get(key) is None:
                raise ConfigError(f"config.json: missing required key {key!r}")
        if not isinstance(d["norm"], dict):
            raise ConfigError("config.json: 'norm' must be an object with 'eps'")
        eps = _num(d["norm"], "eps", "norm")
        if not eps > 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps!r}")
        if not isinstance(d["layers"], list) or not d["layers"]:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        n = len(d["layers"])
        layers: List[FalisunLayer] = []
        for i, e in enumerate(d["layers"]):
            where = f"layers[{i}]"
            if not isinstance(e, dict):
                raise ConfigError(f"config.json: {where} must be an object")
            if e.get("type") not in LAYER_TYPES:
                raise ConfigError(f"config.json: {where}.type must be one of {LAYER_TYPES}, got {e.get('type')!r}")
            m = e.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"config.json: {where}.mixer must be an object")
            mixer = cls._latent(m, where + ".mixer", n, i) if e["type"] == "latent_attention" else cls._mamba(m, where + ".mixer")
            mlp = e.get("mlp")
            if mlp is not None and not isinstance(mlp, dict):
                raise ConfigError(f"config.json: {where}.mlp must be an object or null")
            layers.append(FalisunLayer(type=e["type"], mixer=mixer, mlp=cls._moe(mlp, where + ".mlp") if mlp is not None else None))
        for i, lay in enumerate(layers):
            if lay.type != "latent_attention" or lay.mixer.kv_from is None:
                continue
            j = lay.mixer.kv_from
            src = layers[j]
            if src.type != "latent_attention" or src.mixer.kv_from is not None:
                raise ConfigError(f"config.json: layers[{i}].mixer.kv_from={j}: that layer keeps no latents of its own")
            if j > i:
                raise ConfigError(f"config.json: layers[{i}].mixer.kv_from={j}: the layer runs before the one whose rows it reads")
            a, b = lay.mixer, src.mixer
            if (a.kv_rank, a.rot_dim, a.rot_dims, a.rot_base, a.rot_scaling) != (b.kv_rank, b.rot_dim, b.rot_dims, b.rot_base, b.rot_scaling):
                raise ConfigError(f"config.json: layers[{i}] reads the rows of layers[{j}] but differs from it in kv_rank, "
                                  f"rot_dim or rotation")
        vocab = _int(d, "vocab", "config")
        eos = d.get("eos_token_id")
        if eos is not None and (isinstance(eos, bool) or not isinstance(eos, int) or not (0 <= eos < vocab)):
            raise ConfigError(f"config.json: eos_token_id {eos!r} is not a token of the vocabulary")
        mp = d.get("max_positions")
        if mp is not None:
            mp = _int(d, "max_positions", "config")
        cfg = cls(vocab=vocab, width=_int(d, "width", "config"), norm_eps=eps, layers=layers, eos_token_id=eos,
                  max_positions=mp, raw=copy.deepcopy(d))
        cfg.architecture = "Falisun"
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        d = copy.deepcopy(self.raw)
        d["architecture"] = "Falisun"
        return d
