"""FinuvikConfig: the keys of a Finuvik config.json, typed and checked.

A Finuvik model is a list of layers; every entry names its mixer's sizes and
constants, its feed-forward (or none) and, optionally, another layer whose
tensors it uses (``weights_of``) while keeping a cache and a state of its own
(such a layer runs the other layer's parts, with that layer's constants).
Nothing is assumed equal between layers: every size is read per entry.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .base import ConfigError, ModelConfig

LAYER_TYPES = ("parallel",)
FF_KINDS = ("dense",)


def _int(d, key, where, minimum=1):
    v = d.get(key)
    if isinstance(v, float) and v == int(v):
        v = int(v)
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"config.json: {where}.{key} must be an integer, got {v!r}")
    if v < minimum:
        raise ConfigError(f"config.json: {where}.{key} must be >= {minimum}, got {v}")
    return v


def _num(d, key, where):
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}.{key} must be a number, got {v!r}")
    return float(v)


@dataclass
class SoftmaxBranch:
    """The softmax-attention half of a parallel mixer."""
    heads: int
    kv_heads: int
    dim: int                 # size of a query / key head
    vdim: int                # size of a value head
    scale: float             # factor on q.k
    q_temp_coef: float = 0.0       # query temperature 1 + coef * ln(floor((p + 1) / every) + 1); 0: none
    q_temp_every: int = 1


@dataclass
class RecurrentBranch:
    """The gated linear-recurrence half of a parallel mixer."""
    heads: int
    dim: int                 # rows of a head's state (query / gate channels)
    vdim: int                # columns of a head's state (value channels)


@dataclass
class FinuvikLayer:
    type: str
    left: SoftmaxBranch
    right: RecurrentBranch
    left_scale: float
    right_scale: float
    ff: Optional[int] = None            # inner size of the dense feed-forward; None: the layer has none
    ff_kind: Optional[str] = None
    weights_of: Optional[int] = None    # the layer whose tensors this one uses


@dataclass
class FinuvikConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    max_positions: int = 0
    norm_eps: float = 1e-5
    layers: List[FinuvikLayer] = field(default_factory=list)
    eos_token_id: Optional[int] = None
    raw: Dict[str, Any] = field(default_factory=dict, repr=False)

    def weight_layer(self, i: int) -> int:
        """The layer whose tensors layer i uses (itself if it has its own)."""
        seen = set()
        while self.layers[i].weights_of is not None:
            if i in seen:
                raise ConfigError(f"config.json: layers[{i}].weights_of forms a loop")
            seen.add(i)
            i = self.layers[i].weights_of
        return i

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "FinuvikConfig":
        for key in ("vocab", "width", "max_positions", "norm", "layers"):
            if d.get(key) is None:
                raise ConfigError(f"config.json: missing required key {key!r}")
        if not isinstance(d["norm"], dict):
            raise ConfigError("config.json: 'norm' must be an object with 'eps'")
        eps = _num(d["norm"], "eps", "norm")
        if not eps > 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps!r}")
        if not isinstance(d["layers"], list) or not d["layers"]:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers: List[FinuvikLayer] = []
        n = len(d["layers"])
        for i, e in enumerate(d["layers"]):
            where = f"layers[{i}]"
            if not isinstance(e, dict):
                raise ConfigError(f"config.json: {where} must be an object")
            if e.get("type") not in LAYER_TYPES:
                raise ConfigError(f"config.json: {where}.type must be one of {LAYER_TYPES}, got {e.get('type')!r}")
            m = e.get("mixer")
            if not isinstance(m, dict) or not isinstance(m.get("left"), dict) or not isinstance(m.get("right"), dict):
                raise ConfigError(f"config.json: {where}.mixer must have 'left' and 'right' objects")
            l, r = m["left"], m["right"]
            heads, kv = _int(l, "heads", where + ".mixer.left"), _int(l, "kv_heads", where + ".mixer.left")
            if heads % kv != 0:
                raise ConfigError(f"config.json: {where}.mixer.left: heads={heads} is not a multiple of kv_heads={kv}")
            coef, every = 0.0, 1
            qt = l.get("q_temp")
            if qt is not None:
                if not isinstance(qt, dict):
                    raise ConfigError(f"config.json: {where}.mixer.left.q_temp must be an object")
                coef = _num(qt, "coef", where + ".mixer.left.q_temp")
                every = _int(qt, "every", where + ".mixer.left.q_temp")
            left = SoftmaxBranch(heads=heads, kv_heads=kv, dim=_int(l, "dim", where + ".mixer.left"),
                                 vdim=_int(l, "vdim", where + ".mixer.left"), scale=_num(l, "scale", where + ".mixer.left"),
                                 q_temp_coef=coef, q_temp_every=every)
            right = RecurrentBranch(heads=_int(r, "heads", where + ".mixer.right"),
                                    dim=_int(r, "dim", where + ".mixer.right"),
                                    vdim=_int(r, "vdim", where + ".mixer.right"))
            ff, kind = None, None
            mlp = e.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") not in FF_KINDS:
                    raise ConfigError(f"config.json: {where}.mlp.kind must be one of {FF_KINDS}")
                ff, kind = _int(mlp, "ff", where + ".mlp"), mlp["kind"]
            wo = e.get("weights_of")
            if wo is not None:
                wo = _int(e, "weights_of", where, minimum=0)
                if wo >= n or wo == i:
                    raise ConfigError(f"config.json: {where}.weights_of={wo} names no other layer of the {n}")
            layers.append(FinuvikLayer(type=e["type"], left=left, right=right,
                                       left_scale=_num(m, "left_scale", where + ".mixer"),
                                       right_scale=_num(m, "right_scale", where + ".mixer"), ff=ff, ff_kind=kind,
                                       weights_of=wo))
        eos = d.get("eos_token_id")
        vocab = _int(d, "vocab", "config")
        if eos is not None and (isinstance(eos, bool) or not isinstance(eos, int) or not (0 <= eos < vocab)):
            raise ConfigError(f"config.json: eos_token_id {eos!r} is not a token of the vocabulary")
        cfg = cls(vocab=vocab, width=_int(d, "width", "config"), max_positions=_int(d, "max_positions", "config"),
                  norm_eps=eps, layers=layers, eos_token_id=eos, raw=copy.deepcopy(d))
        cfg.architecture = "Finuvik"
        for i, lay in enumerate(layers):
            j = cfg.weight_layer(i)
            if j != i:
                # the layer runs layer j's parts, so layer j's constants hold; sizes that differ cannot be served
                a, b = lay, layers[j]
                sizes = lambda l: (l.left.heads, l.left.kv_heads, l.left.dim, l.left.vdim, l.right.heads, l.right.dim,
                                   l.right.vdim, l.ff)
                if sizes(a) != sizes(b):
                    raise ConfigError(f"config.json: layers[{i}] uses the tensors of layers[{j}] but differs from it in its sizes")
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        d = copy.deepcopy(self.raw)
        d["architecture"] = "Finuvik"
        return d
