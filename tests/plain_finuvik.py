"""A plain, slow statement of the Finuvik design: whole sequences, no cache, float64.

One function per mechanism, written from the design's equations; it shares no code
with the package.  ``tensors`` maps checkpoint names to torch tensors, ``cfg`` is the
parsed config.json.  ``store`` rounds the values that the engine hands from kernel to
kernel in its activation dtype (identity for the 32-bit path).

Notation: D width, T tokens, p position (from 0), H / G query / key-value heads of the
softmax branch, dk / dv its key and value sizes; Hr, ek, ev the same for the recurrent
branch.
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Optional

import torch

F64 = torch.float64


def _keep(x):
    return x


def to_bf16(x):
    return x.to(torch.bfloat16).to(F64)


def rms_norm(x, w, eps, unit_offset: bool):
    """y = x / sqrt(mean(x^2) + eps) * (1 + w) (or * w without the offset)."""
    r = torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return x / r * ((1.0 + w) if unit_offset else w)


def query_temperature(positions, coef: float, every: int):
    """1 + coef * ln(floor((p + 1) / every) + 1), one factor per position."""
    steps = torch.div(positions + 1, every, rounding_mode="floor").to(F64)
    return 1.0 + coef * torch.log(steps + 1.0)


def distance_bias(n_q: int, n_k: int, q_start: int, r1, r2):
    """[H, n_q, n_k]: r1_h * ln(1 + r2_h * (i - j)) for j <= i (zero elsewhere; masked anyway)."""
    i = torch.arange(q_start, q_start + n_q, dtype=F64)[:, None]
    j = torch.arange(n_k, dtype=F64)[None, :]
    dist = (i - j).clamp(min=0.0)
    return r1[:, None, None] * torch.log1p(r2[:, None, None] * dist[None])


def softmax_branch(h, w: Dict[str, torch.Tensor], c: dict, store: Callable = _keep, out_scale: float = 1.0):
    """Causal softmax attention with grouped key/value heads, a query temperature that grows with the
    position and a logarithmic distance penalty.  h [T, D] -> [T, D], times out_scale (the engine applies a
    branch's factor to the attention's result before it rounds it for the output projection; so does this)."""
    T = h.shape[0]
    H, G, dk, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = store(h @ w["q"].t()).view(T, H, dk)
    k = store(h @ w["k"].t()).view(T, G, dk)
    v = store(h @ w["v"].t()).view(T, G, dv)
    pos = torch.arange(T)
    qt = c.get("q_temp")
    if qt:
        q = q * query_temperature(pos, float(qt["coef"]), int(qt["every"]))[:, None, None]
    out = torch.zeros(T, H, dv, dtype=F64)
    bias = distance_bias(T, T, 0, w["r1"].to(F64), w["r2"].to(F64))
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for hh in range(H):
        g = hh // (H // G)
        s = (q[:, hh] @ k[:, g].t()) * float(c["scale"]) - bias[hh]
        s = s.masked_fill(~mask, float("-inf"))
        out[:, hh] = torch.softmax(s, -1) @ v[:, g]
    return store(out_scale * out.reshape(T, H * dv)) @ w["o"].t()


def forget_gate(z, bias, lower):
    """f = l + (1 - l) * sigmoid(z + b)."""
    return lower + (1.0 - lower) * torch.sigmoid(z + bias)


def gated_recurrence(q, f, v, state: Optional[torch.Tensor] = None):
    """Per head: S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T, o_t = S_t^T q_t.
    q, f [T, Hr, ek]; v [T, Hr, ev]; state [Hr, ek, ev] (zeros when None).  Returns (o [T, Hr, ev], state)."""
    T, Hr, ek = q.shape
    ev = v.shape[-1]
    S = torch.zeros(Hr, ek, ev, dtype=F64) if state is None else state.clone()
    o = torch.zeros(T, Hr, ev, dtype=F64)
    for t in range(T):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return o, S


def recurrent_branch(h, w: Dict[str, torch.Tensor], c: dict, eps: float, store: Callable = _keep, out_scale: float = 1.0):
    """The gated linear-attention branch whose forget gate also sets what is written.  h [T, D] -> [T, D], times
    out_scale (applied where the engine applies it: to the normed outputs, before they are rounded)."""
    T = h.shape[0]
    Hr, ek, ev = c["heads"], c["dim"], c["vdim"]
    q = torch.nn.functional.silu(store(h @ w["q"].t())).view(T, Hr, ek)
    z = store(h @ w["f"].t())
    f = forget_gate(z, w["f.b"].to(F64), w["lower"].to(F64)).view(T, Hr, ek)
    v = store(h @ w["v"].t()).view(T, Hr, ev)
    o, _ = gated_recurrence(q, f, v)
    o = rms_norm(o, w["norm"].to(F64), eps, unit_offset=False)
    return store(out_scale * o.reshape(T, Hr * ev)) @ w["o"].t()


def dense_ff(h, w: Dict[str, torch.Tensor], store: Callable = _keep):
    """W_down (relu(W_gate h) * (W_up h))."""
    g = store(h @ w["gate"].t())
    u = store(h @ w["up"].t())
    return store(torch.relu(g) * u) @ w["down"].t()


def _sub(tensors, prefix):
    n = len(prefix)
    return {k[n:]: v.to(F64) for k, v in tensors.items() if k.startswith(prefix)}


def weight_layer(cfg: dict, i: int) -> int:
    """The layer whose tensors layer i uses."""
    seen = set()
    while "weights_of" in cfg["layers"][i] and cfg["layers"][i]["weights_of"] is not None:
        if i in seen:
            raise ValueError("weights_of forms a loop")
        seen.add(i)
        i = int(cfg["layers"][i]["weights_of"])
    return i


def forward(tensors: Dict[str, torch.Tensor], cfg: dict, ids: List[int], store: Callable = _keep,
            residuals: Optional[list] = None):
    """Logits [T, vocab] (float64) for one whole sequence from position 0."""
    eps = float(cfg["norm"]["eps"])
    T = len(ids)
    x = tensors["embed"].to(F64)[torch.tensor(ids)] + tensors["pos"].to(F64)[:T]
    for i, layer in enumerate(cfg["layers"]):
        if layer["type"] != "parallel":
            raise ValueError(f"layer {i}: unknown type {layer['type']!r}")
        p = f"l{weight_layer(cfg, i)}."
        m = layer["mixer"]
        h1 = store(rms_norm(x, tensors[p + "norm1"].to(F64), eps, unit_offset=True))
        add = softmax_branch(h1, _sub(tensors, p + "mix.left."), m["left"], store, float(m["left_scale"])) \
            + recurrent_branch(h1, _sub(tensors, p + "mix.right."), m["right"], eps, store, float(m["right_scale"]))
        if layer.get("mlp"):
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(f"layer {i}: unknown feed-forward kind {layer['mlp']['kind']!r}")
            h2 = store(rms_norm(x, tensors[p + "norm2"].to(F64), eps, unit_offset=True))
            add = add + dense_ff(h2, _sub(tensors, p + "mlp."), store)
        x = x + add
        if residuals is not None:
            residuals.append(x.clone())
    y = store(rms_norm(x, tensors["final.norm"].to(F64), eps, unit_offset=True))
    return y @ tensors["head"].to(F64).t()
