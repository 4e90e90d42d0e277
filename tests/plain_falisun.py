"""A plain, slow statement of the Falisun design: whole sequences, no cache, float64.

One function per mechanism, written from the design's equations; it shares no code with
the package.  ``tensors`` maps checkpoint names to torch tensors, ``cfg`` is the parsed
config.json.  ``store`` rounds the values that the engine hands from kernel to kernel in
its activation dtype (identity for the 32-bit path).

Notation: D width, T tokens, p position (from 0).  Latent attention: H heads, dn / dr
unrotated / rotated query-key sizes, dv value size, R latent size.  Mamba-2: Hm heads of
size P, N state rows, G groups, taps of the short convolution.
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


def silu(x):
    return x * torch.sigmoid(x)


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


# ------------------------------------------------------------------------------------------- rotation
def rotary_frequencies(dims: int, base: float, scaling: Optional[dict]):
    """(f [dims/2], m): angle of pair i at position p is p * f_i; cos and sin are multiplied by m.
    With YaRN scaling pairs that turn slowly are slowed down by ``factor``, fast ones are left alone and
    a linear ramp lies between."""
    half = dims // 2
    i = torch.arange(half, dtype=F64)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def turn_dim(t):
        return dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(scaling["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, dims: int, base: float, scaling: Optional[dict]):
    """x [..., T, d]: the first ``dims`` entries are rotated in pairs (i, i + dims/2), the rest pass.  The design takes
    the angle in 32-bit: the frequency rounded to float32, times the position, rounded to float32."""
    f, m = rotary_frequencies(dims, base, scaling)
    a = (positions.to(torch.float32)[:, None] * f.to(torch.float32)[None, :]).to(F64)
    cos, sin = torch.cos(a) * m, torch.sin(a) * m
    half = dims // 2
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], -1)


# ------------------------------------------------------------------------------------------- latent attention
def latent_kv(h, w: Dict[str, torch.Tensor], m: dict, eps: float, store: Callable = _keep):
    """What a latent-attention layer keeps of its tokens: the normed latent c [T, R] and the rotated key part
    [T, dr] that all heads share."""
    T = h.shape[0]
    R, dr = m["kv_rank"], m["rot_dim"]
    d = store(h @ w["dkv"].t())
    c = rms_norm(d[:, :R], w["dkv.norm"], eps)
    rot = m["rot"]
    kr = rotate(d[:, R:R + dr], torch.arange(T), rot["dims"], rot["base"], rot.get("scaling"))
    return store(c), store(kr)


def latent_attention(h, w: Dict[str, torch.Tensor], m: dict, eps: float, kv=None, store: Callable = _keep):
    """h [T, D] -> [T, D].  ``kv``: (c, kr) of another layer to use instead of this layer's own."""
    T = h.shape[0]
    H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = m["rot"]
    q = store(h @ w["q"].t()).view(T, H, dn + dr)
    qn = q[..., :dn]
    qr = rotate(q[..., dn:].transpose(0, 1), torch.arange(T), rot["dims"], rot["base"], rot.get("scaling")).transpose(0, 1)
    c, kr = kv if kv is not None else latent_kv(h, w, m, eps, store)
    # the engine never forms the heads' keys and values of cached tokens (it takes W_uk to the query and W_uv to the
    # weighted sum of latents), so nothing is rounded here
    kn = (c @ w["uk"].t()).view(T, H, dn)
    v = (c @ w["uv"].t()).view(T, H, dv)
    s = (torch.einsum("ihd,jhd->hij", qn, kn) + torch.einsum("ihd,jd->hij", qr, kr)) * m["scale"]
    mask = torch.arange(T)[None, :] <= torch.arange(T)[:, None]
    s = s.masked_fill(~mask[None], float("-inf"))
    p = torch.softmax(s, -1)
    o = torch.einsum("hij,jhd->ihd", p, v).reshape(T, H * dv)
    g = torch.sigmoid(store(h @ w["g"].t()))
    return store(o * g) @ w["o"].t()


# ------------------------------------------------------------------------------------------- mamba-2
def short_convolution(u, weight, bias):
    """u [T, C]: y_t = bias + sum_j weight[:, j] * u_(t - (taps - 1) + j), zeros before the start."""
    T, C = u.shape
    taps = weight.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u], 0)
    y = bias[None, :].expand(T, C).clone()
    for j in range(taps):
        y = y + pad[j:j + T] * weight[:, j][None, :]
    return y


def selective_scan(x, B, C, dt, A_log, D, groups: int):
    """x [T, Hm, P], B, C [T, G, N], dt [T, Hm] (after softplus): S_t = exp(-exp(A_log) dt_t) S_(t-1) + dt_t B_t x_t^T,
    y_t = S_t^T C_t + D x_t, one state S [N, P] per head, zero at the start."""
    T, Hm, P = x.shape
    N = B.shape[2]
    per = Hm // groups
    y = torch.zeros(T, Hm, P, dtype=F64)
    for hh in range(Hm):
        g = hh // per
        S = torch.zeros(N, P, dtype=F64)
        a = -torch.exp(A_log[hh])
        for t in range(T):
            S = torch.exp(a * dt[t, hh]) * S + dt[t, hh] * B[t, g][:, None] * x[t, hh][None, :]
            y[t, hh] = S.t() @ C[t, g] + D[hh] * x[t, hh]
    return y


def mamba2(h, w: Dict[str, torch.Tensor], m: dict, eps: float, store: Callable = _keep):
    T = h.shape[0]
    Hm, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = Hm * P
    proj = store(h @ w["in"].t())
    z = proj[:, :inner]
    xbc = proj[:, inner:2 * inner + 2 * G * N]
    dt = proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(short_convolution(xbc, w["conv"], w["conv.b"]))
    x = xbc[:, :inner].reshape(T, Hm, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = torch.nn.functional.softplus(dt + w["dt_bias"][None, :], threshold=1e9)
    y = selective_scan(x, B, C, dt, w["A_log"], w["D"], G).reshape(T, inner)
    y = y * silu(z)
    ng = m["norm_groups"]
    y = rms_norm(y.view(T, ng, inner // ng), 1.0, eps).reshape(T, inner) * w["norm"]
    return store(y) @ w["o"].t()


# ------------------------------------------------------------------------------------------- feed-forward
def gated_expert(h, w: Dict[str, torch.Tensor], prefix: str, store: Callable = _keep, halves_stored: bool = False):
    """W_down (silu(W_gate h) * (W_up h)).  ``halves_stored``: the engine hands the two halves from a product to an
    activation kernel (the shared expert); the routed experts' product applies the activation itself."""
    inner = store if halves_stored else _keep
    return store(silu(inner(h @ w[prefix + "gate"].t())) * inner(h @ w[prefix + "up"].t())) @ w[prefix + "down"].t()


def route(h, router, r: dict):
    """Scores, chosen experts [T, top] and their weights [T, top]."""
    s = torch.softmax(h @ router.t(), -1)
    E, top = r["experts"], r["top"]
    allowed = torch.ones_like(s, dtype=torch.bool)
    grp = r.get("groups")
    if grp:
        n, keep = grp["count"], grp["keep"]
        best = s.view(-1, n, E // n).max(-1).values
        kept = best.topk(keep, -1).indices
        ok = torch.zeros_like(best, dtype=torch.bool).scatter_(1, kept, True)
        allowed = ok[:, :, None].expand(-1, n, E // n).reshape(-1, E)
    chosen = s.masked_fill(~allowed, -1.0).topk(top, -1).indices
    ws = s.gather(1, chosen)
    return s, chosen, ws / (ws.sum(-1, keepdim=True) + 1e-20)


def mixture_of_experts(h, w: Dict[str, torch.Tensor], mlp: dict, store: Callable = _keep):
    r = mlp["router"]
    _, chosen, weights = route(h, w["router"], r)
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=F64)
    for e in range(r["experts"]):
        for k in range(r["top"]):
            rows = (chosen[:, k] == e).nonzero()[:, 0]
            if rows.numel():
                out[rows] += weights[rows, k][:, None] * gated_expert(h[rows], w, f"e{e}.", store)
    if mlp.get("shared"):
        out = out + gated_expert(h, w, "shared.", store, halves_stored=True)
    return out


# ------------------------------------------------------------------------------------------- the model
def sub(tensors: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v.to(F64) for k, v in tensors.items() if k.startswith(prefix)}


def forward(tensors: Dict[str, torch.Tensor], cfg: dict, tokens, store: Callable = _keep, layers_out: Optional[List] = None):
    """Logits [T, vocab] of one whole sequence; ``layers_out`` collects the residual stream after every layer."""
    eps = cfg["norm"]["eps"]
    t = {k: v.to(F64) for k, v in tensors.items()}
    x = t["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    kept = {}
    for i, lay in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = lay["mixer"]
        h = store(rms_norm(x, t[p + "norm1"], eps))
        w = sub(t, p + "mix.")
        if lay["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = latent_kv(h, w, m, eps, store)
            y = latent_attention(h, w, m, eps, kv=kept[i if src is None else src], store=store)
        elif lay["type"] == "mamba2":
            y = mamba2(h, w, m, eps, store)
        else:
            raise ValueError(lay["type"])
        x = x + rms_norm(y, t[p + "norm1b"], eps) * t[p + "ls1"]
        if lay.get("mlp") is not None:
            h = store(rms_norm(x, t[p + "norm2"], eps))
            y = mixture_of_experts(h, sub(t, p + "mlp."), lay["mlp"], store)
            x = x + rms_norm(y, t[p + "norm2b"], eps) * t[p + "ls2"]
        if layers_out is not None:
            layers_out.append(x.clone())
    return store(rms_norm(x, t["final.norm"], eps)) @ t["embed"].t()
