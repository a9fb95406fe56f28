"""Zusitar written out from its equations: whole sequences, float64, one function per mechanism.

Slow and plain on purpose: explicit ``[n, n]`` score matrices, a token-by-token selective scan,
Python loops over heads and experts.  It reads the design's ``config.json`` dictionary itself and
takes the checkpoint's tensors by their stored names; nothing of the package is imported, so the
engine and this file can only agree by computing the same design.

``rounding=torch.bfloat16`` rounds the results of the matrix products and of the activations that
the design allows in 16 bits, which shows how far 16-bit storage alone moves the logits.
"""

from __future__ import annotations

import math
from typing import Dict, List, Mapping, Optional

import torch

F64 = torch.float64


def _r(x: torch.Tensor, rounding) -> torch.Tensor:
    return x if rounding is None else x.to(rounding).to(F64)


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def causal_conv(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor]) -> torch.Tensor:
    """``y[t, c] = b[c] + sum_j w[c, j] * x[t - taps + 1 + j, c]`` with zeros before the start."""
    n, taps = x.shape[0], w.shape[1]
    y = torch.zeros_like(x)
    for j in range(taps):
        back = taps - 1 - j
        if back < n:
            y[back:] += x[:n - back] * w[:, j]
    return y if b is None else y + b


def rotate(x: torch.Tensor, dims: int, base: float, pairing: str) -> torch.Tensor:
    """``x [n, heads, d]``: the first ``dims`` coordinates of every head turned by the position's
    angles ``p * base^(-2i/dims)``; ``pairing`` ``"half"`` pairs ``i`` with ``i + dims/2``,
    ``"interleaved"`` pairs ``2i`` with ``2i + 1``."""
    n = x.shape[0]
    if dims == 0:
        return x
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    ang = torch.arange(n, dtype=F64)[:, None] * freq[None, :]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    if pairing == "half":
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half] = u * cos - v * sin
        out[..., half:dims] = v * cos + u * sin
    else:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * cos - v * sin
        out[..., 1:dims:2] = v * cos + u * sin
    return out


def selective_scan_mixer(h, W: Mapping[str, torch.Tensor], p: str, cfg: Mapping, rounding) -> torch.Tensor:
    n = h.shape[0]
    inner, state, rank = cfg["inner"], cfg["state"], cfg["dt_rank"]
    xz = _r(h @ W[p + ".in"].T, rounding)
    x, z = xz[:, :inner], xz[:, inner:]
    x = _r(silu(_r(causal_conv(x, W[p + ".conv"], W[p + ".conv.b"]), rounding)), rounding)
    proj = _r(x @ W[p + ".x"].T, rounding)
    dt_in, B, C = proj[:, :rank], proj[:, rank:rank + state], proj[:, rank + state:rank + 2 * state]
    dt = softplus(_r(dt_in @ W[p + ".dt"].T, rounding) + W[p + ".dt.b"])
    A = -torch.exp(W[p + ".A_log"])
    S = torch.zeros(inner, state, dtype=F64)
    y = torch.zeros(n, inner, dtype=F64)
    for t in range(n):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + W[p + ".D"] * x[t]
    y = _r(y * silu(z), rounding)
    return _r(y @ W[p + ".o"].T, rounding)


def latent_attention(h, W: Mapping[str, torch.Tensor], p: str, cfg: Mapping, eps: float, rounding) -> torch.Tensor:
    n = h.shape[0]
    H, d, dr, dv, rank = cfg["heads"], cfg["dim"], cfg["rot_dim"], cfg["vdim"], cfg["kv_rank"]
    cq = _r(rms(_r(h @ W[p + ".dq"].T, rounding), eps) * W[p + ".dq.norm"], rounding)
    q = _r(cq @ W[p + ".uq"].T, rounding).view(n, H, d + dr)
    down = _r(h @ W[p + ".dkv"].T, rounding)
    c = _r(rms(down[:, :rank], eps) * W[p + ".dkv.norm"], rounding)
    k_rot = rotate(down[:, None, rank:], cfg["rot"]["dims"], cfg["rot"]["base"], "half")[:, 0]
    q_rot = rotate(q[..., d:], cfg["rot"]["dims"], cfg["rot"]["base"], "half")
    k = (c @ W[p + ".uk"].T).view(n, H, d)
    v = (c @ W[p + ".uv"].T).view(n, H, dv)
    seen = torch.arange(n)[:, None] >= torch.arange(n)[None, :]
    out = torch.zeros(n, H, dv, dtype=F64)
    for a in range(H):
        s = (q[:, a, :d] @ k[:, a].T + q_rot[:, a] @ k_rot.T) * cfg["scale"]
        s = s.masked_fill(~seen, float("-inf"))
        out[:, a] = torch.softmax(s, dim=-1) @ v[:, a]
    gate = torch.sigmoid(_r(h @ W[p + ".g"].T, rounding))
    o = _r(_r(out.reshape(n, H * dv), rounding) * gate, rounding)
    return _r(o @ W[p + ".o"].T, rounding)


def sink_attention(h, W: Mapping[str, torch.Tensor], p: str, cfg: Mapping, rounding) -> torch.Tensor:
    n = h.shape[0]
    H, G, d, dv = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    q = _r(h @ W[p + ".q"].T + W[p + ".q.b"], rounding).view(n, H, d)
    k = _r(h @ W[p + ".k"].T + W[p + ".k.b"], rounding).view(n, G, d)
    v = _r(h @ W[p + ".v"].T + W[p + ".v.b"], rounding).view(n, G, dv)
    q = _r(rotate(q, cfg["rot"]["dims"], cfg["rot"]["base"], "interleaved"), rounding)
    k = _r(rotate(k, cfg["rot"]["dims"], cfg["rot"]["base"], "interleaved"), rounding)
    seen = torch.arange(n)[:, None] >= torch.arange(n)[None, :]
    gate = torch.sigmoid(_r(h @ W[p + ".g"].T, rounding))            # [n, H]
    cap = cfg["softcap"]
    out = torch.zeros(n, H, dv, dtype=F64)
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * cfg["scale"]
        s = cap * torch.tanh(s / cap)
        s = s.masked_fill(~seen, float("-inf"))
        m = torch.maximum(s.max(-1, keepdim=True).values, W[p + ".sink"][a])
        e = torch.exp(s - m)
        den = e.sum(-1, keepdim=True) + torch.exp(W[p + ".sink"][a] - m)
        out[:, a] = (e / den) @ v[:, g] * gate[:, a:a + 1]
    return _r(_r(out.reshape(n, H * dv), rounding) @ W[p + ".o"].T + W[p + ".o.b"], rounding)


def dense_ffn(h, W, p: str, rounding) -> torch.Tensor:
    g = _r(h @ W[p + ".gate"].T, rounding)
    u = _r(h @ W[p + ".up"].T, rounding)
    return _r(_r(silu(g) * u, rounding) @ W[p + ".down"].T, rounding)


def bounded_expert(h, W, p: str, limit: float, rounding) -> torch.Tensor:
    g = torch.clamp(_r(h @ W[p + ".gate"].T, rounding), max=limit)
    u = torch.clamp(_r(h @ W[p + ".up"].T, rounding), -limit, limit)
    y = _r(g * torch.sigmoid(1.702 * g) * (u + 1.0), rounding)
    return _r(y @ W[p + ".down"].T, rounding)


def route(z: torch.Tensor, router: Mapping, margins_out: Optional[list] = None):
    """``z [n, E]`` logits -> ``(chosen [n, top], weights [n, top])``.  ``margins_out`` receives, per token, how far
    the choice was from another one: the gap between the last group kept and the first one left out, and between
    the last expert chosen and the first one left out among those that could be chosen."""
    E, top = router["experts"], router["top"]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    s = torch.sigmoid(z)
    per = E // groups["count"]
    allowed = torch.ones_like(s, dtype=torch.bool)
    if groups["count"] > 1:
        gs = s.view(-1, groups["count"], per)
        score = gs.topk(min(2, per), dim=-1).values.sum(-1)                 # [n, groups]
        best = score.topk(groups["keep"], dim=-1).indices
        keep = torch.zeros_like(score, dtype=torch.bool).scatter_(1, best, True)
        allowed = keep[:, :, None].expand(-1, -1, per).reshape(s.shape)
        if margins_out is not None and groups["keep"] < groups["count"]:
            ordered = score.sort(-1, descending=True).values
            margins_out.append(ordered[:, groups["keep"] - 1] - ordered[:, groups["keep"]])
    open_scores = s.masked_fill(~allowed, float("-inf"))
    if margins_out is not None and top < int(allowed[0].sum()):
        ordered = open_scores.sort(-1, descending=True).values
        margins_out.append(ordered[:, top - 1] - ordered[:, top])
    chosen = open_scores.topk(top, dim=-1).indices
    w = s.gather(1, chosen)
    w = w / (w.sum(-1, keepdim=True) + 1e-20) * router["scale"]
    return chosen, w


def experts_ffn(h, W, p: str, mlp: Mapping, rounding, margins_out: Optional[list] = None) -> torch.Tensor:
    n = h.shape[0]
    router = mlp["router"]
    hr = h if rounding is None else h.to(rounding).to(F64)
    z = hr @ W[p + ".router"].T
    chosen, w = route(z, router, margins_out)
    out = torch.zeros(n, h.shape[1], dtype=F64)
    for e in range(router["experts"]):
        rows, slot = (chosen == e).nonzero(as_tuple=True)
        if rows.numel():
            out[rows] += w[rows, slot][:, None] * bounded_expert(h[rows], W, f"{p}.e{e}", mlp["expert"]["limit"], rounding)
    if mlp.get("shared"):
        out = out + bounded_expert(h, W, p + ".shared", mlp["shared"]["limit"], rounding)
    return _r(out, rounding)


def run_order(config: Mapping) -> List[tuple]:
    """``(layer, pass number or None)`` of every layer run, in order."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop or loop["times"] < 1 or loop["stop"] <= loop["start"]:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, None) for i in range(loop["stop"], n)]


def forward(config: Mapping, W: Mapping[str, torch.Tensor], tokens, rounding=None, layers_out: Optional[list] = None,
            margins_out: Optional[list] = None, mixer_hook=None) -> torch.Tensor:
    """Logits ``[n, vocab]`` (float64) of one whole sequence.  ``layers_out`` receives the stream after every layer
    run, ``margins_out`` the routers' margins (see :func:`route`); ``mixer_hook(run, y)`` may replace a mixer's result."""
    W = {k: v.to(F64) for k, v in W.items()}
    eps = config["norm"]["eps"]
    x0 = W["embed"][torch.as_tensor(tokens, dtype=torch.long)] * config["embedding"]["scale"]
    x = x0.clone()
    loop = config.get("loop")
    for i, t in run_order(config):
        if t is not None and i == loop["start"]:
            if t > 0:
                x = x + x0
            x = x + W["loop.step"][t]
        layer, p = config["layers"][i], f"l{i}"
        h = _r(rms(x, eps) * W[p + ".norm1"], rounding)
        if layer["type"] == "mamba1":
            y = selective_scan_mixer(h, W, p + ".mix", layer["mixer"], rounding)
        elif layer["type"] == "latent_attention":
            y = latent_attention(h, W, p + ".mix", layer["mixer"], eps, rounding)
        else:
            y = sink_attention(h, W, p + ".mix", layer["mixer"], rounding)
        x = x + rms(y, eps) * W[p + ".norm1b"]
        mlp = layer.get("mlp")
        if mlp is not None:
            h = _r(rms(x, eps) * W[p + ".norm2"], rounding)
            y = dense_ffn(h, W, p + ".mlp", rounding) if mlp["kind"] == "dense" \
                else experts_ffn(h, W, p + ".mlp", mlp, rounding, margins_out)
            x = x + rms(y, eps) * W[p + ".norm2b"]
        if layers_out is not None:
            layers_out.append(x.clone())
    h = _r(rms(x, eps) * W["final.norm"], rounding)
    return h @ W["embed"].T
