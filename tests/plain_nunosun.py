"""Nunosun written out from its equations: whole sequences, float64, one function per mechanism.

Slow and plain on purpose: explicit ``[n, n]`` score matrices, token-by-token recurrences, Python
loops over heads and experts.  It reads the design's ``config.json`` dictionary itself and takes
the checkpoint's tensors by their stored names; nothing of the package is imported, so the engine
and this file can only agree by computing the same design.

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


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def causal_conv(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``y[t, c] = sum_j w[c, j] * x[t - taps + 1 + j, c]`` with zeros before the start."""
    n, taps = x.shape[0], w.shape[1]
    y = torch.zeros_like(x)
    for j in range(taps):
        back = taps - 1 - j
        if back < n:
            y[back:] += x[:n - back] * w[:, j]
    return y


def distance_row(n: int, rows: int, far: float) -> int:
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def windowed_attention(h, W: Mapping[str, torch.Tensor], p: str, cfg: Mapping, eps: float, rounding) -> torch.Tensor:
    n = h.shape[0]
    H, G, d, dv = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    q = _r(h @ W[p + ".q"].T, rounding).view(n, H, d)
    k = _r(h @ W[p + ".k"].T, rounding).view(n, G, d)
    v = _r(h @ W[p + ".v"].T, rounding).view(n, G, dv)
    q = _r(rms(q, eps) * W[p + ".q.norm"], rounding)
    k = _r(rms(k, eps) * W[p + ".k.norm"], rounding)
    rel = W[p + ".rel"]
    rows = rel.shape[0]
    dist = torch.arange(n)[:, None] - torch.arange(n)[None, :]
    seen = (dist >= 0) & (dist < cfg["mask"]["size"])
    row_of = torch.tensor([[distance_row(int(x), rows, cfg["bias_max"]) if x >= 0 else 0 for x in r] for r in dist.tolist()])
    out = torch.zeros(n, H, dv, dtype=F64)
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * cfg["scale"] + rel[row_of, a]
        s = s.masked_fill(~seen, float("-inf"))
        out[:, a] = torch.softmax(s, dim=-1) @ v[:, g]
    return _r(_r(out.reshape(n, H * dv), rounding) @ W[p + ".o"].T, rounding)


def rotate_half(x: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """``x [n, heads, d]``: the first ``dims`` coordinates of every head turned by the position's angles."""
    n = x.shape[0]
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    a = torch.arange(n, dtype=F64)[:, None] * f[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def retention(h, W, p: str, cfg: Mapping, eps: float, rounding) -> torch.Tensor:
    n = h.shape[0]
    H, d, dv = cfg["heads"], cfg["dim"], cfg["vdim"]
    q = _r(h @ W[p + ".q"].T, rounding).view(n, H, d)
    k = _r(h @ W[p + ".k"].T, rounding).view(n, H, d)
    v = _r(h @ W[p + ".v"].T, rounding).view(n, H, dv)
    q = rotate_half(q, cfg["rot"]["dims"], cfg["rot"]["base"])
    k = rotate_half(k, cfg["rot"]["dims"], cfg["rot"]["base"]) * d ** -0.5
    out = torch.zeros(n, H, dv, dtype=F64)
    for a in range(H):
        S = torch.zeros(d, dv, dtype=F64)
        for t in range(n):
            S = cfg["decay"][a] * S + torch.outer(k[t, a], v[t, a])
            out[t, a] = S.T @ q[t, a]
    out = rms(out, eps).reshape(n, H * dv)
    gate = silu(_r(h @ W[p + ".g"].T, rounding))
    return _r(_r(out * gate, rounding) @ W[p + ".o"].T, rounding)


def parallel_mixer(h, W, p: str, cfg: Mapping, eps: float, rounding) -> torch.Tensor:
    left = windowed_attention(h, W, p + ".left", cfg["left"], eps, rounding)
    right = retention(h, W, p + ".right", cfg["right"], eps, rounding)
    return 0.5 * (rms(left, eps) * W[p + ".left.out"] + rms(right, eps) * W[p + ".right.out"])


def delta_mixer(h, W, p: str, cfg: Mapping, eps: float, rounding) -> torch.Tensor:
    n = h.shape[0]
    H, G, d, dv = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]

    def branch(name):
        y = _r(h @ W[f"{p}.{name}"].T, rounding)
        return _r(silu(_r(causal_conv(y, W[f"{p}.{name}.conv"]), rounding)), rounding)

    q, k, v = branch("q").view(n, G, d), branch("k").view(n, G, d), branch("v").view(n, H, dv)
    q = q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(_r(h @ W[p + ".b"].T, rounding))
    decay = torch.exp(-torch.exp(W[p + ".A_log"]) * torch.nn.functional.softplus(_r(h @ W[p + ".a"].T, rounding) + W[p + ".dt_bias"]))
    out = torch.zeros(n, H, dv, dtype=F64)
    for a in range(H):
        g = a // (H // G)
        S = torch.zeros(d, dv, dtype=F64)
        for t in range(n):
            S = decay[t, a] * S
            u = beta[t, a] * (v[t, a] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            out[t, a] = S.T @ q[t, g]
    out = (rms(out, eps) * W[p + ".norm"]).reshape(n, H * dv)
    gate = silu(_r(h @ W[p + ".g"].T, rounding))
    return _r(_r(out * gate, rounding) @ W[p + ".o"].T, rounding)


def polynorm_ff(h, W, p: str, eps: float, rounding) -> torch.Tensor:
    z = _r(h @ W[p + ".up"].T, rounding)
    a, b, c, e = W[p + ".act"].tolist()
    act = a * rms(z, eps) + b * rms(z ** 2, eps) + c * rms(z ** 3, eps) + e
    return _r(_r(act, rounding) @ W[p + ".down"].T, rounding)


def experts_ff(h, W, p: str, cfg: Mapping, rounding, chosen_out: Optional[List] = None) -> torch.Tensor:
    n = h.shape[0]
    E, top = cfg["router"]["experts"], cfg["router"]["top"]
    z = h @ W[p + ".router"].T + W[p + ".router.b"]
    val, idx = torch.topk(z, top, dim=-1)
    wgt = torch.softmax(val, dim=-1)
    if chosen_out is not None:
        chosen_out.append((z, idx))
    out = torch.zeros(n, h.shape[1], dtype=F64)
    for e in range(E):
        hit = idx == e
        rows = hit.any(-1).nonzero().flatten()
        if rows.numel() == 0:
            continue
        x = h[rows]
        u = _r(silu(_r(x @ W[f"{p}.e{e}.gate"].T, rounding)) * _r(x @ W[f"{p}.e{e}.up"].T, rounding), rounding)
        y = _r(u @ W[f"{p}.e{e}.down"].T, rounding)
        out[rows] += y * (wgt[rows] * hit[rows]).sum(-1, keepdim=True)
    return out


def side_input(x, tokens, W, p: str, layer: int, dim: int, eps: float, rounding) -> torch.Tensor:
    e = W["side.embed"][tokens][:, layer * dim:(layer + 1) * dim]
    g = _r(gelu_tanh(_r(_r(x, rounding) @ W[p + ".side.gate"].T, rounding)) * e, rounding)
    y = _r(g @ W[p + ".side.proj"].T, rounding)
    return rms(y, eps) * W[p + ".side.norm"]


def forward(config: Mapping, tensors: Mapping[str, torch.Tensor], tokens, rounding=None, layers_out: Optional[List] = None,
            routers_out: Optional[List] = None) -> torch.Tensor:
    """Logits ``[n, vocab]`` (float64) of one whole sequence."""
    W: Dict[str, torch.Tensor] = {k: v.to(F64) for k, v in tensors.items() if v.is_floating_point()}
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    eps = config["norm"]["eps"]
    x = rms(W["embed"][tokens], eps) * W["embed.norm"]
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}"
        h = _r(rms(x, eps) * W[p + ".norm1"], rounding)
        hm = _r(h + causal_conv(h, W[p + ".canon1"]), rounding)
        if layer["type"] == "parallel":
            y = parallel_mixer(hm, W, p + ".mix", layer["mixer"], eps, rounding)
        elif layer["type"] == "delta":
            y = delta_mixer(hm, W, p + ".mix", layer["mixer"], eps, rounding)
        else:
            raise ValueError(layer["type"])
        mlp = layer.get("mlp")
        if mlp is not None:
            if mlp["kind"] == "dense":
                y = y + polynorm_ff(h, W, p + ".mlp", eps, rounding)
            else:
                y = y + experts_ff(h, W, p + ".mlp", mlp, rounding, routers_out)
        x = x + y
        x = x + side_input(x, tokens, W, p, i, config["token_side"]["dim"], eps, rounding)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = _r(rms(x, eps) * W["final.norm"], rounding)
    return (x @ W["head"].T) * config["logit_scale"]
