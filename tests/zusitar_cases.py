"""Small Zusitar configurations with random weights for the tests, and the two ways of running
them: the plain implementation (``plain_zusitar``) and the engine, either over the CUDA kernels
or, without a GPU, over their plain PyTorch twins (``torch_ops.TorchOps``), which still exercises
the package's parts, cache manager, step function and scheduler.

The configurations differ from each other in every size, so that nothing can lean on two numbers
being equal or one: grouped and ungrouped heads, key and value sizes that differ, query and
key/value latents of different sizes, rotations over a part of a head, over all of it and over
none, state sizes that are no multiples of four, convolutions of one tap and of several, a step
rank of one, one group of experts and several, one expert per token and several, layers without
a feed-forward, loops over some layers, over all of them, once, three times, and no loop.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, List, Optional

import numpy as np
import torch

import plain_zusitar as plain
from nagolix_cases import BACKENDS, feed, make_replayer, stored_dtype, tokens_for  # noqa: F401  (generic helpers)


def scan_layer(inner=40, state=6, dt_rank=3, conv=3, mlp=None):
    return {"mixer": {"conv": conv, "dt_rank": dt_rank, "inner": inner, "state": state}, "mlp": mlp, "type": "mamba1"}


def latent_layer(heads=3, dim=8, rot_dim=4, vdim=12, q_rank=20, kv_rank=16, base=10000.0, scale=None, mlp=None):
    return {"mixer": {"dim": dim, "heads": heads, "kv_rank": kv_rank, "q_rank": q_rank, "rot": {"base": base, "dims": rot_dim},
                      "rot_dim": rot_dim, "scale": scale or (dim + rot_dim) ** -0.5, "vdim": vdim}, "mlp": mlp,
            "type": "latent_attention"}


def attention_layer(heads=4, kv_heads=2, dim=16, vdim=24, rot_dims=8, base=10000.0, softcap=20.0, scale=None, mlp=None):
    return {"mixer": {"dim": dim, "heads": heads, "kv_heads": kv_heads, "rot": {"base": base, "dims": rot_dims},
                      "scale": scale or dim ** -0.5, "softcap": softcap, "vdim": vdim}, "mlp": mlp, "type": "attention"}


def dense(ff=80):
    return {"ff": ff, "kind": "dense"}


def moe(experts=6, top=2, ff=24, limit=2.0, groups=(3, 2), scale=1.3, shared=(20, 1.2)):
    out = {"expert": {"ff": ff, "limit": limit}, "kind": "moe",
           "router": {"experts": experts, "groups": {"count": groups[0], "keep": groups[1]}, "scale": scale, "top": top}}
    if shared:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def config(layers, width=48, vocab=89, eps=1e-5, scale=3.0, loop=None):
    out = {"architecture": "Zusitar", "embedding": {"scale": scale}, "layers": layers, "norm": {"eps": eps}, "vocab": vocab,
           "width": width}
    if loop:
        out["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return out


# name -> (config, page size)
CASES = {
    # every kind of layer and feed-forward, sizes all different, the middle layers run three times
    "mixed": (config([
        scan_layer(mlp=dense(80)),
        latent_layer(mlp=moe(6, 2, 24)),
        attention_layer(mlp=moe(8, 3, 16, limit=1.0, groups=(2, 1), scale=0.8, shared=None)),
        scan_layer(inner=24, state=9, dt_rank=5, conv=4, mlp=None),
        latent_layer(heads=2, dim=12, rot_dim=8, vdim=8, q_rank=12, kv_rank=24, base=300.0, mlp=dense(56)),
    ], width=48, vocab=89, loop=(1, 4, 3)), 8),
    # awkward sizes: a width that is no multiple of 8, one key/value head per head, a rotation over the whole head and
    # over none of it, a convolution of one tap, a step rank of one, a state of one number, one group that holds all
    # experts, one expert per token, every layer in the loop, which runs once, an embedding scale of one
    "awkward": (config([
        attention_layer(heads=3, kv_heads=3, dim=10, vdim=6, rot_dims=10, base=50.0, softcap=5.0, mlp=moe(7, 1, 20, groups=(1, 1))),
        scan_layer(inner=18, state=1, dt_rank=1, conv=1, mlp=dense(50)),
        latent_layer(heads=1, dim=6, rot_dim=2, vdim=14, q_rank=7, kv_rank=10, base=7.0, mlp=None),
        attention_layer(heads=2, kv_heads=1, dim=12, vdim=12, rot_dims=0, softcap=50.0, mlp=moe(4, 2, 12, groups=(4, 3), shared=(6, 0.5))),
    ], width=44, vocab=61, eps=1e-4, scale=1.0, loop=(0, 4, 1)), 4),
    # sizes the tensor-core kernels take, prompts longer than pages and than the kernels' chunks; no loop
    "wide": (config([
        latent_layer(heads=4, dim=64, rot_dim=32, vdim=64, q_rank=96, kv_rank=96, base=250000.0, mlp=moe(8, 2, 96, groups=(4, 2))),
        scan_layer(inner=512, state=16, dt_rank=16, conv=4, mlp=dense(384)),
        attention_layer(heads=4, kv_heads=2, dim=64, vdim=128, rot_dims=32, base=1000.0, softcap=30.0, mlp=dense(192)),
    ], width=256, vocab=211, scale=16.0), 16),
}


def tensors_for(cfg: dict, seed: int, sharp: float = 1.0) -> Dict[str, torch.Tensor]:
    """Random float32 tensors under the checkpoint's names.  ``sharp`` scales the query sides and the
    router, so that attention and routing are peaked and a single wrong key or expert moves the logits."""
    g = torch.Generator().manual_seed(seed)
    d = cfg["width"]

    def mat(rows, cols, gain=1.0):
        return torch.randn(rows, cols, generator=g) * (gain / cols ** 0.5)

    def vec(n, centre=0.0, spread=0.1):
        return centre + spread * torch.randn(n, generator=g)

    out = {"embed": torch.randn(cfg["vocab"], d, generator=g) / d ** 0.5, "final.norm": vec(d, 1.0)}
    loop = cfg.get("loop")
    if loop:
        out["loop.step"] = 0.5 * torch.randn(loop["times"], d, generator=g)
    for i, layer in enumerate(cfg["layers"]):
        m, mlp, p = layer["mixer"], layer["mlp"], f"l{i}."
        for n in ("norm1", "norm1b") + (("norm2", "norm2b") if mlp is not None else ()):
            out[p + n] = vec(d, 1.0)
        if layer["type"] == "mamba1":
            c, n, r, taps = m["inner"], m["state"], m["dt_rank"], m["conv"]
            out[p + "mix.in"] = mat(2 * c, d, 2.0)
            out[p + "mix.conv"], out[p + "mix.conv.b"] = 0.5 * torch.randn(c, taps, generator=g), vec(c, 0.0, 0.2)
            out[p + "mix.x"] = mat(r + 2 * n, c, 2.0)
            out[p + "mix.dt"], out[p + "mix.dt.b"] = mat(c, r, 1.0), vec(c, -1.5, 0.7)
            out[p + "mix.A_log"] = torch.log(torch.arange(1, n + 1).float()).expand(c, n) + 0.3 * torch.randn(c, n, generator=g) - 1.0
            out[p + "mix.D"] = vec(c, 1.0)
            out[p + "mix.o"] = mat(d, c)
        elif layer["type"] == "latent_attention":
            H, dk, dr, dv, qr, kr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"], m["kv_rank"]
            out[p + "mix.dq"], out[p + "mix.dq.norm"] = mat(qr, d), vec(qr, 1.0 * sharp)
            out[p + "mix.uq"] = mat(H * (dk + dr), qr, 1.5)
            out[p + "mix.dkv"], out[p + "mix.dkv.norm"] = mat(kr + dr, d, 1.5), vec(kr, 1.0)
            out[p + "mix.uk"], out[p + "mix.uv"] = mat(H * dk, kr, 1.5), mat(H * dv, kr)
            out[p + "mix.g"], out[p + "mix.o"] = mat(H * dv, d, 2.0), mat(d, H * dv)
        else:
            H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out[p + "mix.q"], out[p + "mix.q.b"] = mat(H * dk, d, 1.5 * sharp), vec(H * dk, 0.0, 0.3)
            out[p + "mix.k"], out[p + "mix.k.b"] = mat(G * dk, d, 1.5), vec(G * dk, 0.0, 0.3)
            out[p + "mix.v"], out[p + "mix.v.b"] = mat(G * dv, d), vec(G * dv, 0.0, 0.3)
            out[p + "mix.sink"] = vec(H, 0.5, 1.0)
            out[p + "mix.g"] = mat(H, d, 2.0)
            out[p + "mix.o"], out[p + "mix.o.b"] = mat(d, H * dv), vec(d, 0.0, 0.3)
        if mlp is not None and mlp["kind"] == "dense":
            out[p + "mlp.gate"], out[p + "mlp.up"], out[p + "mlp.down"] = mat(mlp["ff"], d, 2.0), mat(mlp["ff"], d, 2.0), mat(d, mlp["ff"])
        elif mlp is not None:
            r, ff = mlp["router"], mlp["expert"]["ff"]
            for e in range(r["experts"]):
                out[p + f"mlp.e{e}.gate"], out[p + f"mlp.e{e}.up"] = mat(ff, d, 3.0), mat(ff, d, 3.0)      # (large enough to meet the bounds)
                out[p + f"mlp.e{e}.down"] = mat(d, ff)
            out[p + "mlp.router"] = mat(r["experts"], d, 1.5)      # logits of order one: sigmoid scores that do not crowd at 0 and 1
            if mlp.get("shared"):
                sf = mlp["shared"]["ff"]
                out[p + "mlp.shared.gate"], out[p + "mlp.shared.up"] = mat(sf, d, 3.0), mat(sf, d, 3.0)
                out[p + "mlp.shared.down"] = mat(d, sf)
    return out


def write_folder(tmp, name: str, cfg: dict, tensors: Dict[str, torch.Tensor], dtype=torch.float32) -> Path:
    from safetensors.torch import save_file
    folder = Path(tmp) / f"zusitar_{name}"
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.to(dtype).contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
    return folder


def stored(tensors: Dict[str, torch.Tensor], dtype) -> Dict[str, torch.Tensor]:
    """What the file stores is what both sides compute with."""
    return tensors if dtype == torch.float32 else {k: v.to(dtype).float() for k, v in tensors.items()}


def case_folder(tmp, name: str, sharp: Optional[float] = None, dtype=torch.float32):
    """In float32 the weights are sharp (peaked attention and routing: one wrong key or expert moves
    the logits far beyond the tolerance); in bfloat16 they are not, or rounding alone would
    scatter the logits."""
    cfg, page = CASES[name]
    if sharp is None:
        sharp = 3.0 if dtype == torch.float32 else 1.0
    tensors = stored(tensors_for(cfg, seed=sum(map(ord, name)), sharp=sharp), dtype)
    return cfg, tensors, write_folder(tmp, name, cfg, tensors, dtype), page


def clear_tokens(cfg: dict, tensors, n: int, seed: int = 0, dtype: str = "bfloat16") -> List[int]:
    """Random tokens on which no router of the model has a close call: everywhere the last group kept
    and the last expert chosen stand above the first ones left out by a margin in score (0.04 for
    bfloat16, where the rows that the router reads carry the rounding of everything before them;
    1e-4 for float32).  A choice that rounding flips would move that row's logits, and through the
    states all later rows', by far more than rounding does.  The sequence is grown two tokens at
    a time, a block being drawn again until its own positions are clear (the model is causal)."""
    if not any(l["mlp"] is not None and l["mlp"]["kind"] == "moe" for l in cfg["layers"]):
        return np.random.default_rng(1000 + seed).integers(0, cfg["vocab"], size=n).tolist()
    margin = 0.04 if dtype == "bfloat16" else 1e-4
    rng = np.random.default_rng(1000 + seed)
    tokens: List[int] = []
    while len(tokens) < n:
        k = min(2, n - len(tokens))
        for _ in range(400):
            block = rng.integers(0, cfg["vocab"], size=k).tolist()
            margins: list = []
            plain.forward(cfg, tensors, tokens + block, margins_out=margins)
            worst = min((float(m[len(tokens):].min()) for m in margins), default=np.inf)
            if worst >= margin:
                break
        else:
            raise AssertionError("no tokens with clear routing found: make the router sharper")
        tokens += block
    return tokens


class Expected:
    """The plain logits of a sequence and how far an engine may be from them.  In float32: 2.5e-4 of
    the largest logit on every logit (1e-3 at least: the sharp test models are up to eleven layer runs deep, and a wrong key, state or expert moves them by tenths).  In bfloat16 the yardstick is what rounding
    itself does to this model: the plain implementation is run a second time with bfloat16 rounding
    of every projection and activation, and a row of the engine's logits may differ from the exact
    ones (root mean square over the vocabulary) by three times what that emulation differs, the
    typical row's figure standing in where a row's own is smaller; one row in twenty may pass
    that, by half at most."""

    def __init__(self, cfg, tensors, tokens, dtype: str):
        self.dtype = dtype
        self.logits = plain.forward(cfg, tensors, tokens).to(torch.float32).numpy()
        if dtype == "bfloat16":
            rounded = plain.forward(cfg, tensors, tokens, rounding=torch.bfloat16).to(torch.float32).numpy()
            noise = np.sqrt(((rounded - self.logits) ** 2).mean(-1))
            self.allowed = 3.0 * np.maximum(noise, np.median(noise))

    def __getitem__(self, rows):
        return self.logits[rows]

    def check(self, got: np.ndarray, what: str = "") -> None:
        assert got.shape == self.logits.shape, f"{what}: {got.shape} logits for {self.logits.shape}"
        if self.dtype == "float32":
            err = np.abs(got - self.logits).max()
            limit = 2.5e-4 * max(4.0, float(np.abs(self.logits).max()))
            assert err <= limit, f"{what}: logits differ by {err} (allowed {limit})"
        else:
            err = np.sqrt(((got - self.logits) ** 2).mean(-1))
            worst = int(np.argmax(err / self.allowed))
            assert err[worst] <= 1.5 * self.allowed[worst], \
                f"{what}: row {worst} differs by {err[worst]} (rms), rounding alone allows {self.allowed[worst]}"
            assert (err > self.allowed).mean() <= 0.05, f"{what}: {(err > self.allowed).sum()} of {len(err)} rows over their allowance"


def plain_logits(cfg, tensors, tokens, dtype: str) -> Expected:
    return Expected(cfg, tensors, tokens, dtype)
