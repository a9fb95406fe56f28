"""Small Nunosun configurations with random weights for the tests, and the two ways of running
them: the plain implementation (``plain_nunosun``) and the engine, either over the CUDA kernels
or, without a GPU, over their plain PyTorch twins (``torch_ops.TorchOps``), which still exercises
the package's parts, cache manager, step function and scheduler.

The configurations differ from each other in every size, so that nothing can lean on two numbers
being equal: grouped and ungrouped heads, key and value sizes that differ, windows shorter and
longer than a page, tables of distances of several lengths, rotations over a part of a head and
over all of it, a decay of one, convolutions of one tap and of several, layers without a
feed-forward, one expert per token and several.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, List, Optional

import numpy as np
import torch

import plain_nunosun as plain
from nagolix_cases import BACKENDS, feed, make_replayer, stored_dtype, tokens_for  # noqa: F401  (generic helpers)


def parallel_layer(heads=4, kv_heads=2, dim=16, vdim=24, window=7, bias_max=20.0, scale=None, r_heads=3, r_dim=8, r_vdim=12,
                   decay=(0.9, 0.97, 1.0), rot_dims=4, base=10000.0, mlp=None, bias_rows=6):
    left = {"bias_max": bias_max, "dim": dim, "heads": heads, "kv_heads": kv_heads, "mask": {"size": window},
            "scale": scale or dim ** -0.5, "vdim": vdim}
    right = {"decay": list(decay), "dim": r_dim, "heads": r_heads, "rot": {"base": base, "dims": rot_dims}, "vdim": r_vdim}
    return {"mixer": {"left": left, "right": right}, "mlp": mlp, "type": "parallel", "_bias_rows": bias_rows}


def delta_layer(heads=4, kv_heads=2, dim=12, vdim=20, conv=3, mlp=None):
    return {"mixer": {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim}, "mlp": mlp, "type": "delta"}


def dense(ff=80):
    return {"ff": ff, "kind": "dense"}


def moe(experts=6, top=2, ff=24):
    return {"expert": {"ff": ff}, "kind": "moe", "router": {"experts": experts, "top": top}}


def config(layers, width=48, vocab=89, eps=1e-5, taps=3, side=5, logit_scale=0.7):
    return {"architecture": "Nunosun", "canon": {"taps": taps}, "layers": layers, "logit_scale": logit_scale,
            "norm": {"eps": eps}, "token_side": {"dim": side}, "vocab": vocab, "width": width}


def clean(cfg: dict) -> dict:
    """The configuration as a file carries it (without the tests' own notes)."""
    out = dict(cfg)
    out["layers"] = [{k: v for k, v in layer.items() if not k.startswith("_")} for layer in cfg["layers"]]
    return out


# name -> (config, page size)
CASES = {
    # every kind of layer and feed-forward, sizes all different
    "mixed": (config([
        parallel_layer(mlp=dense(80)),
        delta_layer(mlp=moe(6, 2, 24)),
        parallel_layer(heads=2, kv_heads=1, dim=8, vdim=16, window=19, bias_max=64.0, r_heads=2, r_dim=12, r_vdim=8,
                       decay=(0.95, 0.999), rot_dims=12, base=300.0, mlp=None, bias_rows=10),
        delta_layer(heads=2, kv_heads=2, dim=8, vdim=12, conv=4, mlp=dense(56)),
    ], width=48, vocab=89), 8),
    # awkward sizes: a width that is no multiple of 8, one key/value head per head, a window of two, a convolution
    # of one tap in front of the mixers and of one tap inside the delta rule, one expert per token, a decay of one,
    # sizes that are no multiples of four, a scale of one on the logits
    "awkward": (config([
        delta_layer(heads=3, kv_heads=1, dim=10, vdim=6, conv=1, mlp=moe(7, 1, 20)),
        parallel_layer(heads=3, kv_heads=3, dim=12, vdim=10, window=2, bias_max=9.0, r_heads=1, r_dim=6, r_vdim=14, decay=(1.0,),
                       rot_dims=2, base=50.0, mlp=dense(50), bias_rows=4),
        delta_layer(heads=2, kv_heads=1, dim=6, vdim=10, conv=2, mlp=None),
    ], width=44, vocab=61, eps=1e-4, taps=1, side=3, logit_scale=1.0), 4),
    # sizes the tensor-core kernels take, windows and prompts longer than pages and than the kernels' chunks
    "wide": (config([
        parallel_layer(heads=4, kv_heads=1, dim=64, vdim=128, window=48, bias_max=200.0, r_heads=2, r_dim=128, r_vdim=64,
                       decay=(0.98, 0.995), rot_dims=64, base=250000.0, mlp=moe(8, 2, 96), bias_rows=16),
        delta_layer(heads=4, kv_heads=2, dim=64, vdim=64, conv=4, mlp=dense(384)),
        parallel_layer(heads=4, kv_heads=2, dim=32, vdim=64, window=100, bias_max=150.0, r_heads=4, r_dim=32, r_vdim=32,
                       decay=(0.9, 0.95, 0.99, 0.999), rot_dims=16, base=1000.0, mlp=dense(192), bias_rows=32),
    ], width=256, vocab=211, taps=4, side=16), 16),
}


def tensors_for(cfg: dict, seed: int, sharp: float = 1.0) -> Dict[str, torch.Tensor]:
    """Random float32 tensors under the checkpoint's names.  ``sharp`` scales the query and key
    sides and the router, so that attention and routing are peaked and a single wrong key or
    expert moves the logits."""
    g = torch.Generator().manual_seed(seed)
    d, s, n_layers = cfg["width"], cfg["token_side"]["dim"], len(cfg["layers"])

    def mat(rows, cols, gain=1.0):
        return torch.randn(rows, cols, generator=g) * (gain / cols ** 0.5)

    def vec(n, centre=0.0, spread=0.1):
        return centre + spread * torch.randn(n, generator=g)

    out = {"embed": torch.randn(cfg["vocab"], d, generator=g), "embed.norm": vec(d, 1.0), "final.norm": vec(d, 1.0),
           "head": mat(cfg["vocab"], d), "side.embed": torch.randn(cfg["vocab"], s * n_layers, generator=g)}
    for i, layer in enumerate(cfg["layers"]):
        m, mlp, p = layer["mixer"], layer["mlp"], f"l{i}."
        out[p + "norm1"] = vec(d, 1.0)
        out[p + "canon1"] = 0.3 * torch.randn(d, cfg["canon"]["taps"], generator=g)
        out[p + "side.gate"], out[p + "side.proj"], out[p + "side.norm"] = mat(s, d, 2.0), mat(d, s), vec(d, 0.3, 0.05)
        if layer["type"] == "parallel":
            a, r = m["left"], m["right"]
            H, G, dk, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            out[p + "mix.left.q"], out[p + "mix.left.k"], out[p + "mix.left.v"] = mat(H * dk, d), mat(G * dk, d), mat(G * dv, d)
            out[p + "mix.left.q.norm"], out[p + "mix.left.k.norm"] = vec(dk, 1.0 * sharp), vec(dk, 1.0 * sharp)
            out[p + "mix.left.rel"] = torch.randn(layer.get("_bias_rows", 6), H, generator=g)
            out[p + "mix.left.o"] = mat(d, H * dv)
            rh, rk, rv = r["heads"], r["dim"], r["vdim"]
            out[p + "mix.right.q"], out[p + "mix.right.k"] = mat(rh * rk, d, 2.0), mat(rh * rk, d, 2.0)
            out[p + "mix.right.v"], out[p + "mix.right.g"], out[p + "mix.right.o"] = mat(rh * rv, d), mat(rh * rv, d, 2.0), mat(d, rh * rv)
            out[p + "mix.left.out"], out[p + "mix.right.out"] = vec(d, 1.0), vec(d, 0.8)
        else:
            H, G, dk, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            for name, rows in (("q", G * dk), ("k", G * dk), ("v", H * dv)):
                out[p + f"mix.{name}"] = mat(rows, d, 2.0)
                out[p + f"mix.{name}.conv"] = 0.5 * torch.randn(rows, taps, generator=g)
            out[p + "mix.b"], out[p + "mix.a"] = mat(H, d, 2.0), mat(H, d, 2.0)
            out[p + "mix.A_log"], out[p + "mix.dt_bias"] = vec(H, -1.0, 0.5), vec(H, 0.0, 0.5)
            out[p + "mix.norm"] = vec(dv, 1.0)
            out[p + "mix.g"], out[p + "mix.o"] = mat(H * dv, d, 2.0), mat(d, H * dv)
        if mlp is not None and mlp["kind"] == "dense":
            out[p + "mlp.up"], out[p + "mlp.down"] = mat(mlp["ff"], d, 2.0), mat(d, mlp["ff"])
            out[p + "mlp.act"] = torch.tensor([1.0, 0.5, 0.25, 0.1]) + 0.1 * torch.randn(4, generator=g)
        elif mlp is not None:
            r, ff = mlp["router"], mlp["expert"]["ff"]
            for e in range(r["experts"]):
                out[p + f"mlp.e{e}.gate"], out[p + f"mlp.e{e}.up"] = mat(ff, d, 2.0), mat(ff, d, 2.0)
                out[p + f"mlp.e{e}.down"] = mat(d, ff)
            out[p + "mlp.router"] = mat(r["experts"], d, 6.0)      # decisive whatever the dtype: see clear_tokens
            out[p + "mlp.router.b"] = vec(r["experts"], 0.0, 0.5)
    return out


def write_folder(tmp, name: str, cfg: dict, tensors: Dict[str, torch.Tensor], dtype=torch.float32) -> Path:
    from safetensors.torch import save_file
    folder = Path(tmp) / f"nunosun_{name}"
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(clean(cfg)))
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
    """Random tokens on which no router of the model has a close call: everywhere the last chosen
    expert's logit stands above the first one left out by a margin (0.3 for bfloat16, where the
    rows that the router reads carry the rounding of everything before them; 1e-3 for float32).
    A choice that rounding flips would move that row's logits, and through the states all later
    rows', by far more than rounding does.  The sequence is grown eight tokens at a time, a block
    being drawn again until its own positions are clear (the model is causal)."""
    if not any(l["mlp"] is not None and l["mlp"]["kind"] == "moe" for l in cfg["layers"]):
        return np.random.default_rng(1000 + seed).integers(0, cfg["vocab"], size=n).tolist()
    margin = 0.3 if dtype == "bfloat16" else 1e-3
    rng = np.random.default_rng(1000 + seed)
    tokens: List[int] = []
    while len(tokens) < n:
        k = min(8, n - len(tokens))
        for _ in range(200):
            block = rng.integers(0, cfg["vocab"], size=k).tolist()
            routers: list = []
            plain.forward(cfg, tensors, tokens + block, routers_out=routers)
            worst = np.inf
            for z, idx in routers:
                top = idx.shape[1]
                if top < z.shape[1]:
                    ordered = z[len(tokens):].sort(-1, descending=True).values
                    worst = min(worst, float((ordered[:, top - 1] - ordered[:, top]).min()))
            if worst >= margin:
                break
        else:
            raise AssertionError("no tokens with clear routing found: make the router sharper")
        tokens += block
    return tokens


class Expected:
    """The plain logits of a sequence and how far an engine may be from them.  In float32: 5e-5 of
    the largest logit on every logit (2e-4 at least).  In bfloat16 the yardstick is what rounding
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
            limit = 5e-5 * max(4.0, float(np.abs(self.logits).max()))
            assert err <= limit, f"{what}: logits differ by {err} (allowed {limit})"
        else:
            err = np.sqrt(((got - self.logits) ** 2).mean(-1))
            worst = int(np.argmax(err / self.allowed))
            assert err[worst] <= 1.5 * self.allowed[worst], \
                f"{what}: row {worst} differs by {err[worst]} (rms), rounding alone allows {self.allowed[worst]}"
            assert (err > self.allowed).mean() <= 0.05, f"{what}: {(err > self.allowed).sum()} of {len(err)} rows over their allowance"


def plain_logits(cfg, tensors, tokens, dtype: str) -> Expected:
    return Expected(cfg, tensors, tokens, dtype)
