"""Nunosun as an :class:`~torchllms_b200.config.registry.Architecture`.

A small decoder whose ``config.json`` lists its layers one by one; every layer names its mixer
(``parallel`` or ``delta``) with that mixer's own sizes, and its feed-forward (``dense``, ``moe`` or
none).  What the design fixes and no file carries:

* the stream starts as the RMS norm of the embedding table's row; the head is a matrix of its own and
  its products leave multiplied by ``logit_scale``;
* a layer has one norm ``h = norm1(x)`` that both sublayers read, and one sum
  ``x += mixer(h + conv(h)) + ff(h)``, the convolution being causal over time per channel with
  ``canon.taps`` taps; then the layer's own slice of a per-token table enters:
  ``x += norm(W_proj (gelu_tanh(W_gate x) * table[token]))``;
* ``parallel``: sliding-window softmax attention (grouped key/value heads, RMS norm per head on q and
  k, no rotation, a learned bias by distance and head) beside a retention (fixed decay per head,
  rotary positions in the rotate-half layout, k scaled by ``dim^-1/2``, a weightless RMS norm per
  head, a ``silu`` gate); half the sum of the two results, each RMS-normed over the width;
* ``delta``: the gated delta rule over short convolutions of q, k and v with ``silu``, unit q and k,
  q scaled by ``dim^-1/2``, an RMS norm per head with one shared weight, a ``silu`` gate;
* ``dense``: ``down(PolyNorm(up x))``;  ``moe``: experts ``down(silu(gate x) * up x)``, router logits
  with a bias, the softmax taken over the chosen logits only.

This module only describes: it reads the configuration, names the generic parts with their numbers
(:func:`build_spec`), and maps the checkpoint's tensor names to the parts' own.
"""

from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Any, Dict, Iterator, Mapping, Optional, Tuple

import torch

from ..config.model_config import ConfigError, ModelConfig, require_key, typed_value
from ..config.registry import Architecture, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, RunEntry, part
from ..weights.loader import LazyTensor

NAME = "Nunosun"

# The design has no longest sequence (a window, recurrent states, a table of distances that ends in
# one last row); tables are made this long unless whoever builds the engine asks for more.
DEFAULT_MAX_POSITIONS = 32768

EXPERT_ACTIVATION = "silu"
UNIT_EPS = 1e-6                     # inside the root that makes q and k of the delta rule unit vectors


def _object(raw: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    value = raw.get(key)
    if not isinstance(value, Mapping):
        raise ConfigError(f"{where}: key '{key}' must be an object")
    return value


@dataclass(frozen=True)
class WindowAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int
    bias_max: float

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "WindowAttentionConfig":
        heads = require_key(raw, "heads", int, where)
        return cls(heads=heads, kv_heads=typed_value(raw.get("kv_heads", heads), "kv_heads", int, where),
                   dim=require_key(raw, "dim", int, where), vdim=require_key(raw, "vdim", int, where),
                   scale=require_key(raw, "scale", float, where),
                   window=require_key(_object(raw, "mask", where), "size", int, f"{where}.mask"),
                   bias_max=require_key(raw, "bias_max", float, where))

    def to_dict(self) -> Dict[str, Any]:
        return {"bias_max": self.bias_max, "dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads,
                "mask": {"size": self.window}, "scale": self.scale, "vdim": self.vdim}


@dataclass(frozen=True)
class RetentionConfig:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]
    rot_dims: int
    rot_base: float

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "RetentionConfig":
        rot = _object(raw, "rot", where)
        decay = raw.get("decay")
        if not isinstance(decay, (list, tuple)):
            raise ConfigError(f"{where}: key 'decay' must be a list with one number per head")
        return cls(heads=require_key(raw, "heads", int, where), dim=require_key(raw, "dim", int, where),
                   vdim=require_key(raw, "vdim", int, where),
                   decay=tuple(typed_value(x, "decay", float, where) for x in decay),
                   rot_dims=require_key(rot, "dims", int, f"{where}.rot"), rot_base=require_key(rot, "base", float, f"{where}.rot"))

    def to_dict(self) -> Dict[str, Any]:
        return {"decay": list(self.decay), "dim": self.dim, "heads": self.heads,
                "rot": {"base": self.rot_base, "dims": self.rot_dims}, "vdim": self.vdim}


@dataclass(frozen=True)
class ParallelConfig:
    left: WindowAttentionConfig
    right: RetentionConfig

    kind = "parallel"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "ParallelConfig":
        return cls(WindowAttentionConfig.from_dict(_object(raw, "left", where), f"{where}.left"),
                   RetentionConfig.from_dict(_object(raw, "right", where), f"{where}.right"))

    def to_dict(self) -> Dict[str, Any]:
        return {"left": self.left.to_dict(), "right": self.right.to_dict()}


@dataclass(frozen=True)
class DeltaConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    kind = "delta"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "DeltaConfig":
        heads = require_key(raw, "heads", int, where)
        return cls(heads=heads, kv_heads=typed_value(raw.get("kv_heads", heads), "kv_heads", int, where),
                   dim=require_key(raw, "dim", int, where), vdim=require_key(raw, "vdim", int, where),
                   conv=require_key(raw, "conv", int, where))

    def to_dict(self) -> Dict[str, Any]:
        return {"conv": self.conv, "dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "vdim": self.vdim}


@dataclass(frozen=True)
class MlpConfig:
    kind: str                       # "dense" or "moe"
    ff: int                         # dense: the hidden size; moe: one expert's
    experts: int = 0
    top: int = 0

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "MlpConfig":
        kind = require_key(raw, "kind", str, where)
        if kind == "dense":
            return cls(kind, require_key(raw, "ff", int, where))
        if kind == "moe":
            router = _object(raw, "router", where)
            return cls(kind, require_key(_object(raw, "expert", where), "ff", int, f"{where}.expert"),
                       experts=require_key(router, "experts", int, f"{where}.router"),
                       top=require_key(router, "top", int, f"{where}.router"))
        raise ConfigError(f"{where}: unknown feed-forward kind {kind!r}; known: dense, moe")

    def to_dict(self) -> Dict[str, Any]:
        if self.kind == "dense":
            return {"ff": self.ff, "kind": "dense"}
        return {"expert": {"ff": self.ff}, "kind": "moe", "router": {"experts": self.experts, "top": self.top}}


@dataclass(frozen=True)
class LayerConfig:
    mixer: Any                      # ParallelConfig or DeltaConfig
    mlp: Optional[MlpConfig]


_MIXERS = {"parallel": ParallelConfig, "delta": DeltaConfig}


@dataclass(frozen=True)
class NunosunConfig(ModelConfig):
    architecture: str
    vocab_size: int
    dim: int
    norm_eps: float
    conv_taps: int                  # taps of the convolution in front of every mixer
    side_dim: int                   # a layer's slice of the per-token table
    logit_scale: float
    layers: Tuple[LayerConfig, ...]
    max_seq_len: int = DEFAULT_MAX_POSITIONS

    @classmethod
    def from_json(cls, raw: Mapping[str, Any], where: str) -> "NunosunConfig":
        layers = raw.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError(f"{where}: key 'layers' must be a list with one object per layer")
        parsed = []
        for i, layer in enumerate(layers):
            at = f"{where}: layers[{i}]"
            if not isinstance(layer, Mapping):
                raise ConfigError(f"{at} must be an object")
            kind = require_key(layer, "type", str, at)
            if kind not in _MIXERS:
                raise ConfigError(f"{at}: unknown layer type {kind!r}; known: {', '.join(sorted(_MIXERS))}")
            mixer = _MIXERS[kind].from_dict(_object(layer, "mixer", at), f"{at}.mixer")
            mlp = layer.get("mlp")
            parsed.append(LayerConfig(mixer, None if mlp is None else MlpConfig.from_dict(mlp, f"{at}.mlp")))
        return cls(
            architecture=NAME,
            vocab_size=require_key(raw, "vocab", int, where),
            dim=require_key(raw, "width", int, where),
            norm_eps=require_key(_object(raw, "norm", where), "eps", float, f"{where}: norm"),
            conv_taps=require_key(_object(raw, "canon", where), "taps", int, f"{where}: canon"),
            side_dim=require_key(_object(raw, "token_side", where), "dim", int, f"{where}: token_side"),
            logit_scale=require_key(raw, "logit_scale", float, where),
            layers=tuple(parsed),
        ).validate(where)

    def validate(self, where: str = "config") -> "NunosunConfig":
        for key in ("vocab_size", "dim", "max_seq_len", "conv_taps", "side_dim"):
            if getattr(self, key) <= 0:
                raise ConfigError(f"{where}: '{key}' must be positive, got {getattr(self, key)}")
        for i, layer in enumerate(self.layers):
            m, at = layer.mixer, f"{where}: layers[{i}]"
            if m.kind == "parallel":
                a, r = m.left, m.right
                for key in ("heads", "kv_heads", "dim", "vdim", "window"):
                    if getattr(a, key) <= 0:
                        raise ConfigError(f"{at}: left '{key}' must be positive, got {getattr(a, key)}")
                if a.heads % a.kv_heads != 0:
                    raise ConfigError(f"{at}: left 'heads' ({a.heads}) must be a multiple of 'kv_heads' ({a.kv_heads})")
                for key in ("heads", "dim", "vdim"):
                    if getattr(r, key) <= 0:
                        raise ConfigError(f"{at}: right '{key}' must be positive, got {getattr(r, key)}")
                if len(r.decay) != r.heads:
                    raise ConfigError(f"{at}: right 'decay' must list one number per head ({r.heads}), got {len(r.decay)}")
                if r.rot_dims < 0 or r.rot_dims % 2 or r.rot_dims > r.dim or not r.rot_base > 0:
                    raise ConfigError(f"{at}: right 'rot.dims' must be even and at most 'dim' ({r.dim}), 'rot.base' positive")
            else:
                for key in ("heads", "kv_heads", "dim", "vdim", "conv"):
                    if getattr(m, key) <= 0:
                        raise ConfigError(f"{at}: mixer '{key}' must be positive, got {getattr(m, key)}")
                if m.heads % m.kv_heads != 0:
                    raise ConfigError(f"{at}: 'heads' ({m.heads}) must be a multiple of 'kv_heads' ({m.kv_heads})")
            mlp = layer.mlp
            if mlp is not None:
                if mlp.ff <= 0:
                    raise ConfigError(f"{at}: the feed-forward's 'ff' must be positive")
                if mlp.kind == "moe" and not 0 < mlp.top <= mlp.experts:
                    raise ConfigError(f"{at}: router 'top' must lie between 1 and 'experts' ({mlp.experts}), got {mlp.top}")
        return self

    def to_hf(self) -> Dict[str, Any]:
        return {
            "architecture": NAME,
            "canon": {"taps": self.conv_taps},
            "layers": [{"mixer": l.mixer.to_dict(), "mlp": None if l.mlp is None else l.mlp.to_dict(), "type": l.mixer.kind}
                       for l in self.layers],
            "logit_scale": self.logit_scale,
            "norm": {"eps": self.norm_eps},
            "token_side": {"dim": self.side_dim},
            "vocab": self.vocab_size,
            "width": self.dim,
        }


def parse_config(raw: Mapping[str, Any], source: str) -> NunosunConfig:
    return NunosunConfig.from_json(raw, source)


def build_spec(cfg: NunosunConfig) -> ModelSpec:
    norm = part("rmsnorm", dim=cfg.dim, eps=cfg.norm_eps)
    layers, runs = [], []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if m.kind == "parallel":
            a, r = m.left, m.right
            left = part("gated_attention", dim=cfg.dim, n_heads=a.heads, n_kv_heads=a.kv_heads, head_dim=a.dim,
                        v_head_dim=a.vdim, scale=a.scale, window=a.window, qk_norm="head", norm_eps=cfg.norm_eps,
                        distance_bias=True, bias_rows=None, bias_far=a.bias_max)
            right = part("retention", dim=cfg.dim, n_heads=r.heads, head_dim=r.dim, v_head_dim=r.vdim, decay=r.decay,
                         k_scale=r.dim ** -0.5, rot_dims=r.rot_dims, rot_base=r.rot_base, norm_eps=cfg.norm_eps)
            mixer = part("side_by_side", dim=cfg.dim, left=left, right=right, eps=cfg.norm_eps, coef=0.5)
        else:
            mixer = part("gated_delta", dim=cfg.dim, n_heads=m.heads, n_qk_heads=m.kv_heads, head_dim=m.dim,
                         v_head_dim=m.vdim, conv_taps=m.conv, q_scale=m.dim ** -0.5, norm_eps=cfg.norm_eps, unit_eps=UNIT_EPS)
        mlp = layer.mlp
        if mlp is None:
            ffn = None
        elif mlp.kind == "dense":
            ffn = part("polynorm", dim=cfg.dim, hidden=mlp.ff, eps=cfg.norm_eps)
        else:
            ffn = part("routed_experts", dim=cfg.dim, n_experts=mlp.experts, top=mlp.top, hidden=mlp.ff,
                       activation=EXPERT_ACTIVATION, gated=True, router_bias=True, renormalize=True)
        block = part("parallel", mixer=mixer, feed_forward=ffn, norm=norm, mixer_prefix="mix", ffn_prefix="mlp",
                     norm_prefix="norm1", input_conv_taps=cfg.conv_taps, input_conv_tensor="canon1",
                     token_side_dim=cfg.side_dim, token_side_vocab=cfg.vocab_size, token_side_eps=cfg.norm_eps,
                     side_prefix="side")
        layers.append(LayerSpec(name=f"l{i}", block=block))
        runs.append(RunEntry(i))
    return ModelSpec(
        dim=cfg.dim, vocab_size=cfg.vocab_size, max_positions=cfg.max_seq_len,
        embedding_tensor="embed", layers=tuple(layers), run_order=tuple(runs),
        final_norm=norm, final_norm_prefix="final.norm", head_tensor="head", tie_head=False,
        embedding_norm=norm, embedding_norm_prefix="embed.norm", logit_scale=cfg.logit_scale,
    )


# checkpoint name (inside a layer) -> the parts' own names
_SIDES = {"mix.left": "mix.left", "mix.right": "mix.right"}
_LAYER_NAMES = {
    "norm1": "norm1.weight", "canon1": "canon1",
    "side.gate": "side.gate.weight", "side.proj": "side.proj.weight", "side.norm": "side.norm.weight",
    # window attention
    "mix.left.q": "mix.left.wq.weight", "mix.left.k": "mix.left.wk.weight", "mix.left.v": "mix.left.wv.weight",
    "mix.left.o": "mix.left.wo.weight", "mix.left.q.norm": "mix.left.q_norm.weight",
    "mix.left.k.norm": "mix.left.k_norm.weight", "mix.left.rel": "mix.left.distance_bias", "mix.left.out": "mix.left.out",
    # retention
    "mix.right.q": "mix.right.wq.weight", "mix.right.k": "mix.right.wk.weight", "mix.right.v": "mix.right.wv.weight",
    "mix.right.g": "mix.right.wg.weight", "mix.right.o": "mix.right.wo.weight", "mix.right.out": "mix.right.out",
    # delta rule
    "mix.q": "mix.wq.weight", "mix.k": "mix.wk.weight", "mix.v": "mix.wv.weight", "mix.q.conv": "mix.wq.conv",
    "mix.k.conv": "mix.wk.conv", "mix.v.conv": "mix.wv.conv", "mix.b": "mix.wb.weight", "mix.a": "mix.wa.weight",
    "mix.A_log": "mix.A_log", "mix.dt_bias": "mix.dt_bias", "mix.norm": "mix.norm.weight", "mix.g": "mix.wg.weight",
    "mix.o": "mix.wo.weight",
    # feed-forwards
    "mlp.up": "mlp.up.weight", "mlp.down": "mlp.down.weight", "mlp.act": "mlp.act",
    "mlp.router": "mlp.router.weight", "mlp.router.b": "mlp.router.bias",
}
_TOP_NAMES = {"final.norm": "final.norm.weight", "embed.norm": "embed.norm.weight"}
_LAYER_RE = re.compile(r"^(l\d+)\.(.+)$")
_EXPERT_RE = re.compile(r"^mlp\.e(\d+)\.(gate|up|down)$")
SIDE_TABLE = "side.embed"


def adapt_tensors(cfg: NunosunConfig, found: Dict[str, LazyTensor]) -> Dict[str, LazyTensor]:
    """The checkpoint's names to the parts' names; anything unknown keeps its name, so that the
    strict check reports it.  The per-token table is stored once for all layers, layer ``i`` owning
    the columns ``i * side_dim .. (i + 1) * side_dim``: every layer gets its slice under its own name."""
    out: Dict[str, LazyTensor] = {}
    s, n_layers = cfg.side_dim, len(cfg.layers)
    for name, t in found.items():
        if name == SIDE_TABLE and len(t.shape) == 2 and t.shape[1] == s * n_layers:
            for i in range(n_layers):
                out[f"l{i}.side.table"] = t.mapped(lambda x, i=i: x[:, i * s:(i + 1) * s].contiguous(), shape=(t.shape[0], s))
            continue
        new = _TOP_NAMES.get(name, name)
        m = _LAYER_RE.match(name)
        if m:
            inner = m.group(2)
            e = _EXPERT_RE.match(inner)
            if e:
                new = f"{m.group(1)}.mlp.experts.{int(e.group(1))}.{e.group(2)}.weight"
            elif inner in _LAYER_NAMES:
                new = f"{m.group(1)}.{_LAYER_NAMES[inner]}"
        if new in out:
            raise ValueError(f"checkpoint provides tensor {new!r} under two names")
        out[new] = t
    return out


def tensor_shapes(cfg: NunosunConfig) -> Iterator[Tuple[str, Tuple[int, ...], str]]:
    """``(name, shape, kind of initial values)`` of every tensor a checkpoint of this configuration has, in file order."""
    d, s = cfg.dim, cfg.side_dim
    yield "embed", (cfg.vocab_size, d), "table"
    yield "embed.norm", (d,), "gain"
    yield SIDE_TABLE, (cfg.vocab_size, s * len(cfg.layers)), "table"
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}", layer.mixer
        yield f"{p}.norm1", (d,), "gain"
        if m.kind == "parallel":
            a, r = m.left, m.right
            yield f"{p}.mix.left.q", (a.heads * a.dim, d), "matrix"
            yield f"{p}.mix.left.k", (a.kv_heads * a.dim, d), "matrix"
            yield f"{p}.mix.left.v", (a.kv_heads * a.vdim, d), "matrix"
            yield f"{p}.mix.left.q.norm", (a.dim,), "gain"
            yield f"{p}.mix.left.k.norm", (a.dim,), "gain"
            yield f"{p}.mix.left.rel", (2 * max(2, min(16, a.window // 2)), a.heads), "bias"
            yield f"{p}.mix.left.o", (d, a.heads * a.vdim), "matrix"
            for name, rows in (("q", r.heads * r.dim), ("k", r.heads * r.dim), ("v", r.heads * r.vdim), ("g", r.heads * r.vdim)):
                yield f"{p}.mix.right.{name}", (rows, d), "matrix"
            yield f"{p}.mix.right.o", (d, r.heads * r.vdim), "matrix"
            yield f"{p}.mix.left.out", (d,), "gain"
            yield f"{p}.mix.right.out", (d,), "gain"
        else:
            for name, rows in (("q", m.kv_heads * m.dim), ("k", m.kv_heads * m.dim), ("v", m.heads * m.vdim)):
                yield f"{p}.mix.{name}", (rows, d), "matrix"
                yield f"{p}.mix.{name}.conv", (rows, m.conv), "taps"
            yield f"{p}.mix.b", (m.heads, d), "matrix"
            yield f"{p}.mix.A_log", (m.heads,), "small"
            yield f"{p}.mix.norm", (m.vdim,), "gain"
            yield f"{p}.mix.a", (m.heads, d), "matrix"
            yield f"{p}.mix.dt_bias", (m.heads,), "small"
            yield f"{p}.mix.g", (m.heads * m.vdim, d), "matrix"
            yield f"{p}.mix.o", (d, m.heads * m.vdim), "matrix"
        mlp = layer.mlp
        if mlp is not None and mlp.kind == "dense":
            yield f"{p}.mlp.up", (mlp.ff, d), "matrix"
            yield f"{p}.mlp.down", (d, mlp.ff), "matrix"
            yield f"{p}.mlp.act", (4,), "poly"
        elif mlp is not None:
            for e in range(mlp.experts):
                yield f"{p}.mlp.e{e}.gate", (mlp.ff, d), "matrix"
                yield f"{p}.mlp.e{e}.up", (mlp.ff, d), "matrix"
                yield f"{p}.mlp.e{e}.down", (d, mlp.ff), "matrix"
            yield f"{p}.mlp.router", (mlp.experts, d), "matrix"
            yield f"{p}.mlp.router.b", (mlp.experts,), "bias"
        yield f"{p}.canon1", (d, cfg.conv_taps), "taps"
        yield f"{p}.side.gate", (s, d), "matrix"
        yield f"{p}.side.proj", (d, s), "matrix"
        yield f"{p}.side.norm", (d,), "side_gain"
    yield "final.norm", (d,), "gain"
    yield "head", (cfg.vocab_size, d), "matrix"


def random_tensors(cfg: NunosunConfig, seed: int, *, device="cpu", dtype: torch.dtype = torch.float32) -> Iterator[Tuple[str, torch.Tensor]]:
    """Seeded random weights under the checkpoint's names (one generator, one order, drawn in
    float32, then cast): matrices ``N(0, 1/fan_in)``, table rows of unit size, gains around one,
    convolution taps and distance biases small, the side input's gain well below one."""
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    for name, shape, init in tensor_shapes(cfg):
        t = torch.randn(shape, generator=gen, device=device, dtype=torch.float32)
        if init == "matrix":
            t = t * shape[1] ** -0.5
        elif init == "bias":
            t = t * 0.5
        elif init in ("small", "taps"):
            t = t * 0.3
        elif init == "gain":
            t = 1.0 + t * 0.1
        elif init == "side_gain":
            t = 0.3 + t * 0.05
        elif init == "poly":
            t = torch.tensor([1.0, 0.5, 0.25, 0.0], device=device) + t * 0.1
        yield name, t.to(dtype)


NUNOSUN = register_architecture(Architecture(
    name=NAME,
    parse_config=parse_config,
    build_spec=build_spec,
    adapt_tensors=adapt_tensors,
    random_tensors=random_tensors,
    chat_template=None,
))
