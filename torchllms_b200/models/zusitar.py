"""Zusitar as an :class:`~torchllms_b200.config.registry.Architecture`.

A small decoder whose ``config.json`` lists its layers one by one; every layer names its mixer
(``mamba1``, ``latent_attention`` or ``attention``) with that mixer's own sizes, and its
feed-forward (``dense``, ``moe`` or none).  A span of layers (``loop``: ``start``, ``stop``,
``times``) runs several times in a row with the same weights, every pass with a cache and state
of its own.  What the design fixes and no file carries:

* the stream is the embedding table's row times ``embedding.scale``; the head is the table itself, unscaled;
* a layer is ``x += norm1b(mixer(norm1(x)))``, ``x += norm2b(ff(norm2(x)))``, every norm an RMS
  norm with a plain weight per coordinate;
* before every pass of the looped span the row ``loop.step[pass]`` is added to the stream, and
  before every pass but the first the embedding output as well;
* ``mamba1``: a selective scan behind a causal convolution with bias and ``silu``, gated by ``silu(z)``;
* ``latent_attention``: queries through a normed latent, keys and values linear in a normed
  latent that is all the cache keeps beside one rotated key part shared by the heads (rotate-half
  pairing), ordinary causal softmax, an element-wise sigmoid output gate;
* ``attention``: grouped heads with biases on q, k, v and the output, interleaved rotation on the
  first ``rot.dims`` coordinates, a capped score ``softcap * tanh(score / softcap)``, a learned sink
  per head in the softmax's denominator, a sigmoid output gate per head;
* ``dense``: ``down(silu(gate x) * up x)``;  ``moe``: experts
  ``down(g * sigmoid(1.702 g) * (u + 1))`` with ``g = min(gate x, limit)``, ``u = clamp(up x, +-limit)``,
  sigmoid scores, a choice restricted to the best groups of neighbouring experts (a group's score
  the sum of its two largest), weights ``score / (sum + 1e-20) * router.scale``, and a shared
  expert of the same form with a bound of its own.

This module only describes: it reads the configuration, names the generic parts with their
numbers (:func:`build_spec`), and maps the checkpoint's tensor names to the parts' own.
"""

from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Any, Dict, Iterator, List, Mapping, Optional, Tuple

import torch

from ..config.model_config import ConfigError, ModelConfig, require_key
from ..config.registry import Architecture, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, RunEntry, part
from ..weights.loader import LazyTensor

NAME = "Zusitar"

# The design has no longest sequence (rotary positions, a recurrent state); tables are made this
# long unless whoever builds the engine asks for more.
DEFAULT_MAX_POSITIONS = 32768

EXPERT_ALPHA = 1.702          # g * sigmoid(EXPERT_ALPHA * g)
EXPERT_UP_OFFSET = 1.0        # (u + EXPERT_UP_OFFSET)
RENORM_EPS = 1e-20            # weights = score / (sum of the chosen scores + RENORM_EPS)
GROUP_SCORE_TOP = 2           # a group's score is the sum of its so many largest scores
LOOP_TENSOR = "loop.step"


def _object(raw: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    value = raw.get(key)
    if not isinstance(value, Mapping):
        raise ConfigError(f"{where}: key '{key}' must be an object")
    return value


@dataclass(frozen=True)
class ScanConfig:
    inner: int
    state: int
    dt_rank: int
    conv: int

    kind = "mamba1"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "ScanConfig":
        return cls(inner=require_key(raw, "inner", int, where), state=require_key(raw, "state", int, where),
                   dt_rank=require_key(raw, "dt_rank", int, where), conv=require_key(raw, "conv", int, where))

    def to_dict(self) -> Dict[str, Any]:
        return {"conv": self.conv, "dt_rank": self.dt_rank, "inner": self.inner, "state": self.state}

    def validate(self, at: str) -> None:
        for key in ("inner", "state", "dt_rank", "conv"):
            if getattr(self, key) <= 0:
                raise ConfigError(f"{at}: mixer '{key}' must be positive, got {getattr(self, key)}")


@dataclass(frozen=True)
class LatentConfig:
    heads: int
    dim: int                        # unrotated query/key size of a head
    rot_dim: int                    # rotated query/key size of a head (the key part is shared by the heads)
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot_dims: int
    rot_base: float

    kind = "latent_attention"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "LatentConfig":
        rot = _object(raw, "rot", where)
        return cls(heads=require_key(raw, "heads", int, where), dim=require_key(raw, "dim", int, where),
                   rot_dim=require_key(raw, "rot_dim", int, where), vdim=require_key(raw, "vdim", int, where),
                   q_rank=require_key(raw, "q_rank", int, where), kv_rank=require_key(raw, "kv_rank", int, where),
                   scale=require_key(raw, "scale", float, where), rot_dims=require_key(rot, "dims", int, f"{where}.rot"),
                   rot_base=require_key(rot, "base", float, f"{where}.rot"))

    def to_dict(self) -> Dict[str, Any]:
        return {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank, "q_rank": self.q_rank,
                "rot": {"base": self.rot_base, "dims": self.rot_dims}, "rot_dim": self.rot_dim, "scale": self.scale,
                "vdim": self.vdim}

    def validate(self, at: str) -> None:
        for key in ("heads", "dim", "vdim", "q_rank", "kv_rank"):
            if getattr(self, key) <= 0:
                raise ConfigError(f"{at}: mixer '{key}' must be positive, got {getattr(self, key)}")
        if self.rot_dim < 0 or self.rot_dim % 2:
            raise ConfigError(f"{at}: 'rot_dim' must be even and not negative, got {self.rot_dim}")
        if self.rot_dims != self.rot_dim:
            raise ConfigError(f"{at}: the rotated part is turned as a whole: 'rot.dims' ({self.rot_dims}) must equal "
                              f"'rot_dim' ({self.rot_dim})")
        if not self.rot_base > 0:
            raise ConfigError(f"{at}: 'rot.base' must be positive")


@dataclass(frozen=True)
class AttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float
    rot_dims: int
    rot_base: float

    kind = "attention"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "AttentionConfig":
        rot = _object(raw, "rot", where)
        return cls(heads=require_key(raw, "heads", int, where), kv_heads=require_key(raw, "kv_heads", int, where),
                   dim=require_key(raw, "dim", int, where), vdim=require_key(raw, "vdim", int, where),
                   scale=require_key(raw, "scale", float, where), softcap=require_key(raw, "softcap", float, where),
                   rot_dims=require_key(rot, "dims", int, f"{where}.rot"), rot_base=require_key(rot, "base", float, f"{where}.rot"))

    def to_dict(self) -> Dict[str, Any]:
        return {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads,
                "rot": {"base": self.rot_base, "dims": self.rot_dims}, "scale": self.scale, "softcap": self.softcap,
                "vdim": self.vdim}

    def validate(self, at: str) -> None:
        for key in ("heads", "kv_heads", "dim", "vdim"):
            if getattr(self, key) <= 0:
                raise ConfigError(f"{at}: mixer '{key}' must be positive, got {getattr(self, key)}")
        if self.heads % self.kv_heads != 0:
            raise ConfigError(f"{at}: 'heads' ({self.heads}) must be a multiple of 'kv_heads' ({self.kv_heads})")
        if self.rot_dims < 0 or self.rot_dims % 2 or self.rot_dims > self.dim:
            raise ConfigError(f"{at}: 'rot.dims' must be even and at most 'dim' ({self.dim}), got {self.rot_dims}")
        if not self.rot_base > 0 or not self.softcap > 0:
            raise ConfigError(f"{at}: 'rot.base' and 'softcap' must be positive")


@dataclass(frozen=True)
class MlpConfig:
    kind: str                       # "dense" or "moe"
    ff: int                         # dense: the hidden size; moe: one expert's
    limit: float = 0.0              # moe: the experts' bound
    experts: int = 0
    top: int = 0
    router_scale: float = 1.0
    groups: int = 1
    keep_groups: int = 1
    shared_ff: int = 0              # 0: no shared expert
    shared_limit: float = 0.0

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "MlpConfig":
        kind = require_key(raw, "kind", str, where)
        if kind == "dense":
            return cls(kind, require_key(raw, "ff", int, where))
        if kind == "moe":
            router, expert = _object(raw, "router", where), _object(raw, "expert", where)
            groups = router.get("groups")
            count = keep = 1
            if groups is not None:
                groups = _object(router, "groups", f"{where}.router")
                count = require_key(groups, "count", int, f"{where}.router.groups")
                keep = require_key(groups, "keep", int, f"{where}.router.groups")
            shared = raw.get("shared")
            if shared is not None:
                shared = _object(raw, "shared", where)
            return cls(kind, require_key(expert, "ff", int, f"{where}.expert"),
                       limit=require_key(expert, "limit", float, f"{where}.expert"),
                       experts=require_key(router, "experts", int, f"{where}.router"),
                       top=require_key(router, "top", int, f"{where}.router"),
                       router_scale=require_key(router, "scale", float, f"{where}.router"),
                       groups=count, keep_groups=keep,
                       shared_ff=0 if shared is None else require_key(shared, "ff", int, f"{where}.shared"),
                       shared_limit=0.0 if shared is None else require_key(shared, "limit", float, f"{where}.shared"))
        raise ConfigError(f"{where}: unknown feed-forward kind {kind!r}; known: dense, moe")

    def to_dict(self) -> Dict[str, Any]:
        if self.kind == "dense":
            return {"ff": self.ff, "kind": "dense"}
        out: Dict[str, Any] = {"expert": {"ff": self.ff, "limit": self.limit}, "kind": "moe",
                               "router": {"experts": self.experts, "groups": {"count": self.groups, "keep": self.keep_groups},
                                          "scale": self.router_scale, "top": self.top}}
        if self.shared_ff:
            out["shared"] = {"ff": self.shared_ff, "limit": self.shared_limit}
        return out

    def validate(self, at: str) -> None:
        if self.ff <= 0:
            raise ConfigError(f"{at}: the feed-forward's 'ff' must be positive")
        if self.kind != "moe":
            return
        if not 0 < self.top <= self.experts:
            raise ConfigError(f"{at}: router 'top' must lie between 1 and 'experts' ({self.experts}), got {self.top}")
        if self.groups < 1 or self.experts % self.groups != 0:
            raise ConfigError(f"{at}: 'groups.count' ({self.groups}) must divide 'experts' ({self.experts})")
        if not 0 < self.keep_groups <= self.groups:
            raise ConfigError(f"{at}: 'groups.keep' must lie between 1 and 'groups.count' ({self.groups}), got {self.keep_groups}")
        if self.keep_groups * (self.experts // self.groups) < self.top:
            raise ConfigError(f"{at}: the kept groups hold fewer experts than 'top' ({self.top})")
        if not self.limit > 0 or (self.shared_ff and not self.shared_limit > 0) or self.shared_ff < 0:
            raise ConfigError(f"{at}: an expert's 'limit' must be positive")


@dataclass(frozen=True)
class LayerConfig:
    mixer: Any                      # ScanConfig, LatentConfig or AttentionConfig
    mlp: Optional[MlpConfig]


_MIXERS = {"mamba1": ScanConfig, "latent_attention": LatentConfig, "attention": AttentionConfig}


@dataclass(frozen=True)
class ZusitarConfig(ModelConfig):
    architecture: str
    vocab_size: int
    dim: int
    norm_eps: float
    embedding_scale: float
    layers: Tuple[LayerConfig, ...]
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    max_seq_len: int = DEFAULT_MAX_POSITIONS

    @classmethod
    def from_json(cls, raw: Mapping[str, Any], where: str) -> "ZusitarConfig":
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
        loop = raw.get("loop")
        start = stop = 0
        times = 1
        if loop is not None:
            loop = _object(raw, "loop", where)
            start, stop = require_key(loop, "start", int, f"{where}: loop"), require_key(loop, "stop", int, f"{where}: loop")
            times = require_key(loop, "times", int, f"{where}: loop")
        return cls(
            architecture=NAME,
            vocab_size=require_key(raw, "vocab", int, where),
            dim=require_key(raw, "width", int, where),
            norm_eps=require_key(_object(raw, "norm", where), "eps", float, f"{where}: norm"),
            embedding_scale=require_key(_object(raw, "embedding", where), "scale", float, f"{where}: embedding"),
            layers=tuple(parsed), loop_start=start, loop_stop=stop, loop_times=times,
        ).validate(where)

    @property
    def loops(self) -> bool:
        return self.loop_stop > self.loop_start

    def validate(self, where: str = "config") -> "ZusitarConfig":
        for key in ("vocab_size", "dim", "max_seq_len"):
            if getattr(self, key) <= 0:
                raise ConfigError(f"{where}: '{key}' must be positive, got {getattr(self, key)}")
        for i, layer in enumerate(self.layers):
            at = f"{where}: layers[{i}]"
            layer.mixer.validate(at)
            if layer.mlp is not None:
                layer.mlp.validate(at)
        if self.loops or self.loop_times != 1:
            if not (0 <= self.loop_start < self.loop_stop <= len(self.layers)) or self.loop_times < 1:
                raise ConfigError(f"{where}: 'loop' must name layers start .. stop - 1 of the {len(self.layers)} there are, "
                                  f"run at least once; got start {self.loop_start}, stop {self.loop_stop}, times {self.loop_times}")
        return self

    def runs(self) -> List[Tuple[int, Optional[int]]]:
        """``(layer, pass)`` of every layer run in order; ``pass`` is a number for the first layer
        of every pass of the looped span and ``None`` elsewhere."""
        n = len(self.layers)
        if not self.loops:
            return [(i, None) for i in range(n)]
        out: List[Tuple[int, Optional[int]]] = [(i, None) for i in range(self.loop_start)]
        for t in range(self.loop_times):
            out += [(i, t if i == self.loop_start else None) for i in range(self.loop_start, self.loop_stop)]
        return out + [(i, None) for i in range(self.loop_stop, n)]

    def to_hf(self) -> Dict[str, Any]:
        out = {
            "architecture": NAME,
            "embedding": {"scale": self.embedding_scale},
            "layers": [{"mixer": l.mixer.to_dict(), "mlp": None if l.mlp is None else l.mlp.to_dict(), "type": l.mixer.kind}
                       for l in self.layers],
            "norm": {"eps": self.norm_eps},
            "vocab": self.vocab_size,
            "width": self.dim,
        }
        if self.loops:
            out["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        return out


def parse_config(raw: Mapping[str, Any], source: str) -> ZusitarConfig:
    return ZusitarConfig.from_json(raw, source)


def build_spec(cfg: ZusitarConfig) -> ModelSpec:
    norm = part("rmsnorm", dim=cfg.dim, eps=cfg.norm_eps)
    layers = []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if m.kind == "mamba1":
            mixer = part("selective_scan", dim=cfg.dim, inner=m.inner, state=m.state, dt_rank=m.dt_rank, conv_taps=m.conv)
        elif m.kind == "latent_attention":
            mixer = part("rotary_latent_attention", dim=cfg.dim, n_heads=m.heads, head_dim=m.dim, rot_dim=m.rot_dim,
                         v_head_dim=m.vdim, q_rank=m.q_rank, rank=m.kv_rank, scale=m.scale, rot_base=m.rot_base,
                         rot_pairing="half", norm_eps=cfg.norm_eps, gate="element")
        else:
            mixer = part("rotary_gated_attention", dim=cfg.dim, n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim,
                         v_head_dim=m.vdim, scale=m.scale, softcap=m.softcap, sinks=True, rot_dims=m.rot_dims,
                         rot_base=m.rot_base, rot_pairing="interleaved", qkv_bias=True, out_bias=True, gate="head")
        mlp = layer.mlp
        if mlp is None:
            ffn = None
        elif mlp.kind == "dense":
            ffn = part("glu", dim=cfg.dim, hidden=mlp.ff, activation="silu")
        else:
            ffn = part("routed_experts", dim=cfg.dim, n_experts=mlp.experts, top=mlp.top, hidden=mlp.ff, gated=True,
                       activation="clamped_swish", act_limit=mlp.limit, act_alpha=EXPERT_ALPHA, act_up_offset=EXPERT_UP_OFFSET,
                       score="sigmoid", n_groups=mlp.groups, keep_groups=mlp.keep_groups, group_score_top=GROUP_SCORE_TOP,
                       router_scale=mlp.router_scale, renormalize=True, renorm_eps=RENORM_EPS,
                       shared_hidden=mlp.shared_ff or None, shared_act_limit=mlp.shared_limit or None)
        block = part("sandwich", mixer=mixer, feed_forward=ffn, mixer_norm=norm, mixer_out_norm=norm,
                     ffn_norm=None if ffn is None else norm, ffn_out_norm=None if ffn is None else norm,
                     mixer_prefix="mix", ffn_prefix="mlp", mixer_norm_prefix="norm1", mixer_out_norm_prefix="norm1b",
                     ffn_norm_prefix="norm2", ffn_out_norm_prefix="norm2b")
        layers.append(LayerSpec(name=f"l{i}", block=block))
    # every run has a cache and state of its own, also the runs of one layer in different passes
    runs = tuple(RunEntry(i, add_embedding=bool(t), add_row=None if t is None else (LOOP_TENSOR, t)) for i, t in cfg.runs())
    return ModelSpec(
        dim=cfg.dim, vocab_size=cfg.vocab_size, max_positions=cfg.max_seq_len,
        embedding_tensor="embed", layers=tuple(layers), run_order=runs,
        final_norm=norm, final_norm_prefix="final.norm", head_tensor="head", tie_head=True,
        embedding_scale=cfg.embedding_scale,
        row_tensors=((LOOP_TENSOR, cfg.loop_times),) if cfg.loops else (),
    )


# checkpoint name (inside a layer) -> the parts' own names
_LAYER_NAMES = {
    "norm1": "norm1.weight", "norm1b": "norm1b.weight", "norm2": "norm2.weight", "norm2b": "norm2b.weight",
    # selective scan
    "mix.in": "mix.w_in.weight", "mix.conv": "mix.conv.weight", "mix.conv.b": "mix.conv.bias", "mix.x": "mix.w_x.weight",
    "mix.dt": "mix.w_dt.weight", "mix.dt.b": "mix.w_dt.bias", "mix.A_log": "mix.A_log", "mix.D": "mix.D",
    # all mixers
    "mix.o": "mix.wo.weight", "mix.g": "mix.wg.weight",
    # latent attention
    "mix.dq": "mix.wq_down.weight", "mix.dq.norm": "mix.q_norm.weight", "mix.uq": "mix.wq_up.weight",
    "mix.dkv": "mix.w_down.weight", "mix.dkv.norm": "mix.latent_norm.weight", "mix.uk": "mix.w_up_k.weight",
    "mix.uv": "mix.w_up_v.weight",
    # attention
    "mix.q": "mix.wq.weight", "mix.q.b": "mix.wq.bias", "mix.k": "mix.wk.weight", "mix.k.b": "mix.wk.bias",
    "mix.v": "mix.wv.weight", "mix.v.b": "mix.wv.bias", "mix.o.b": "mix.wo.bias", "mix.sink": "mix.sinks",
    # feed-forwards
    "mlp.gate": "mlp.gate.weight", "mlp.up": "mlp.up.weight", "mlp.down": "mlp.down.weight",
    "mlp.router": "mlp.router.weight", "mlp.shared.gate": "mlp.shared.w_gate.weight", "mlp.shared.up": "mlp.shared.up.weight",
    "mlp.shared.down": "mlp.shared.down.weight",
}
_TOP_NAMES = {"final.norm": "final.norm.weight"}
_LAYER_RE = re.compile(r"^(l\d+)\.(.+)$")
_EXPERT_RE = re.compile(r"^mlp\.e(\d+)\.(gate|up|down)$")


def adapt_tensors(cfg: ZusitarConfig, found: Dict[str, LazyTensor]) -> Dict[str, LazyTensor]:
    """The checkpoint's names to the parts' names; anything unknown keeps its name, so that the
    strict check reports it."""
    out: Dict[str, LazyTensor] = {}
    unread = {f"l{i}.{n}" for i, layer in enumerate(cfg.layers) if layer.mlp is None for n in ("norm2", "norm2b")}
    for name, t in found.items():
        if name in unread:
            continue                 # norms stored for a feed-forward that the layer does not have: nothing reads them
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


def tensor_shapes(cfg: ZusitarConfig) -> Iterator[Tuple[str, Tuple[int, ...], str]]:
    """``(checkpoint name, shape, init)`` of every tensor, in the order random weights are drawn in."""
    d = cfg.dim
    yield "embed", (cfg.vocab_size, d), "embed"
    if cfg.loops:
        yield LOOP_TENSOR, (cfg.loop_times, d), "small"
    for i, layer in enumerate(cfg.layers):
        m, mlp, p = layer.mixer, layer.mlp, f"l{i}"
        for n in ("norm1", "norm1b") + (("norm2", "norm2b") if mlp is not None else ()):
            yield f"{p}.{n}", (d,), "gain"
        if m.kind == "mamba1":
            yield f"{p}.mix.in", (2 * m.inner, d), "matrix"
            yield f"{p}.mix.conv", (m.inner, m.conv), "taps"
            yield f"{p}.mix.conv.b", (m.inner,), "bias"
            yield f"{p}.mix.x", (m.dt_rank + 2 * m.state, m.inner), "matrix"
            yield f"{p}.mix.dt", (m.inner, m.dt_rank), "matrix"
            yield f"{p}.mix.dt.b", (m.inner,), "dt_bias"
            yield f"{p}.mix.A_log", (m.inner, m.state), "a_log"
            yield f"{p}.mix.D", (m.inner,), "gain"
            yield f"{p}.mix.o", (d, m.inner), "matrix"
        elif m.kind == "latent_attention":
            yield f"{p}.mix.dq", (m.q_rank, d), "matrix"
            yield f"{p}.mix.dq.norm", (m.q_rank,), "gain"
            yield f"{p}.mix.uq", (m.heads * (m.dim + m.rot_dim), m.q_rank), "matrix"
            yield f"{p}.mix.dkv", (m.kv_rank + m.rot_dim, d), "matrix"
            yield f"{p}.mix.dkv.norm", (m.kv_rank,), "gain"
            yield f"{p}.mix.uk", (m.heads * m.dim, m.kv_rank), "matrix"
            yield f"{p}.mix.uv", (m.heads * m.vdim, m.kv_rank), "matrix"
            yield f"{p}.mix.g", (m.heads * m.vdim, d), "matrix"
            yield f"{p}.mix.o", (d, m.heads * m.vdim), "matrix"
        else:
            for n, rows in (("q", m.heads * m.dim), ("k", m.kv_heads * m.dim), ("v", m.kv_heads * m.vdim)):
                yield f"{p}.mix.{n}", (rows, d), "matrix"
                yield f"{p}.mix.{n}.b", (rows,), "bias"
            yield f"{p}.mix.sink", (m.heads,), "small"
            yield f"{p}.mix.g", (m.heads, d), "matrix"
            yield f"{p}.mix.o", (d, m.heads * m.vdim), "matrix"
            yield f"{p}.mix.o.b", (d,), "bias"
        if mlp is not None and mlp.kind == "dense":
            yield f"{p}.mlp.gate", (mlp.ff, d), "matrix"
            yield f"{p}.mlp.up", (mlp.ff, d), "matrix"
            yield f"{p}.mlp.down", (d, mlp.ff), "matrix"
        elif mlp is not None:
            for e in range(mlp.experts):
                yield f"{p}.mlp.e{e}.gate", (mlp.ff, d), "matrix"
                yield f"{p}.mlp.e{e}.up", (mlp.ff, d), "matrix"
                yield f"{p}.mlp.e{e}.down", (d, mlp.ff), "matrix"
            yield f"{p}.mlp.router", (mlp.experts, d), "matrix"
            if mlp.shared_ff:
                yield f"{p}.mlp.shared.gate", (mlp.shared_ff, d), "matrix"
                yield f"{p}.mlp.shared.up", (mlp.shared_ff, d), "matrix"
                yield f"{p}.mlp.shared.down", (d, mlp.shared_ff), "matrix"
    yield "final.norm", (d,), "gain"


def random_tensors(cfg: ZusitarConfig, seed: int, *, device="cpu", dtype: torch.dtype = torch.float32) -> Iterator[Tuple[str, torch.Tensor]]:
    """Seeded random weights under the checkpoint's names (one generator, one order, drawn in
    float32, then cast): matrices ``N(0, 1/fan_in)``, table rows of unit size (so that the scaled
    embedding and the tied head both stay moderate), gains around one, decays spread over a range."""
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    for name, shape, init in tensor_shapes(cfg):
        t = torch.randn(shape, generator=gen, device=device, dtype=torch.float32)
        if init == "matrix":
            t = t * shape[1] ** -0.5
        elif init == "embed":
            t = t * shape[1] ** -0.5
        elif init == "taps":
            t = t * shape[1] ** -0.5
        elif init == "bias":
            t = t * 0.1
        elif init == "small":
            t = t * 0.2
        elif init == "gain":
            t = 1.0 + t * 0.1
        elif init == "dt_bias":
            t = t * 0.5 - 2.0                     # softplus of it: steps around 0.1
        elif init == "a_log":
            t = torch.log(torch.arange(1, shape[1] + 1, device=device, dtype=torch.float32)).expand(shape) + t * 0.1
        yield name, t.to(dtype)


ZUSITAR = register_architecture(Architecture(
    name=NAME,
    parse_config=parse_config,
    build_spec=build_spec,
    adapt_tensors=adapt_tensors,
    random_tensors=random_tensors,
    chat_template=None,
))
