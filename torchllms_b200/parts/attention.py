"""Grouped-query attention over the paged cache.

Reference: ``Attention`` (torchllms/models/networks.py:460-558): projections
``wq, wk, wv`` (``nn.Linear`` layout ``[out, in]``, no bias), rotary encoding of
q and k, append of k and v to the pool, attention of every query over the keys
at positions ``<=`` its own with scale ``head_dim ** -0.5`` (:842; eager form
:355-397, query head ``h`` reads kv head ``h // (H / KV)``), then ``wo``.  The
reference calls a library for the paged attention
(torchllms/models/paged_attention.py:217-301); the kernel here is our own and
treats prompt portions and single decoded tokens alike.
"""

from __future__ import annotations

import math
from typing import Dict, Mapping, Optional

import torch

from ..kernels.lazy import PendingProduct
from ..weights.loader import ExpectedTensor
from .base import (POSITION_ENCODINGS, BuildEnv, CacheNeed, Mixer, as_compute, register_mixer)
from .rope import precise_rotary_table
from .spec import PartSpec


@register_mixer("attention")
class PagedAttention(Mixer):
    def __init__(self, env: BuildEnv, *, dim: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 scale: float, position: PartSpec, window: Optional[int] = None):
        if n_heads % n_kv_heads != 0:
            raise ValueError(f"n_heads ({n_heads}) must be a multiple of n_kv_heads ({n_kv_heads})")
        self.env = env
        self.dim, self.n_heads, self.n_kv_heads, self.head_dim = int(dim), int(n_heads), int(n_kv_heads), int(head_dim)
        self.scale = float(scale)
        self.window = None if window is None else int(window)
        self.position = POSITION_ENCODINGS.build(position, env)
        self.graph_safe = self.position.graph_safe
        # x only goes into the q/k/v product, whose result the position encoding's kernel may scale
        self.takes_row_scaled = self.position.takes_row_scaled
        env.ops.check_attention_sizes(self.n_heads, self.n_kv_heads, self.head_dim, env.dtype)
        self.wqkv: Optional[torch.Tensor] = None
        self.wo: Optional[torch.Tensor] = None

    def cache_need(self) -> CacheNeed:
        if self.window is None:
            return CacheNeed("full", self.n_kv_heads, self.head_dim)
        return CacheNeed("window", self.n_kv_heads, self.head_dim, self.window)

    def expected_tensors(self) -> Dict[str, ExpectedTensor]:
        q, kv = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
        out = {
            "wq.weight": ExpectedTensor((q, self.dim)),
            "wk.weight": ExpectedTensor((kv, self.dim)),
            "wv.weight": ExpectedTensor((kv, self.dim)),
            "wo.weight": ExpectedTensor((self.dim, q)),
        }
        # a position encoding with tensors of its own (none for rope) keeps them under "position."
        for name, e in self.position.expected_tensors().items():
            out[f"position.{name}"] = e
        return out

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        # One projection for q, k and v: rows [wq; wk; wv].
        self.wqkv = torch.cat([as_compute(tensors[n], self.env) for n in ("wq.weight", "wk.weight", "wv.weight")])
        self.wo = as_compute(tensors["wo.weight"], self.env)
        self.position.load({name: tensors[f"position.{name}"] for name in self.position.expected_tensors()})

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        ops = self.env.ops
        qkv = ops.linear(x, self.wqkv, partials_ok=True)   # the encoding adds up split-K partial sums
        q = self.position.encode_and_store(qkv, ctx, cache, self.n_heads, self.n_kv_heads, self.head_dim)
        common = dict(scale=self.scale, window=self.window, page_size=cache.page_size)
        nd, B = getattr(ctx, "n_decode", 0), ctx.n_seqs
        if 0 < nd < B and ctx.max_q_len > 1:
            # decoded tokens beside prompt portions: the requests at the head of the batch bring one
            # token each and long histories, the rest bring portions; each kind goes to the kernel
            # shape made for it, both writing into one output
            o = torch.empty_like(q)
            ops.paged_attention(q, cache.k_pages, cache.v_pages, cache.block_table[:nd], ctx.q_start[:nd + 1],
                                ctx.kv_len[:nd], n_seqs=nd, max_q_len=1, max_kv_len=ctx.decode_kv_bound,
                                n_tokens=nd, out=o, **common)
            ops.paged_attention(q, cache.k_pages, cache.v_pages, cache.block_table[nd:], ctx.q_start[nd:],
                                ctx.kv_len[nd:], n_seqs=B - nd, max_q_len=ctx.max_q_len, max_kv_len=ctx.max_kv_len,
                                out=o, allow_split=False, **common)   # (a merge pass would run over the first call's rows too)
        else:
            o = ops.paged_attention(
                q, cache.k_pages, cache.v_pages, cache.block_table, ctx.q_start, ctx.kv_len,
                n_seqs=B, max_q_len=ctx.max_q_len, max_kv_len=ctx.max_kv_len, **common)
        # the output projection is left to the norm that follows: it may add the product to the
        # residual stream in the product's own kernel, or take it and add up its partial sums
        return PendingProduct(o.view(o.shape[0], self.n_heads * self.head_dim), self.wo)


def distance_buckets(n_rows: int, far: float, n_positions: int) -> torch.Tensor:
    """``[n_positions]`` int32: the row of a distance-bias table for a key ``n`` places back.
    Distances below half the rows have a row each; from there the rows are spread evenly over
    ``ln(n)`` up to the distance ``far``; everything beyond falls into the last row:

        ``row(n) = n``                                                              for ``n < n_rows // 2``
        ``row(n) = min(n_rows - 1, half + floor(ln(n / half) / ln(far / half) * (n_rows - half)))``   otherwise

    Tabulated once on the host (64-bit logarithms); the attention kernels look a distance up."""
    half = n_rows // 2
    if half < 1 or not far > half:
        raise ValueError(f"a distance-bias table needs at least two rows and a far distance above {half}, got {n_rows} and {far}")
    out = []
    for n in range(n_positions):
        if n < half:
            out.append(n)
        else:
            out.append(min(n_rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (n_rows - half)))))
    return torch.tensor(out, dtype=torch.int32)


@register_mixer("gated_attention")
class GatedBiasedAttention(Mixer):
    """Grouped-query attention without rotation, for designs that put positions elsewhere:

    * projections ``wq, wk, wv`` with optional biases (``qkv_bias``), keys and values of different
      sizes (``head_dim``, ``v_head_dim``);
    * optionally an RMS norm over the *whole* projected row of q and of k (``qk_norm``: before the
      row is cut into heads; plain weights ``q_norm.weight``, ``k_norm.weight``), or, with
      ``qk_norm="head"``, over every head of q and of k by itself, the weights (``head_dim`` numbers
      each) shared by all heads;
    * score ``= q . k * scale`` plus, with ``distance_bias``, a learned bias by distance and head
      (tensor ``distance_bias`` ``[rows, n_heads]``, row chosen by :func:`distance_buckets`; the scale
      does not touch it; ``bias_rows=None`` takes the number of rows from the stored table);
    * a sliding window that may keep a request's first ``keep_first`` tokens visible for ever;
    * ordinary softmax, then an element-wise output gate ``sigmoid(wg x)`` (``gated``) ahead of ``wo``.

    All four projections of the input are one stacked product; what follows it (biases, norms,
    the cache write, the gate's sigmoid) is one kernel; the gate is applied where the attention
    kernel writes its result."""

    graph_safe = True

    def __init__(self, env: BuildEnv, *, dim: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 v_head_dim: Optional[int] = None, scale: float, window: Optional[int] = None, keep_first: int = 0,
                 qkv_bias: bool = False, qk_norm=False, norm_eps: float = 1e-6,
                 distance_bias: bool = False, bias_rows: Optional[int] = None, bias_far: float = 0.0,
                 gated: bool = False):
        if n_heads % n_kv_heads != 0:
            raise ValueError(f"n_heads ({n_heads}) must be a multiple of n_kv_heads ({n_kv_heads})")
        if keep_first and window is None:
            raise ValueError("keep_first goes with a window")
        self.env = env
        self.dim, self.n_heads, self.n_kv_heads = int(dim), int(n_heads), int(n_kv_heads)
        self.head_dim = int(head_dim)
        self.v_head_dim = int(v_head_dim if v_head_dim is not None else head_dim)
        self.scale = float(scale)
        self.window = None if window is None else int(window)
        self.keep_first = int(keep_first)
        self.qkv_bias, self.qk_norm, self.gated = bool(qkv_bias), bool(qk_norm), bool(gated)
        self.norm_per_head = qk_norm == "head"
        self.norm_eps = float(norm_eps)
        self.has_bias = bool(distance_bias)
        self.bias_rows, self.bias_far = (None if bias_rows is None else int(bias_rows)), float(bias_far)
        self.n_q = self.n_heads * self.head_dim
        self.n_k = self.n_kv_heads * self.head_dim
        self.n_v = self.n_kv_heads * self.v_head_dim
        self.n_g = self.n_heads * self.v_head_dim if self.gated else 0
        env.ops.check_attention_sizes(self.n_heads, self.n_kv_heads, self.head_dim, env.dtype, v_head_dim=self.v_head_dim)
        self.buckets: Optional[torch.Tensor] = None
        self.w_in: Optional[torch.Tensor] = None
        self.b_in: Optional[torch.Tensor] = None
        self.q_norm_w: Optional[torch.Tensor] = None
        self.k_norm_w: Optional[torch.Tensor] = None
        self.distance_bias: Optional[torch.Tensor] = None
        self.wo: Optional[torch.Tensor] = None

    def cache_need(self) -> CacheNeed:
        if self.window is None:
            return CacheNeed("full", self.n_kv_heads, self.head_dim, None, self.v_head_dim)
        return CacheNeed("window", self.n_kv_heads, self.head_dim, self.window, self.v_head_dim, self.keep_first)

    def expected_tensors(self) -> Dict[str, ExpectedTensor]:
        out = {
            "wq.weight": ExpectedTensor((self.n_q, self.dim)),
            "wk.weight": ExpectedTensor((self.n_k, self.dim)),
            "wv.weight": ExpectedTensor((self.n_v, self.dim)),
            "wo.weight": ExpectedTensor((self.dim, self.n_heads * self.v_head_dim)),
        }
        if self.qkv_bias:
            out.update({"wq.bias": ExpectedTensor((self.n_q,)), "wk.bias": ExpectedTensor((self.n_k,)),
                        "wv.bias": ExpectedTensor((self.n_v,))})
        if self.qk_norm:
            if self.norm_per_head:
                out.update({"q_norm.weight": ExpectedTensor((self.head_dim,)), "k_norm.weight": ExpectedTensor((self.head_dim,))})
            else:
                out.update({"q_norm.weight": ExpectedTensor((self.n_q,)), "k_norm.weight": ExpectedTensor((self.n_k,))})
        if self.has_bias:
            out["distance_bias"] = ExpectedTensor((-1 if self.bias_rows is None else self.bias_rows, self.n_heads))
        if self.gated:
            out["wg.weight"] = ExpectedTensor((self.n_g, self.dim))
        return out

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        f32 = dict(device=self.env.device, dtype=torch.float32)
        names = ["wq.weight", "wk.weight", "wv.weight"] + (["wg.weight"] if self.gated else [])
        self.w_in = torch.cat([as_compute(tensors[n], self.env) for n in names])       # rows [wq; wk; wv; wg]
        if self.qkv_bias:
            parts = [tensors[n].to(**f32) for n in ("wq.bias", "wk.bias", "wv.bias")]
            parts.append(torch.zeros(self.n_g, **f32))
            self.b_in = torch.cat(parts).contiguous()
        if self.qk_norm:
            self.q_norm_w = tensors["q_norm.weight"].to(**f32).contiguous()
            self.k_norm_w = tensors["k_norm.weight"].to(**f32).contiguous()
        if self.has_bias:
            self.distance_bias = tensors["distance_bias"].to(**f32).contiguous()
            self.buckets = distance_buckets(self.distance_bias.shape[0], self.bias_far, self.env.max_positions).to(self.env.device)
        self.wo = as_compute(tensors["wo.weight"], self.env)

    def forward(self, x: torch.Tensor, ctx, cache) -> PendingProduct:
        ops = self.env.ops
        proj = ops.linear(x, self.w_in, partials_ok=True)
        q, gate = ops.project_and_store(
            proj, n_q=self.n_q, n_k=self.n_k, n_v=self.n_v, n_extra=self.n_g, bias=self.b_in,
            q_norm=self.q_norm_w, k_norm=self.k_norm_w, eps=self.norm_eps,
            norm_head_dim=self.head_dim if self.norm_per_head else None, k_pages=cache.k_pages if cache.writes else None, v_pages=cache.v_pages if cache.writes else None,
            slot_mapping=cache.slot_mapping, page_size=cache.page_size, out_dtype=self.env.dtype)
        o = ops.paged_attention(
            q.view(-1, self.n_heads, self.head_dim), cache.k_pages, cache.v_pages, cache.block_table, ctx.q_start,
            ctx.kv_len, n_seqs=ctx.n_seqs, max_q_len=ctx.max_q_len, max_kv_len=ctx.max_kv_len, scale=self.scale,
            window=self.window, page_size=cache.page_size, keep_first=self.keep_first,
            distance_bias=self.distance_bias, distance_buckets=self.buckets, gate=gate, impl="auto")
        return PendingProduct(o.view(o.shape[0], self.n_heads * self.v_head_dim), self.wo)


@register_mixer("differential_attention")
class DifferentialAttention(Mixer):
    """Grouped-query attention with two softmax maps per head over one set of values, combined by
    subtraction:

    * ``wq`` has ``n_heads * 2 * head_dim`` rows and ``wk`` ``n_kv_heads * 2 * head_dim``, head by
      head as ``[map 1, map 2]``; ``wv`` has ``n_kv_heads * v_head_dim`` rows; no biases;
    * rotary positions on the first ``rot_dims`` coordinates of every map of q and k (``rot_pairing``
      ``"half"``: coordinate ``i`` with ``i + rot_dims / 2``), angles ``p * rot_base^(-2i/rot_dims) /
      rot_factor``; keys are stored rotated;
    * each map is causal softmax attention with ``score = q . k * scale``;
    * ``o = a1 - lambda a2`` with ``lambda = exp(lambda_q1 . lambda_k1) - exp(lambda_q2 . lambda_k2)
      + lambda_init`` (four stored vectors of ``head_dim``, one number for the layer), then
      ``o / sqrt(mean(o^2) + norm_eps)`` over the head's values, times ``1 - lambda_init``;
    * with ``gated``, head ``h`` is multiplied by ``sigmoid(wg x)_h`` (``wg [n_heads, dim]``);
    * ``wo`` on the concatenated heads.  ``own_kv=False``: a run that reads another run's keys
      and values has neither ``wk`` nor ``wv``.

    The cache holds ``2 * n_kv_heads`` key heads (map-major: all first maps, then all second
    maps, the order q is projected in too, so that each map is ordinary grouped attention) and
    ``n_kv_heads`` value heads.  One stacked product gives q, k, v and the gate; one kernel
    rotates, stores and takes the gate's sigmoid; the attention kernel returns both maps in
    32-bit, and one kernel combines, normalises and gates them."""

    graph_safe = True

    def __init__(self, env: BuildEnv, *, dim: int, n_heads: int, n_kv_heads: int, head_dim: int, v_head_dim: int,
                 scale: float, lambda_init: float, norm_eps: float, rot_dims: int, rot_base: float,
                 rot_factor: float = 1.0, rot_pairing: str = "half", gated: bool = True, own_kv: bool = True):
        if n_heads % n_kv_heads != 0:
            raise ValueError(f"n_heads ({n_heads}) must be a multiple of n_kv_heads ({n_kv_heads})")
        if rot_dims < 0 or rot_dims % 2 or rot_dims > head_dim:
            raise ValueError(f"rot_dims must be even and at most head_dim ({head_dim}), got {rot_dims}")
        if rot_pairing not in ("half", "interleaved"):
            raise ValueError(f"rot_pairing must be 'half' or 'interleaved', got {rot_pairing!r}")
        self.env = env
        self.dim, self.n_heads, self.n_kv_heads = int(dim), int(n_heads), int(n_kv_heads)
        self.head_dim, self.v_head_dim = int(head_dim), int(v_head_dim)
        self.scale, self.lambda_init, self.norm_eps = float(scale), float(lambda_init), float(norm_eps)
        self.rot_dims, self.rot_pairing = int(rot_dims), rot_pairing
        self.gated, self.own_kv = bool(gated), bool(own_kv)
        self.n_q = 2 * self.n_heads * self.head_dim
        self.n_k = 2 * self.n_kv_heads * self.head_dim
        self.n_v = self.n_kv_heads * self.v_head_dim
        env.ops.check_attention_sizes(2 * self.n_heads, 2 * self.n_kv_heads, self.head_dim, env.dtype, v_head_dim=self.v_head_dim)
        self.table = precise_rotary_table(max(self.rot_dims, 2), rot_base, rot_factor, env.max_positions, env.device)
        self.lam = 0.0
        self.w_in: Optional[torch.Tensor] = None
        self.wo: Optional[torch.Tensor] = None

    def cache_need(self) -> CacheNeed:
        return CacheNeed("full", 2 * self.n_kv_heads, self.head_dim, None, self.v_head_dim, 0, self.n_kv_heads)

    def expected_tensors(self) -> Dict[str, ExpectedTensor]:
        out = {"wq.weight": ExpectedTensor((self.n_q, self.dim)),
               "wo.weight": ExpectedTensor((self.dim, self.n_heads * self.v_head_dim))}
        if self.own_kv:
            out["wk.weight"] = ExpectedTensor((self.n_k, self.dim))
            out["wv.weight"] = ExpectedTensor((self.n_v, self.dim))
        for name in ("lambda_q1", "lambda_k1", "lambda_q2", "lambda_k2"):
            out[name] = ExpectedTensor((self.head_dim,))
        if self.gated:
            out["wg.weight"] = ExpectedTensor((self.n_heads, self.dim))
        return out

    def _map_major(self, w: torch.Tensor, heads: int) -> torch.Tensor:
        """Rows ``[head][map][coordinate]`` as ``[map][head][coordinate]``."""
        return w.view(heads, 2, self.head_dim, self.dim).transpose(0, 1).reshape(2 * heads * self.head_dim, self.dim)

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        rows = [self._map_major(as_compute(tensors["wq.weight"], self.env), self.n_heads)]
        if self.own_kv:
            rows += [self._map_major(as_compute(tensors["wk.weight"], self.env), self.n_kv_heads),
                     as_compute(tensors["wv.weight"], self.env)]
        if self.gated:
            rows.append(as_compute(tensors["wg.weight"], self.env))
        self.w_in = torch.cat(rows).contiguous()                               # rows [wq; wk; wv; wg]
        dots = [float((tensors[f"lambda_q{i}"].double() * tensors[f"lambda_k{i}"].double()).sum()) for i in (1, 2)]
        self.lam = math.exp(dots[0]) - math.exp(dots[1]) + self.lambda_init
        self.wo = as_compute(tensors["wo.weight"], self.env)

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.wo))     # (the table is gathered by rows)

    def forward(self, x: torch.Tensor, ctx, cache) -> PendingProduct:
        ops = self.env.ops
        H, G = self.n_heads, self.n_kv_heads
        if cache.writes != self.own_kv:
            raise RuntimeError("a differential attention layer owns its keys and values exactly when it projects them")
        proj = ops.linear(x, self.w_in, partials_ok=True)
        q, gate = ops.rope_store(
            proj, ctx.positions, self.table, n_q_heads=2 * H, n_k_heads=2 * G if self.own_kv else 0,
            n_v_heads=G if self.own_kv else 0, head_dim=self.head_dim, v_head_dim=self.v_head_dim, rot_dims=self.rot_dims,
            interleaved=self.rot_pairing == "interleaved", n_extra=H if self.gated else 0,
            k_pages=cache.k_pages if self.own_kv else None, v_pages=cache.v_pages if self.own_kv else None,
            slot_mapping=cache.slot_mapping, page_size=cache.page_size, out_dtype=self.env.dtype)
        maps = ops.paged_attention(
            q, cache.k_pages, cache.v_pages, cache.block_table, ctx.q_start, ctx.kv_len, n_seqs=ctx.n_seqs,
            max_q_len=ctx.max_q_len, max_kv_len=ctx.max_kv_len, scale=self.scale, window=None, page_size=cache.page_size,
            n_v_heads=G, out_dtype=torch.float32)                              # [T, 2 H, v_head_dim], map-major
        o = ops.differential_combine(maps, self.lam, eps=self.norm_eps, out_scale=1.0 - self.lambda_init, gate=gate,
                                     out_dtype=self.env.dtype)
        return PendingProduct(o, self.wo)


@register_mixer("rotary_gated_attention")
class RotaryGatedAttention(Mixer):
    """Grouped-query attention with rotary positions and the options below, all of them numbers or
    switches of the spec:

    * projections ``wq, wk, wv`` (and ``wo``) with optional biases (``qkv_bias``, ``out_bias``), keys and
      values of sizes of their own (``head_dim``, ``v_head_dim``);
    * rotation of the first ``rot_dims`` coordinates of every q and k head by ``p * rot_base^(-2i/rot_dims)``
      (``rot_pairing`` ``"interleaved"``: coordinate ``2i`` with ``2i + 1``; ``"half"``: ``i`` with ``i + rot_dims / 2``);
    * score ``= q . k * scale``, then, with ``softcap = c > 0``, ``c * tanh(score / c)``;
    * causal, optionally behind a sliding ``window``;
    * softmax whose denominator, with ``sinks``, also holds ``exp(sinks[h])``: a learned number per head
      (tensor ``sinks``) that stands for a key without a value and is neither scaled nor capped;
    * an output gate ``sigmoid(wg x)``, one number per head (``gate="head"``) or per element
      (``"element"``), ahead of ``wo``.

    One stacked product gives q, k, v and the gate's logits; one kernel adds the biases, rotates,
    stores keys and values and takes the gate's sigmoid; cap, sink and gate live in the attention
    kernel; the output bias is added where the output product is added up."""

    graph_safe = True

    def __init__(self, env: BuildEnv, *, dim: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 v_head_dim: Optional[int] = None, scale: float, softcap: float = 0.0, sinks: bool = False,
                 rot_dims: int = 0, rot_base: float = 10000.0, rot_pairing: str = "interleaved", window: Optional[int] = None,
                 qkv_bias: bool = False, out_bias: bool = False, gate: Optional[str] = None):
        if n_heads % n_kv_heads != 0:
            raise ValueError(f"n_heads ({n_heads}) must be a multiple of n_kv_heads ({n_kv_heads})")
        if rot_dims < 0 or rot_dims % 2 or rot_dims > head_dim:
            raise ValueError(f"rot_dims must be even and at most head_dim ({head_dim}), got {rot_dims}")
        if rot_pairing not in ("half", "interleaved"):
            raise ValueError(f"rot_pairing must be 'half' or 'interleaved', got {rot_pairing!r}")
        if gate not in (None, "element", "head"):
            raise ValueError(f"gate must be None, 'element' or 'head', got {gate!r}")
        if softcap < 0:
            raise ValueError(f"softcap must not be negative, got {softcap}")
        self.env = env
        self.dim, self.n_heads, self.n_kv_heads = int(dim), int(n_heads), int(n_kv_heads)
        self.head_dim = int(head_dim)
        self.v_head_dim = int(v_head_dim if v_head_dim is not None else head_dim)
        self.scale, self.softcap = float(scale), float(softcap)
        self.has_sinks, self.qkv_bias, self.out_bias, self.gate = bool(sinks), bool(qkv_bias), bool(out_bias), gate
        self.rot_dims, self.interleaved = int(rot_dims), rot_pairing == "interleaved"
        self.window = None if window is None else int(window)
        self.n_q, self.n_k, self.n_v = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim, self.n_kv_heads * self.v_head_dim
        self.n_g = {None: 0, "head": self.n_heads, "element": self.n_heads * self.v_head_dim}[gate]
        env.ops.check_attention_sizes(self.n_heads, self.n_kv_heads, self.head_dim, env.dtype, v_head_dim=self.v_head_dim)
        self.table = precise_rotary_table(max(self.rot_dims, 2), rot_base, 1.0, env.max_positions, env.device)
        self.w_in = self.b_in = self.sinks = self.wo = self.bo = None

    def cache_need(self) -> CacheNeed:
        if self.window is None:
            return CacheNeed("full", self.n_kv_heads, self.head_dim, None, self.v_head_dim)
        return CacheNeed("window", self.n_kv_heads, self.head_dim, self.window, self.v_head_dim)

    def expected_tensors(self) -> Dict[str, ExpectedTensor]:
        out = {"wq.weight": ExpectedTensor((self.n_q, self.dim)), "wk.weight": ExpectedTensor((self.n_k, self.dim)),
               "wv.weight": ExpectedTensor((self.n_v, self.dim)),
               "wo.weight": ExpectedTensor((self.dim, self.n_heads * self.v_head_dim))}
        if self.qkv_bias:
            out.update({"wq.bias": ExpectedTensor((self.n_q,)), "wk.bias": ExpectedTensor((self.n_k,)),
                        "wv.bias": ExpectedTensor((self.n_v,))})
        if self.out_bias:
            out["wo.bias"] = ExpectedTensor((self.dim,))
        if self.has_sinks:
            out["sinks"] = ExpectedTensor((self.n_heads,))
        if self.gate:
            out["wg.weight"] = ExpectedTensor((self.n_g, self.dim))
        return out

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        f32 = dict(device=self.env.device, dtype=torch.float32)
        names = ["wq.weight", "wk.weight", "wv.weight"] + (["wg.weight"] if self.gate else [])
        self.w_in = torch.cat([as_compute(tensors[n], self.env) for n in names])       # rows [wq; wk; wv; wg]
        if self.qkv_bias:
            self.b_in = torch.cat([tensors[n].to(**f32) for n in ("wq.bias", "wk.bias", "wv.bias")]
                                  + [torch.zeros(self.n_g, **f32)]).contiguous()
        if self.out_bias:
            self.bo = tensors["wo.bias"].to(**f32).contiguous()
        if self.has_sinks:
            self.sinks = tensors["sinks"].to(**f32).contiguous()
        self.wo = as_compute(tensors["wo.weight"], self.env)

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.wo))

    def forward(self, x: torch.Tensor, ctx, cache) -> PendingProduct:
        ops = self.env.ops
        proj = ops.linear(x, self.w_in, partials_ok=True)
        q, gate = ops.rope_store(
            proj, ctx.positions, self.table, n_q_heads=self.n_heads, n_k_heads=self.n_kv_heads, n_v_heads=self.n_kv_heads,
            head_dim=self.head_dim, v_head_dim=self.v_head_dim, rot_dims=self.rot_dims, interleaved=self.interleaved,
            n_extra=self.n_g, k_pages=cache.k_pages, v_pages=cache.v_pages, slot_mapping=cache.slot_mapping,
            page_size=cache.page_size, out_dtype=self.env.dtype, bias=self.b_in)
        o = ops.paged_attention(
            q, cache.k_pages, cache.v_pages, cache.block_table, ctx.q_start, ctx.kv_len, n_seqs=ctx.n_seqs,
            max_q_len=ctx.max_q_len, max_kv_len=ctx.max_kv_len, scale=self.scale, window=self.window,
            page_size=cache.page_size, gate=gate, softcap=self.softcap, sinks=self.sinks, impl="auto")
        return PendingProduct(o.view(o.shape[0], self.n_heads * self.v_head_dim), self.wo, bias=self.bo)
