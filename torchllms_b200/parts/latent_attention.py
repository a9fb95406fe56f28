"""Latent attention: keys and values of every head are linear in one small cached vector.

Per token the mixer stores only a latent ``c = norm(w_down x)`` of ``rank`` elements.  Head ``h``
has ``k_h = Uk_h c`` and ``v_h = Uv_h c``; its score against a query ``q_h`` is
``q_h . (Uk_h c) = (Uk_h^T q_h) . c``, and its output ``sum_j p_j Uv_h c_j = Uv_h (sum_j p_j c_j)``.
So the attention itself runs over the stored latents with one shared "head" of size ``rank`` for
keys and values alike (queries ``Uk_h^T q_h``, one per head), and the two small per-head
products stand before and after it; no key or value is ever expanded, for prompts and decoded
tokens alike.  There is no rotation: this mixer knows of positions only through its causal
sliding window.

A run that reads another run's cache (``own_latent=False``) has no down-projection: it takes
the latents that the other run stored, with up-projections, queries, window and gate of its own.

The output gate is one number per head, ``sigmoid(wg x)_h``; it is applied to the attended
latent of the head (the up-projection that follows is linear, so it is the same number).
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..kernels.lazy import PendingProduct
from ..weights.loader import ExpectedTensor
from .base import BuildEnv, CacheNeed, Mixer, as_compute, register_mixer


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    graph_safe = True

    def __init__(self, env: BuildEnv, *, dim: int, n_heads: int, head_dim: int, v_head_dim: int, rank: int,
                 scale: float, window: Optional[int] = None, norm_eps: float = 1e-6, gated: bool = True,
                 own_latent: bool = True):
        self.env = env
        self.dim, self.n_heads, self.head_dim, self.v_head_dim = int(dim), int(n_heads), int(head_dim), int(v_head_dim)
        self.rank = int(rank)
        self.scale = float(scale)
        self.window = None if window is None else int(window)
        self.norm_eps = float(norm_eps)
        self.gated, self.own_latent = bool(gated), bool(own_latent)
        self.n_q = self.n_heads * self.head_dim
        self.n_c = self.rank if self.own_latent else 0
        self.n_g = self.n_heads if self.gated else 0
        env.ops.check_attention_sizes(self.n_heads, 1, self.rank, env.dtype)
        self.w_in: Optional[torch.Tensor] = None
        self.latent_norm_w: Optional[torch.Tensor] = None
        self.w_uk_t: Optional[torch.Tensor] = None      # [heads, rank, head_dim]: Uk_h^T
        self.w_uv: Optional[torch.Tensor] = None        # [heads, v_head_dim, rank]
        self.wo: Optional[torch.Tensor] = None

    def cache_need(self) -> CacheNeed:
        # one vector per token, read as key and as value: nothing is stored for values
        if self.window is None:
            return CacheNeed("full", 1, self.rank, None, 0)
        return CacheNeed("window", 1, self.rank, self.window, 0)

    def expected_tensors(self) -> Dict[str, ExpectedTensor]:
        out = {
            "wq.weight": ExpectedTensor((self.n_q, self.dim)),
            "w_up_k.weight": ExpectedTensor((self.n_q, self.rank)),
            "w_up_v.weight": ExpectedTensor((self.n_heads * self.v_head_dim, self.rank)),
            "wo.weight": ExpectedTensor((self.dim, self.n_heads * self.v_head_dim)),
        }
        if self.own_latent:
            out["w_down.weight"] = ExpectedTensor((self.rank, self.dim))
            out["latent_norm.weight"] = ExpectedTensor((self.rank,))
        if self.gated:
            out["wg.weight"] = ExpectedTensor((self.n_heads, self.dim))
        return out

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        names = ["wq.weight"] + (["w_down.weight"] if self.own_latent else []) + (["wg.weight"] if self.gated else [])
        self.w_in = torch.cat([as_compute(tensors[n], self.env) for n in names])       # rows [wq; w_down; wg]
        if self.own_latent:
            self.latent_norm_w = tensors["latent_norm.weight"].to(device=self.env.device, dtype=torch.float32).contiguous()
        uk = as_compute(tensors["w_up_k.weight"], self.env).view(self.n_heads, self.head_dim, self.rank)
        self.w_uk_t = uk.transpose(1, 2).contiguous()
        self.w_uv = as_compute(tensors["w_up_v.weight"], self.env).view(self.n_heads, self.v_head_dim, self.rank).contiguous()
        self.wo = as_compute(tensors["wo.weight"], self.env)

    def forward(self, x: torch.Tensor, ctx, cache) -> PendingProduct:
        ops = self.env.ops
        if cache.writes != self.own_latent:
            raise RuntimeError("a latent mixer stores latents exactly when it has a down-projection of its own")
        proj = ops.linear(x, self.w_in, partials_ok=True)
        q, gate = ops.project_and_store(
            proj, n_q=self.n_q, n_k=self.n_c, n_v=0, n_extra=self.n_g, bias=None,
            q_norm=None, k_norm=self.latent_norm_w, eps=self.norm_eps,
            k_pages=cache.k_pages if cache.writes else None, v_pages=None,
            slot_mapping=cache.slot_mapping, page_size=cache.page_size, out_dtype=self.env.dtype)
        q_lat = ops.head_linear(q.view(-1, self.n_heads, self.head_dim), self.w_uk_t)          # [T, H, rank]
        o_lat = ops.paged_attention(
            q_lat, cache.k_pages, cache.k_pages, cache.block_table, ctx.q_start, ctx.kv_len,
            n_seqs=ctx.n_seqs, max_q_len=ctx.max_q_len, max_kv_len=ctx.max_kv_len, scale=self.scale,
            window=self.window, page_size=cache.page_size, gate=gate, impl="auto")
        o = ops.head_linear(o_lat, self.w_uv)                                                    # [T, H, v_head_dim]
        return PendingProduct(o.view(o.shape[0], self.n_heads * self.v_head_dim), self.wo)


@register_mixer("rotary_latent_attention")
class RotaryLatentAttention(Mixer):
    """Latent attention whose heads also carry a rotated part, with queries through a latent of
    their own:

    * ``c_q = norm(wq_down x)`` (``q_rank`` numbers, plain weight), ``q = wq_up c_q``, head by head
      ``[head_dim unrotated | rot_dim rotated]``;
    * ``w_down x`` has ``rank + rot_dim`` rows: the first ``rank``, normed, are the latent ``c``; the
      last ``rot_dim`` are one key part shared by all heads, rotated by the position (all of it;
      ``rot_pairing`` ``"half"``: coordinate ``i`` with ``i + rot_dim / 2``, or ``"interleaved"``);
    * head ``h``: ``k_h = Uk_h c``, ``v_h = Uv_h c``, score ``(q_h . k_h + q_rot_h . k_rot) * scale``, causal
      softmax (optionally behind a window);
    * the concatenated heads times ``sigmoid(wg x)`` element by element (``gate="element"``), or head by
      head (``"head"``), or as they are (``None``); then ``wo``.

    The cache keeps ``[c | k_rot]`` per token and nothing else.  As in :class:`LatentAttention` the
    up-projections are absorbed: the attention runs with queries ``[Uk_h^T q_h | q_rot_h]`` over the
    stored vectors as one shared key head, the values being the stored vectors' first ``rank``
    coordinates, and ``Uv_h`` is applied to the attended latent."""

    graph_safe = True

    def __init__(self, env: BuildEnv, *, dim: int, n_heads: int, head_dim: int, rot_dim: int, v_head_dim: int, q_rank: int,
                 rank: int, scale: float, rot_base: float, rot_pairing: str = "half", window: Optional[int] = None,
                 norm_eps: float = 1e-6, gate: Optional[str] = "element"):
        if rot_dim < 0 or rot_dim % 2:
            raise ValueError(f"rot_dim must be even and not negative, got {rot_dim}")
        if rot_pairing not in ("half", "interleaved"):
            raise ValueError(f"rot_pairing must be 'half' or 'interleaved', got {rot_pairing!r}")
        if gate not in (None, "element", "head"):
            raise ValueError(f"gate must be None, 'element' or 'head', got {gate!r}")
        from .rope import precise_rotary_table
        self.env = env
        self.dim, self.n_heads, self.head_dim, self.rot_dim = int(dim), int(n_heads), int(head_dim), int(rot_dim)
        self.v_head_dim, self.q_rank, self.rank = int(v_head_dim), int(q_rank), int(rank)
        self.scale, self.norm_eps = float(scale), float(norm_eps)
        self.window = None if window is None else int(window)
        self.interleaved, self.gate = rot_pairing == "interleaved", gate
        self.q_head = self.head_dim + self.rot_dim            # a head of the projected q
        self.key_dim = self.rank + self.rot_dim               # a stored vector
        self.n_g = {None: 0, "head": self.n_heads, "element": self.n_heads * self.v_head_dim}[gate]
        env.ops.check_attention_sizes(self.n_heads, 1, self.key_dim, env.dtype, v_head_dim=self.rank)
        self.table = precise_rotary_table(max(self.rot_dim, 2), rot_base, 1.0, env.max_positions, env.device)
        self.w_in = self.q_norm_w = self.latent_norm_w = self.wq_up = self.w_uk_t = self.w_uv = self.wo = None

    def cache_need(self) -> CacheNeed:
        # one vector per token, read as key and (its first part) as value: nothing is stored for values
        if self.window is None:
            return CacheNeed("full", 1, self.key_dim, None, 0)
        return CacheNeed("window", 1, self.key_dim, self.window, 0)

    def expected_tensors(self) -> Dict[str, ExpectedTensor]:
        H = self.n_heads
        out = {
            "wq_down.weight": ExpectedTensor((self.q_rank, self.dim)), "q_norm.weight": ExpectedTensor((self.q_rank,)),
            "wq_up.weight": ExpectedTensor((H * self.q_head, self.q_rank)),
            "w_down.weight": ExpectedTensor((self.key_dim, self.dim)), "latent_norm.weight": ExpectedTensor((self.rank,)),
            "w_up_k.weight": ExpectedTensor((H * self.head_dim, self.rank)),
            "w_up_v.weight": ExpectedTensor((H * self.v_head_dim, self.rank)),
            "wo.weight": ExpectedTensor((self.dim, H * self.v_head_dim)),
        }
        if self.gate:
            out["wg.weight"] = ExpectedTensor((self.n_g, self.dim))
        return out

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        f32 = dict(device=self.env.device, dtype=torch.float32)
        names = ["wq_down.weight", "w_down.weight"] + (["wg.weight"] if self.gate else [])
        self.w_in = torch.cat([as_compute(tensors[n], self.env) for n in names])       # rows [wq_down; w_down; wg]
        self.q_norm_w = tensors["q_norm.weight"].to(**f32).contiguous()
        self.latent_norm_w = tensors["latent_norm.weight"].to(**f32).contiguous()
        self.wq_up = as_compute(tensors["wq_up.weight"], self.env)
        uk = as_compute(tensors["w_up_k.weight"], self.env).view(self.n_heads, self.head_dim, self.rank)
        self.w_uk_t = uk.transpose(1, 2).contiguous()                                   # [heads, rank, head_dim]: Uk_h^T
        self.w_uv = as_compute(tensors["w_up_v.weight"], self.env).view(self.n_heads, self.v_head_dim, self.rank).contiguous()
        self.wo = as_compute(tensors["wo.weight"], self.env)

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.wq_up, self.w_uk_t, self.w_uv, self.wo))

    def forward(self, x: torch.Tensor, ctx, cache) -> PendingProduct:
        ops = self.env.ops
        H = self.n_heads
        if not cache.writes:
            raise RuntimeError("a rotary latent mixer stores its own latents")
        proj = ops.linear(x, self.w_in, partials_ok=True)
        cq, gate = ops.latent_store(
            proj, ctx.positions, self.table, n_q=self.q_rank, n_latent=self.rank, n_rot=self.rot_dim, n_extra=self.n_g,
            q_norm=self.q_norm_w, latent_norm=self.latent_norm_w, eps=self.norm_eps, interleaved=self.interleaved,
            k_pages=cache.k_pages, slot_mapping=cache.slot_mapping, page_size=cache.page_size, out_dtype=self.env.dtype)
        q = ops.linear(cq, self.wq_up).view(-1, H, self.q_head)                         # [T, H, head_dim + rot_dim]
        q_lat = ops.latent_query(q, self.w_uk_t, ctx.positions, self.table, rot_dim=self.rot_dim,
                                 interleaved=self.interleaved)                            # [T, H, rank + rot_dim]
        o_lat = ops.paged_attention(
            q_lat, cache.k_pages, cache.k_pages, cache.block_table, ctx.q_start, ctx.kv_len,
            n_seqs=ctx.n_seqs, max_q_len=ctx.max_q_len, max_kv_len=ctx.max_kv_len, scale=self.scale,
            window=self.window, page_size=cache.page_size, value_dim=self.rank,
            gate=gate if self.gate == "head" else None, impl="auto")                      # [T, H, rank]
        o = ops.head_linear(o_lat, self.w_uv, gate=gate if self.gate == "element" else None)     # [T, H, v_head_dim]
        return PendingProduct(o.view(o.shape[0], H * self.v_head_dim), self.wo)
