"""The arrangements of a layer: where the norms sit and how the residual is carried.

Pre-norm residual block.

Reference: ``TransformerBlock.forward`` (torchllms/models/networks.py:635-644):
``h = x + mixer(norm1(x)); out = h + ffn(norm2(h))``.  The sums are left pending
on the residual so the following norm adds them in 32-bit in the same pass.
"""

from __future__ import annotations

import dataclasses
from typing import Dict, Mapping, Optional

import torch

from ..kernels.lazy import NormedSum, PendingProduct
from ..weights.loader import ExpectedTensor
from .base import (FEED_FORWARDS, MIXERS, NORMS, Block, BuildEnv, Residual, StateNeed, as_compute, join_states,
                   register_block, state_field)
from .norm import RMSNorm
from .spec import PartSpec


@register_block("prenorm")
class PreNormBlock(Block):
    """Sub-part tensor prefixes are parameters, so the block does not know whose names they are."""

    def __init__(self, env: BuildEnv, *, mixer: PartSpec, feed_forward: PartSpec,
                 mixer_norm: PartSpec, ffn_norm: PartSpec,
                 mixer_prefix: str, ffn_prefix: str, mixer_norm_prefix: str, ffn_norm_prefix: str):
        self.env = env
        self.mixer = MIXERS.build(mixer, env)
        self.feed_forward = FEED_FORWARDS.build(feed_forward, env)
        self.mixer_norm = NORMS.build(mixer_norm, env)
        self.ffn_norm = NORMS.build(ffn_norm, env)
        self.graph_safe = all(x.graph_safe for x in (self.mixer, self.feed_forward, self.mixer_norm, self.ffn_norm))
        self._subparts = ((mixer_prefix, self.mixer), (ffn_prefix, self.feed_forward),
                          (mixer_norm_prefix, self.mixer_norm), (ffn_norm_prefix, self.ffn_norm))

    def cache_need(self):
        return self.mixer.cache_need()

    def state_need(self):
        return self.mixer.state_need()

    def expected_tensors(self) -> Dict[str, ExpectedTensor]:
        out: Dict[str, ExpectedTensor] = {}
        for prefix, sub in self._subparts:
            for name, e in sub.expected_tensors().items():
                out[f"{prefix}.{name}"] = e
        return out

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for prefix, sub in self._subparts:
            sub.load({name: tensors[f"{prefix}.{name}"] for name in sub.expected_tensors()})

    def forward(self, residual: Residual, ctx, cache) -> None:
        x = self._normed(self.mixer_norm, self.mixer, residual)
        residual.delta = self.mixer.forward(x, ctx, cache)
        x = self._normed(self.ffn_norm, self.feed_forward, residual)
        residual.delta = self.feed_forward.forward(x, ctx)

    @staticmethod
    def _normed(norm, reader, residual: Residual):
        """The rows for ``reader``: with their normalisation deferred where both sides can."""
        if norm.can_defer and reader.takes_row_scaled:
            return norm.forward(residual, deferred_ok=True)
        return norm.forward(residual)


@register_block("outnorm")
class OutputNormBlock(Block):
    """The norm sits on each sublayer's output and nowhere else: ``x += norm1(mixer(x))``, then
    ``x += norm2(ff(x))``; both sublayers read the stream itself.  A layer may have no feed-forward
    (``feed_forward=None``), in which case it has no second norm either.

    The sum is taken by the norm's own kernel (``Norm.fold_normed``), which also leaves the new
    stream in the activation dtype for the next reader, so nothing is pending between sublayers."""

    reads_stream = True      # its first sublayer takes the stream as it is: whoever makes the stream may leave ``Residual.rows``

    def __init__(self, env: BuildEnv, *, mixer: PartSpec, feed_forward: Optional[PartSpec],
                 mixer_norm: PartSpec, ffn_norm: Optional[PartSpec],
                 mixer_prefix: str, ffn_prefix: str, mixer_norm_prefix: str, ffn_norm_prefix: str):
        self.env = env
        self.mixer = MIXERS.build(mixer, env)
        self.mixer_norm = NORMS.build(mixer_norm, env)
        self.feed_forward = None if feed_forward is None else FEED_FORWARDS.build(feed_forward, env)
        self.ffn_norm = None if feed_forward is None else NORMS.build(ffn_norm, env)
        self._subparts = [(mixer_prefix, self.mixer), (mixer_norm_prefix, self.mixer_norm)]
        if self.feed_forward is not None:
            self._subparts += [(ffn_prefix, self.feed_forward), (ffn_norm_prefix, self.ffn_norm)]
        self.graph_safe = all(sub.graph_safe for _p, sub in self._subparts)

    def cache_need(self):
        return self.mixer.cache_need()

    def state_need(self):
        return self.mixer.state_need()

    def expected_tensors(self) -> Dict[str, ExpectedTensor]:
        out: Dict[str, ExpectedTensor] = {}
        for prefix, sub in self._subparts:
            for name, e in sub.expected_tensors().items():
                out[f"{prefix}.{name}"] = e
        return out

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for prefix, sub in self._subparts:
            sub.load({name: tensors[f"{prefix}.{name}"] for name in sub.expected_tensors()})

    def _input(self, residual: Residual) -> torch.Tensor:
        """The stream as a sublayer reads it: in the activation dtype."""
        if residual.delta is not None:
            raise RuntimeError("an output-norm block cannot follow a block that leaves its sum pending")
        if residual.rows is None:
            residual.rows = self.env.ops.stream_rows(residual.h, self.env.dtype)
        return residual.rows

    def forward(self, residual: Residual, ctx, cache) -> None:
        self.mixer_norm.fold_normed(residual, self.mixer.forward(self._input(residual), ctx, cache))
        if self.feed_forward is not None:
            self.ffn_norm.fold_normed(residual, self.feed_forward.forward(self._input(residual), ctx))


@register_block("sandwich")
class SandwichBlock(Block):
    """A norm in front of each sublayer and another on its output: ``x += out_norm1(mixer(norm1(x)))``,
    then ``x += out_norm2(ff(norm2(x)))``.  A layer may have no feed-forward.

    With ``depth_inputs = n`` the layer ends in an average over depth: what goes on is
    ``sum_j c[j] X_j`` over the first ``n`` levels of the model's history (level 0 the embedding
    output, level ``j`` the result of the ``j``-th layer run before any averaging, the last of the
    ``n`` this layer's own), with the coefficients in the layer's tensor ``depth_tensor``.  Such a
    block needs a model that keeps its history (``ModelSpec.keeps_history``).

    The output norm's kernel adds to the stream and, where a feed-forward follows, also takes the
    norm in front of it, so two kernels stand between the mixer's and the feed-forward's products."""

    def __init__(self, env: BuildEnv, *, mixer: PartSpec, feed_forward: Optional[PartSpec],
                 mixer_norm: PartSpec, mixer_out_norm: PartSpec, ffn_norm: Optional[PartSpec],
                 ffn_out_norm: Optional[PartSpec], mixer_prefix: str, ffn_prefix: str, mixer_norm_prefix: str,
                 mixer_out_norm_prefix: str, ffn_norm_prefix: str, ffn_out_norm_prefix: str,
                 depth_inputs: Optional[int] = None, depth_tensor: str = "depth"):
        self.env = env
        self.mixer = MIXERS.build(mixer, env)
        self.mixer_norm = NORMS.build(mixer_norm, env)
        self.input_norm = self.mixer_norm
        self.mixer_out_norm = NORMS.build(mixer_out_norm, env)
        self._subparts = [(mixer_prefix, self.mixer), (mixer_norm_prefix, self.mixer_norm),
                          (mixer_out_norm_prefix, self.mixer_out_norm)]
        self.feed_forward = self.ffn_norm = self.ffn_out_norm = None
        if feed_forward is not None:
            self.feed_forward = FEED_FORWARDS.build(feed_forward, env)
            self.ffn_norm = NORMS.build(ffn_norm, env)
            self.ffn_out_norm = NORMS.build(ffn_out_norm, env)
            self._subparts += [(ffn_prefix, self.feed_forward), (ffn_norm_prefix, self.ffn_norm),
                               (ffn_out_norm_prefix, self.ffn_out_norm)]
        self.depth_inputs = None if depth_inputs is None else int(depth_inputs)
        if self.depth_inputs is not None and self.depth_inputs < 1:
            raise ValueError(f"an average over depth reads at least one level, got {depth_inputs}")
        self.depth_tensor = depth_tensor
        self.depth_coef: Optional[torch.Tensor] = None
        self.graph_safe = all(sub.graph_safe for _p, sub in self._subparts)

    def cache_need(self):
        return self.mixer.cache_need()

    def state_need(self):
        return self.mixer.state_need()

    def expected_tensors(self) -> Dict[str, ExpectedTensor]:
        out: Dict[str, ExpectedTensor] = {}
        for prefix, sub in self._subparts:
            for name, e in sub.expected_tensors().items():
                out[f"{prefix}.{name}"] = e
        if self.depth_inputs is not None:
            out[self.depth_tensor] = ExpectedTensor((self.depth_inputs,))
        return out

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for prefix, sub in self._subparts:
            sub.load({name: tensors[f"{prefix}.{name}"] for name in sub.expected_tensors()})
        if self.depth_inputs is not None:
            self.depth_coef = tensors[self.depth_tensor].to(device=self.env.device, dtype=torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return sum(sub.weight_bytes() for _p, sub in self._subparts)

    def forward(self, residual: Residual, ctx, cache) -> None:
        if residual.delta is not None:
            raise RuntimeError("a sandwich block cannot follow a block that leaves its sum pending")
        if residual.normed is not None and residual.normed[0] is self.mixer_norm:
            x = residual.normed[1]                       # the block before took this norm along with its last kernel
        else:
            x = self.mixer_norm.forward(residual)
        residual.normed = None
        y = self.mixer.forward(x, ctx, cache)
        if self.feed_forward is None:
            self.mixer_out_norm.fold_normed(residual, y, want_rows=False)
        else:
            x = self.mixer_out_norm.fold_normed(residual, y, then=self.ffn_norm)
            self.ffn_out_norm.fold_normed(residual, self.feed_forward.forward(x, ctx), want_rows=False)
        if self.depth_inputs is not None:
            history, level = residual.history, residual.level
            if history is None or self.depth_inputs != level + 2:
                raise RuntimeError(f"this layer averages over {self.depth_inputs} levels of the model's history, "
                                   f"but {'there is none' if history is None else f'{level + 2} exist'}")
            nxt = history[level + 2]
            follow = residual.next_norm
            if isinstance(follow, RMSNorm):
                # the average and the next layer's input norm of it in one kernel
                rows = self.env.ops.depth_mix(history, self.depth_coef, self.depth_inputs, nxt, then_weight=follow.weight,
                                              then_eps=follow.eps, out_dtype=self.env.dtype)
                residual.normed = (follow, rows)
            else:
                self.env.ops.depth_mix(history, self.depth_coef, self.depth_inputs, nxt)
            residual.h, residual.rows, residual.level = nxt, None, level + 1


@register_block("parallel")
class ParallelBlock(Block):
    """One norm in front, both sublayers reading its output, one sum: with ``h = norm(x)``,
    ``x += mixer(h') + ff(h)``.  A layer may have no feed-forward.

    ``input_conv_taps = n``: what the mixer reads is ``h' = h + conv(h)``, a causal convolution over
    time on every channel (tensor ``input_conv_tensor`` ``[dim, n]``, the last column the current
    token's, zeros before a request's start); the last ``n - 1`` rows of ``h`` are part of the
    request's state.  The feed-forward reads ``h`` as it is.

    ``token_side_dim = s``: after the sum the layer takes an input of its own from the token:
    ``g = gelu_tanh(W_gate x) * table[token]`` (``s`` numbers), ``y = W_proj g``, ``x += norm(y)`` with
    a plain-weight RMS norm.  Tensors ``<side_prefix>.table [vocab, s]``, ``.gate.weight``,
    ``.proj.weight``, ``.norm.weight``.

    The sum is one kernel in 32-bit that also leaves the new stream in the activation dtype; a mixer
    that returns normed terms (:class:`~torchllms_b200.kernels.lazy.NormedSum`) has its norms taken
    there.  The side input's norm kernel also takes the next layer's input norm."""

    def __init__(self, env: BuildEnv, *, mixer: PartSpec, feed_forward: Optional[PartSpec], norm: PartSpec,
                 mixer_prefix: str, ffn_prefix: str, norm_prefix: str, input_conv_taps: int = 0,
                 input_conv_tensor: str = "input_conv", token_side_dim: int = 0, token_side_vocab: int = 0,
                 token_side_eps: float = 1e-6, side_prefix: str = "side"):
        self.env = env
        self.mixer = MIXERS.build(mixer, env)
        self.norm = NORMS.build(norm, env)
        self.input_norm = self.norm
        self.feed_forward = None if feed_forward is None else FEED_FORWARDS.build(feed_forward, env)
        self._subparts = [(mixer_prefix, self.mixer), (norm_prefix, self.norm)]
        if self.feed_forward is not None:
            self._subparts.append((ffn_prefix, self.feed_forward))
        self.taps, self.conv_tensor = int(input_conv_taps), input_conv_tensor
        self.side_dim, self.side_vocab, self.side_prefix = int(token_side_dim), int(token_side_vocab), side_prefix
        self.side_norm = None
        if self.side_dim:
            self.side_norm = NORMS.build(PartSpec("rmsnorm", {"dim": env.dim, "eps": float(token_side_eps)}), env)
            self._subparts.append((f"{side_prefix}.norm", self.side_norm))
        self._need = join_states([("input_conv", StateNeed((self.taps - 1, env.dim)) if self.taps > 1 else None),
                                  ("mixer", self.mixer.state_need())])
        self.graph_safe = all(sub.graph_safe for _p, sub in self._subparts)
        self.conv_w = self.side_table = self.side_gate_w = self.side_proj_w = None

    def cache_need(self):
        return self.mixer.cache_need()

    def state_need(self):
        return self._need

    def expected_tensors(self) -> Dict[str, ExpectedTensor]:
        out: Dict[str, ExpectedTensor] = {}
        for prefix, sub in self._subparts:
            for name, e in sub.expected_tensors().items():
                out[f"{prefix}.{name}"] = e
        if self.taps:
            out[self.conv_tensor] = ExpectedTensor((self.env.dim, self.taps))
        if self.side_dim:
            p = self.side_prefix
            out[f"{p}.table"] = ExpectedTensor((self.side_vocab, self.side_dim))
            out[f"{p}.gate.weight"] = ExpectedTensor((self.side_dim, self.env.dim))
            out[f"{p}.proj.weight"] = ExpectedTensor((self.env.dim, self.side_dim))
        return out

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for prefix, sub in self._subparts:
            sub.load({name: tensors[f"{prefix}.{name}"] for name in sub.expected_tensors()})
        if self.taps:
            self.conv_w = tensors[self.conv_tensor].to(device=self.env.device, dtype=torch.float32).contiguous()
        if self.side_dim:
            p = self.side_prefix
            self.side_table = as_compute(tensors[f"{p}.table"], self.env)
            self.side_gate_w = as_compute(tensors[f"{p}.gate.weight"], self.env)
            self.side_proj_w = as_compute(tensors[f"{p}.proj.weight"], self.env)

    def weight_bytes(self) -> int:
        extra = sum(t.numel() * t.element_size() for t in (self.side_gate_w, self.side_proj_w) if t is not None)
        return sum(sub.weight_bytes() for _p, sub in self._subparts) + extra

    def forward(self, residual: Residual, ctx, cache) -> None:
        ops = self.env.ops
        if residual.delta is not None:
            raise RuntimeError("a parallel block cannot follow a block that leaves its sum pending")
        if residual.normed is not None and residual.normed[0] is self.norm:
            h = residual.normed[1]                       # the block before took this norm along with its last kernel
        else:
            h = self.norm.forward(residual)
        residual.normed = None
        hm = h
        if self.taps:
            state = state_field(cache.state, self._need, "input_conv") if self.taps > 1 else None
            hm = ops.short_conv(h, self.conv_w, state, ctx.q_start, ctx.state_slot, ctx.fresh, n_seqs=ctx.n_seqs,
                                max_q_len=ctx.max_q_len, activation=None, residual=True, out_dtype=self.env.dtype)
        mixer_state = None if self.mixer.state_need() is None else state_field(cache.state, self._need, "mixer")
        y = self.mixer.forward(hm, ctx, dataclasses.replace(cache, state=mixer_state))
        f = None if self.feed_forward is None else self.feed_forward.forward(h, ctx)
        normed, coef, eps, plain = (), 1.0, 0.0, []
        for term in (y, f):
            if isinstance(term, NormedSum):
                normed, coef, eps = term.terms, term.coef, term.eps
            elif isinstance(term, PendingProduct):
                plain.append(term.take(ops, partials_ok=True))
            elif term is not None:
                plain.append(term)
        rows = ops.stream_add(residual.h, normed=normed, coef=coef, eps=eps, plain=tuple(plain), out_dtype=self.env.dtype)
        residual.rows = rows
        if not self.side_dim:
            return
        u = ops.linear(rows, self.side_gate_w, partials_ok=True)
        g = ops.side_gate(u, ctx.token_ids, self.side_table, out_dtype=self.env.dtype)
        follow = residual.next_norm
        if isinstance(follow, RMSNorm):
            residual.normed = (follow, self.side_norm.fold_normed(residual, PendingProduct(g, self.side_proj_w), then=follow))
        else:
            self.side_norm.fold_normed(residual, PendingProduct(g, self.side_proj_w), want_rows=False)
