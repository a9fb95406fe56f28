"""A model assembled from a spec: embedding, runs of blocks, final norm, head.

Reference: ``Transformer.__init__`` and ``forward``
(torchllms/models/networks.py:790-810, :1017-1047): embed, run every block,
keep the wanted rows, final norm, output projection (tied to the embedding
table when the configuration says so, :806-809).  The class knows nothing of
any architecture: the spec decides which parts exist, with which numbers, and
in which order they run.
"""

from __future__ import annotations

from typing import Dict, List, Mapping, Optional, Sequence, Tuple

import torch

from ..parts import attention, block, ffn, latent_attention, moe, norm, pair, recurrent, rope  # noqa: F401  (register the built-in parts)
from ..parts.base import BLOCKS, NORMS, BuildEnv, CacheNeed, Residual, StateNeed, as_compute
from ..parts.spec import ModelSpec
from ..weights.loader import ExpectedTensor


class Model:
    def __init__(self, spec: ModelSpec, *, dtype: torch.dtype, device, ops, max_positions: Optional[int] = None):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"the engine computes in float32 or bfloat16, not {dtype}")
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        self.ops = ops
        self.max_positions = int(max_positions or spec.max_positions)
        if spec.position_tensor is not None:
            # a learned position table ends where it ends: no request can grow past its last row
            self.max_positions = min(self.max_positions, spec.max_positions)
        self.env = BuildEnv(dim=spec.dim, dtype=dtype, device=self.device,
                            max_positions=self.max_positions, ops=ops)
        self.blocks = [BLOCKS.build(layer.block, self.env) for layer in spec.layers]
        self.final_norm = NORMS.build(spec.final_norm, self.env)
        self.embedding_norm = None if spec.embedding_norm is None else NORMS.build(spec.embedding_norm, self.env)
        self.graph_safe = self.final_norm.graph_safe and all(b.graph_safe for b in self.blocks)
        self.embedding: Optional[torch.Tensor] = None
        self.position_table: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None
        self.row_tensors: Dict[str, torch.Tensor] = {}
        self.keeps_embedding = any(run.add_embedding for run in spec.run_order)

    # ----------------------------------------------------------------- weights
    def expected_tensors(self) -> Dict[str, ExpectedTensor]:
        spec = self.spec
        out: Dict[str, ExpectedTensor] = {spec.embedding_tensor: ExpectedTensor((spec.vocab_size, spec.dim))}
        if spec.position_tensor is not None:
            out[spec.position_tensor] = ExpectedTensor((spec.max_positions, spec.dim))
        for layer, blk in zip(spec.layers, self.blocks):
            for name, e in blk.expected_tensors().items():
                out[f"{layer.name}.{name}"] = e
        for name, e in self.final_norm.expected_tensors().items():
            out[f"{spec.final_norm_prefix}.{name}"] = e
        if self.embedding_norm is not None:
            for name, e in self.embedding_norm.expected_tensors().items():
                out[f"{spec.embedding_norm_prefix}.{name}"] = e
        if not spec.tie_head:
            out[spec.head_tensor] = ExpectedTensor((spec.vocab_size, spec.dim))
        for name, rows in spec.row_tensors:
            out[name] = ExpectedTensor((rows, spec.dim))
        return out

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        """``tensors`` holds exactly :meth:`expected_tensors` (checked by the caller)."""
        spec = self.spec
        self.embedding = as_compute(tensors[spec.embedding_tensor], self.env)
        if spec.position_tensor is not None:
            self.position_table = as_compute(tensors[spec.position_tensor], self.env)
        for layer, blk in zip(spec.layers, self.blocks):
            blk.load({name: tensors[f"{layer.name}.{name}"] for name in blk.expected_tensors()})
        self.final_norm.load({name: tensors[f"{spec.final_norm_prefix}.{name}"]
                              for name in self.final_norm.expected_tensors()})
        if self.embedding_norm is not None:
            self.embedding_norm.load({name: tensors[f"{spec.embedding_norm_prefix}.{name}"]
                                      for name in self.embedding_norm.expected_tensors()})
        self.head = self.embedding if spec.tie_head else as_compute(tensors[spec.head_tensor], self.env)
        # rows that runs add to the stream: kept in 32-bit, as the stream is
        self.row_tensors = {name: tensors[name].to(device=self.device, dtype=torch.float32).contiguous()
                            for name, _rows in spec.row_tensors}

    def weight_bytes(self) -> int:
        """Bytes of weights a step has to read: every layer's matrices and the head once
        (of the embedding table a step reads only the rows of its tokens)."""
        return sum(blk.weight_bytes() for blk in self.blocks) + self.final_norm.weight_bytes() \
            + self.head.numel() * self.head.element_size()

    # ------------------------------------------------------------------- cache
    def run_needs(self) -> List[Tuple[Optional[CacheNeed], Optional[StateNeed], Optional[int]]]:
        """What each run of the run order wants from the cache manager."""
        return [(self.blocks[run.layer].cache_need(), self.blocks[run.layer].state_need(), run.cache_of)
                for run in self.spec.run_order]

    # ----------------------------------------------------------------- forward
    def _residual_with_history(self, ctx) -> Residual:
        """Level 0 holds the embedding output, one more level every layer run, and a last one for
        what leaves the last run.  The stream of the first run starts as a copy of level 0."""
        h0 = self.ops.embed(ctx.token_ids, self.embedding, scale=self.spec.embedding_scale,
                            positions=ctx.positions if self.position_table is not None else None,
                            position_table=self.position_table)
        history = torch.empty((len(self.spec.run_order) + 2, *h0.shape), dtype=torch.float32, device=h0.device)
        history[0].copy_(h0)
        history[1].copy_(h0)
        return Residual(history[1], history=history)

    def _next_level(self, residual: Residual) -> None:
        """A run is finished and left its result in the level being written; the next run's
        stream starts from it."""
        if residual.delta is not None:
            raise RuntimeError("a block of a model that keeps its history must not leave a sum pending")
        residual.level += 1
        nxt = residual.history[residual.level + 1]
        nxt.copy_(residual.h)
        residual.h, residual.rows = nxt, None

    def _add_before_run(self, residual: Residual, run, embedding_output: Optional[torch.Tensor]) -> None:
        """``h += embedding output + row`` (either may be absent), in 32-bit, before a run that asks for it."""
        if residual.delta is not None or residual.normed is not None or residual.history is not None:
            raise RuntimeError("a sum in front of a run needs a stream with nothing pending and no kept history")
        row = None
        if run.add_row is not None:
            row = self.row_tensors[run.add_row[0]][run.add_row[1]]
        self.ops.stream_inject(residual.h, embedding_output if run.add_embedding else None, row)
        residual.rows = None

    def forward(self, ctx, views: Sequence) -> Optional[torch.Tensor]:
        """Run the step's tokens; returns float32 logits ``[n_wanted, vocab]`` or ``None``."""
        first = self.blocks[self.spec.run_order[0].layer] if self.spec.run_order else None
        if self.spec.keeps_history:
            residual = self._residual_with_history(ctx)
        elif self.position_table is None and self.spec.embedding_scale == 1.0 and not getattr(first, "reads_stream", False):
            residual = Residual(self.ops.embed(ctx.token_ids, self.embedding))
        elif getattr(first, "reads_stream", False):
            # the first layer reads the stream itself: the embedding's kernel leaves it in the activation dtype too
            h, rows = self.ops.embed(ctx.token_ids, self.embedding, scale=self.spec.embedding_scale,
                                     positions=ctx.positions, position_table=self.position_table, rows_dtype=self.dtype)
            residual = Residual(h, rows=rows)
        else:
            residual = Residual(self.ops.embed(ctx.token_ids, self.embedding, scale=self.spec.embedding_scale,
                                               positions=ctx.positions, position_table=self.position_table))
        if self.embedding_norm is not None:
            # the stream is the norm of the table's rows, taken in 32-bit and kept so
            if residual.history is not None:
                raise RuntimeError("a normed embedding and a kept history are not built together")
            residual = Residual(self.ops.rmsnorm(residual.h, None, self.embedding_norm.weight, self.embedding_norm.eps,
                                                 out_dtype=torch.float32))
        order = self.spec.run_order
        embedding_output = residual.h.clone() if self.keeps_embedding else None
        for i, run in enumerate(order):
            if run.add_embedding or run.add_row is not None:
                self._add_before_run(residual, run, embedding_output)
            follows = order[i + 1] if i + 1 < len(order) else None
            # (a run that starts with a sum onto the stream takes its own input norm afterwards)
            residual.next_norm = (self.blocks[follows.layer].input_norm
                                  if follows is not None and not (follows.add_embedding or follows.add_row is not None) else None)
            self.blocks[run.layer].forward(residual, ctx, views[i])
            if residual.history is not None and residual.level != i + 1:
                self._next_level(residual)      # a block that reads no earlier results: the stream passes as it is
        if ctx.n_want == 0:
            return None
        x = self.final_norm.forward(residual, rows=ctx.want_rows)
        logits = self.ops.linear(x, self.head, out_dtype=torch.float32)
        return logits if self.spec.logit_scale == 1.0 else logits.mul_(self.spec.logit_scale)
