"""Two mixers side by side: both read the same rows, and the result is a weighted sum of their
outputs, each RMS-normed over the stream's width first.

One of the two may keep keys and values in the paged cache and either may keep state rows; the
pair asks the cache manager for both in its members' names and hands each member what is its own.
"""

from __future__ import annotations

import dataclasses
from typing import Dict, Mapping

import torch

from ..kernels.lazy import NormedSum, PendingProduct
from ..weights.loader import ExpectedTensor
from .base import MIXERS, BuildEnv, Mixer, join_states, register_mixer, state_field
from .spec import PartSpec


@register_mixer("side_by_side")
class SideBySide(Mixer):
    """``coef * (norm_l(left(x)) + norm_r(right(x)))`` with plain-weight RMS norms over the width.

    Tensors: the members' under ``<left_prefix>.`` and ``<right_prefix>.``, the norms' weights
    ``<left_prefix>.<out_norm>`` and ``<right_prefix>.<out_norm>``.  The sum is left untaken
    (:class:`~torchllms_b200.kernels.lazy.NormedSum`): the kernel that adds the layer's result to
    the stream takes both norms in 32-bit on the way."""

    def __init__(self, env: BuildEnv, *, dim: int, left: PartSpec, right: PartSpec, eps: float, coef: float = 0.5,
                 left_prefix: str = "left", right_prefix: str = "right", out_norm: str = "out"):
        self.env = env
        self.dim, self.eps, self.coef = int(dim), float(eps), float(coef)
        self.members = ((left_prefix, MIXERS.build(left, env)), (right_prefix, MIXERS.build(right, env)))
        self.out_norm = out_norm
        if sum(m.cache_need() is not None for _p, m in self.members) > 1:
            raise ValueError("of two mixers side by side at most one may keep keys and values in the paged cache")
        self.graph_safe = all(m.graph_safe for _p, m in self.members)
        self._need = join_states([(p, m.state_need()) for p, m in self.members])
        self.out_w: Dict[str, torch.Tensor] = {}

    def cache_need(self):
        for _p, m in self.members:
            if m.cache_need() is not None:
                return m.cache_need()
        return None

    def state_need(self):
        return self._need

    def expected_tensors(self) -> Dict[str, ExpectedTensor]:
        out: Dict[str, ExpectedTensor] = {}
        for prefix, m in self.members:
            for name, e in m.expected_tensors().items():
                out[f"{prefix}.{name}"] = e
            out[f"{prefix}.{self.out_norm}"] = ExpectedTensor((self.dim,))
        return out

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for prefix, m in self.members:
            m.load({name: tensors[f"{prefix}.{name}"] for name in m.expected_tensors()})
            self.out_w[prefix] = tensors[f"{prefix}.{self.out_norm}"].to(device=self.env.device, dtype=torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return sum(m.weight_bytes() for _p, m in self.members)

    def forward(self, x: torch.Tensor, ctx, cache) -> NormedSum:
        terms = []
        for prefix, m in self.members:
            state = None if m.state_need() is None else state_field(cache.state, self._need, prefix)
            y = m.forward(x, ctx, dataclasses.replace(cache, state=state))
            if isinstance(y, PendingProduct):
                y = y.take(self.env.ops, partials_ok=True)
            terms.append((y, self.out_w[prefix]))
        return NormedSum(tuple(terms), self.coef, self.eps)
