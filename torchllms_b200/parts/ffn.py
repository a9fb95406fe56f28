"""Dense gated feed-forward (SwiGLU).

Reference: ``FeedForward.forward`` (torchllms/models/networks.py:592-605):
``w2(silu(w1 x) * w3 x)`` with ``w1, w3: [hidden, dim]`` and ``w2: [dim, hidden]``,
no biases.  ``w1`` and ``w3`` are stacked so that one product yields gate and up.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..kernels.lazy import PendingProduct
from ..weights.loader import ExpectedTensor
from .base import BuildEnv, FeedForward, as_compute, register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    graph_safe = True
    takes_row_scaled = True      # x only goes into the gate/up product, whose activation applies the scale

    def __init__(self, env: BuildEnv, *, dim: int, hidden: int):
        self.env = env
        self.dim, self.hidden = int(dim), int(hidden)
        self.w13: Optional[torch.Tensor] = None
        self.w2: Optional[torch.Tensor] = None

    def expected_tensors(self) -> Dict[str, ExpectedTensor]:
        return {
            "w1.weight": ExpectedTensor((self.hidden, self.dim)),
            "w2.weight": ExpectedTensor((self.dim, self.hidden)),
            "w3.weight": ExpectedTensor((self.hidden, self.dim)),
        }

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.w13 = torch.cat([as_compute(tensors["w1.weight"], self.env), as_compute(tensors["w3.weight"], self.env)])
        self.w2 = as_compute(tensors["w2.weight"], self.env)

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        ops = self.env.ops
        # gate and up in one product over the stacked weight, the activation in its epilogue where the
        # kernel can (decode steps), else product [T, 2 * hidden] + SwiGLU kernel
        # the down projection is left to the norm that follows (see PendingProduct)
        return PendingProduct(ops.linear_swiglu(x, self.w13), self.w2)


@register_feed_forward("clamped_glu")
class ClampedGLU(FeedForward):
    """Dense gated feed-forward with bounded branches:
    ``g = min(gate x, limit)``, ``u = clamp(up x, -limit, limit)``,
    ``y = g * sigmoid(alpha * g) * (u + up_offset)``, output ``down y``.  Weights ``gate.weight`` and
    ``up.weight`` are ``[hidden, dim]``, ``down.weight`` is ``[dim, hidden]``; gate and up are
    stacked so that one product yields both."""

    graph_safe = True

    def __init__(self, env: BuildEnv, *, dim: int, hidden: int, limit: float, alpha: float = 1.702,
                 up_offset: float = 1.0):
        self.env = env
        self.dim, self.hidden = int(dim), int(hidden)
        self.limit, self.alpha, self.up_offset = float(limit), float(alpha), float(up_offset)
        if not self.limit > 0:
            raise ValueError(f"the bound of a clamped feed-forward must be positive, got {limit}")
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def expected_tensors(self) -> Dict[str, ExpectedTensor]:
        return {
            "gate.weight": ExpectedTensor((self.hidden, self.dim)),
            "up.weight": ExpectedTensor((self.hidden, self.dim)),
            "down.weight": ExpectedTensor((self.dim, self.hidden)),
        }

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.w_gate_up = torch.cat([as_compute(tensors["gate.weight"], self.env), as_compute(tensors["up.weight"], self.env)])
        self.w_down = as_compute(tensors["down.weight"], self.env)

    def forward(self, x: torch.Tensor, ctx) -> PendingProduct:
        y = self.env.ops.linear_glu(x, self.w_gate_up, limit=self.limit, alpha=self.alpha, up_offset=self.up_offset)
        return PendingProduct(y, self.w_down)       # the down projection is left to the norm that follows


GATE_ACTIVATIONS = ("silu", "gelu_tanh")


@register_feed_forward("glu")
class GatedLinearUnit(FeedForward):
    """Dense gated feed-forward with a choice of activation: ``down(act(gate x) * up x)``, ``act``
    being ``silu`` or ``gelu_tanh`` (``0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)))``).
    Weights ``gate.weight`` and ``up.weight`` are ``[hidden, dim]``, ``down.weight`` is ``[dim, hidden]``;
    gate and up are stacked so that one product yields both.  The activation is float32 arithmetic."""

    graph_safe = True

    def __init__(self, env: BuildEnv, *, dim: int, hidden: int, activation: str):
        if activation not in GATE_ACTIVATIONS:
            raise ValueError(f"unknown gate activation {activation!r}; known: {', '.join(GATE_ACTIVATIONS)}")
        self.env = env
        self.dim, self.hidden, self.activation = int(dim), int(hidden), activation
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def expected_tensors(self) -> Dict[str, ExpectedTensor]:
        return {
            "gate.weight": ExpectedTensor((self.hidden, self.dim)),
            "up.weight": ExpectedTensor((self.hidden, self.dim)),
            "down.weight": ExpectedTensor((self.dim, self.hidden)),
        }

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.w_gate_up = torch.cat([as_compute(tensors["gate.weight"], self.env), as_compute(tensors["up.weight"], self.env)])
        self.w_down = as_compute(tensors["down.weight"], self.env)

    def forward(self, x: torch.Tensor, ctx) -> PendingProduct:
        y = self.env.ops.linear_gated_act(x, self.w_gate_up, activation=self.activation)
        return PendingProduct(y, self.w_down)       # the down projection is left to the norm that follows


@register_feed_forward("polynorm")
class PolyNormFeedForward(FeedForward):
    """Dense feed-forward without a gate whose activation is a polynomial of normalised powers:
    ``down(a N(z) + b N(z^2) + c N(z^3) + e)`` with ``z = up x``, powers taken element by element and
    ``N(y) = y / sqrt(mean(y^2) + eps)`` over a token's ``hidden`` values.  The four numbers are the
    stored tensor ``act``; the three norms are float32 and one kernel."""

    graph_safe = True

    def __init__(self, env: BuildEnv, *, dim: int, hidden: int, eps: float):
        self.env = env
        self.dim, self.hidden, self.eps = int(dim), int(hidden), float(eps)
        self.w_up = self.w_down = self.coef = None

    def expected_tensors(self) -> Dict[str, ExpectedTensor]:
        return {"up.weight": ExpectedTensor((self.hidden, self.dim)), "down.weight": ExpectedTensor((self.dim, self.hidden)),
                "act": ExpectedTensor((4,))}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.w_up = as_compute(tensors["up.weight"], self.env)
        self.w_down = as_compute(tensors["down.weight"], self.env)
        self.coef = tensors["act"].to(device=self.env.device, dtype=torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_up, self.w_down))

    def forward(self, x: torch.Tensor, ctx) -> PendingProduct:
        ops = self.env.ops
        y = ops.polynorm(ops.linear(x, self.w_up, partials_ok=True), self.coef, self.eps, out_dtype=self.env.dtype)
        return PendingProduct(y, self.w_down)
