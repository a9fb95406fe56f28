"""Feed-forward layers made of many small experts, of which every token uses a few.

Routing runs on the device: a kernel takes the router's scores and picks the experts, another
sorts the (token, expert) pairs by expert, the experts' products run as one grouped product over
the sorted rows, and a last kernel adds up every token's weighted results.  A step of few tokens
that touch most experts between them (a decode batch) instead takes all experts as one matrix
each way, with zeros where a token did not choose an expert: the weights stream once at the
speed of the other decode products.  Nothing is read back, so the shapes of a step's launches
depend on its token count alone.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..kernels.lazy import PendingProduct
from ..weights.loader import ExpectedTensor
from .base import BuildEnv, FeedForward, as_compute, register_feed_forward

EXPERT_ACTIVATIONS = ("relu2", "silu", "gelu_tanh", "clamped_swish")


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    """``n_experts`` feed-forwards ``down_e(act(up_e x))`` without biases (with ``gated``:
    ``down_e(act(gate_e x) * up_e x)``); a token uses ``top`` of them.

    * router logits ``z = W_router x`` (plus the stored vector ``router.bias`` with ``router_bias``) and scores ``s = softmax(z)`` over all experts, in float32;
    * the experts with the largest ``s + correction`` are chosen (``choice_correction``: a stored
      vector ``correction`` that steers the choice and nothing else);
    * their weights are ``s * router_scale``, divided by their sum first with ``renormalize``;
    * with ``shared_hidden`` a shared expert of the same form runs for every token and is added,
      multiplied by ``sigmoid(W_sg x)`` (one number per token) with ``shared_gate``.

    Options of the router: ``score="sigmoid"`` takes ``s = sigmoid(z)`` instead of the softmax; with
    ``n_groups > 1`` the experts form so many equal groups of neighbours, a group's score is the sum of
    its ``group_score_top`` largest ``s + correction``, and only experts of the ``keep_groups`` best groups
    can be chosen; ``renorm_eps`` is added to the sum that ``renormalize`` divides by.

    ``activation="clamped_swish"`` (gated experts only): with ``g = min(gate_e x, act_limit)`` and
    ``u = clamp(up_e x, -act_limit, act_limit)`` the hidden row is ``g * sigmoid(act_alpha g) * (u + act_up_offset)``.
    A shared expert beside gated experts is gated too (``shared.w_gate.weight``) and has a bound of its
    own, ``shared_act_limit``.

    Tensors: ``router.weight [E, dim]``, ``correction [E]``, ``experts.<e>.up.weight [hidden, dim]``,
    ``experts.<e>.down.weight [dim, hidden]``, ``shared.up.weight``, ``shared.down.weight``,
    ``shared.gate.weight [1, dim]``."""

    graph_safe = True

    def __init__(self, env: BuildEnv, *, dim: int, n_experts: int, top: int, hidden: int, activation: str = "relu2",
                 router_scale: float = 1.0, choice_correction: bool = False, renormalize: bool = False,
                 shared_hidden: Optional[int] = None, shared_gate: bool = False, gated: bool = False,
                 router_bias: bool = False, score: str = "softmax", n_groups: int = 1, keep_groups: int = 1,
                 group_score_top: int = 2, renorm_eps: float = 0.0, act_limit: Optional[float] = None,
                 act_alpha: float = 1.702, act_up_offset: float = 1.0, shared_act_limit: Optional[float] = None):
        if activation not in EXPERT_ACTIVATIONS:
            raise ValueError(f"unknown expert activation {activation!r}; known: {', '.join(EXPERT_ACTIVATIONS)}")
        if not 0 < top <= n_experts:
            raise ValueError(f"a token uses between 1 and {n_experts} experts, got {top}")
        if shared_gate and not shared_hidden:
            raise ValueError("a gate of the shared expert needs a shared expert")
        self.env = env
        self.dim, self.n_experts, self.top, self.hidden = int(dim), int(n_experts), int(top), int(hidden)
        self.activation = activation
        self.router_scale = float(router_scale)
        self.choice_correction, self.renormalize = bool(choice_correction), bool(renormalize)
        self.shared_hidden = None if not shared_hidden else int(shared_hidden)
        self.shared_gate = bool(shared_gate)
        self.gated, self.router_bias = bool(gated), bool(router_bias)
        if score not in ("softmax", "sigmoid"):
            raise ValueError(f"a router's scores are 'softmax' or 'sigmoid', got {score!r}")
        self.score, self.n_groups, self.keep_groups = score, int(n_groups), int(keep_groups)
        self.group_score_top, self.renorm_eps = int(group_score_top), float(renorm_eps)
        if self.n_groups < 1 or self.n_experts % self.n_groups or not 0 < self.keep_groups <= self.n_groups \
                or self.keep_groups * (self.n_experts // self.n_groups) < self.top or self.group_score_top < 1:
            raise ValueError(f"{n_experts} experts cannot form {n_groups} equal groups of which {keep_groups} hold the {top} chosen")
        self.clamped = activation == "clamped_swish"
        if self.clamped and not (self.gated and act_limit is not None and act_limit > 0):
            raise ValueError("the clamped activation goes with gated experts and a positive act_limit")
        if self.gated and self.shared_hidden and not self.clamped:
            raise ValueError("a shared expert beside gated experts is built for the clamped activation only")
        if self.gated and self.shared_gate:
            raise ValueError("a sigmoid gate on the shared expert goes with experts that have no gate matrix")
        self.act_params = (float(act_limit), float(act_alpha), float(act_up_offset)) if self.clamped else None
        self.shared_act_params = None
        if self.clamped and self.shared_hidden:
            if shared_act_limit is None or not shared_act_limit > 0:
                raise ValueError("a shared expert with the clamped activation needs a positive shared_act_limit")
            self.shared_act_params = (float(shared_act_limit), float(act_alpha), float(act_up_offset))
        self.up_rows = self.hidden * (2 if self.gated else 1)      # rows of one expert's stacked [gate; up]
        self.logit_bias: Optional[torch.Tensor] = None
        self.w_router: Optional[torch.Tensor] = None       # float32 [E (+ 1), dim]: the gate's row rides along
        self.correction: Optional[torch.Tensor] = None
        # every expert's up matrix stacked, the shared expert's last: [E * hidden + shared, dim]; the down matrices
        # side by side in the same order: [dim, E * hidden + shared].  The grouped products read an expert's own
        # block of either; a step that touches most experts anyway takes each as one matrix.
        self.w_up_all: Optional[torch.Tensor] = None
        self.w_down_all: Optional[torch.Tensor] = None
        self.w_up: Optional[torch.Tensor] = None           # [E, hidden, dim], a view of w_up_all
        self.w_shared_up: Optional[torch.Tensor] = None    # a view of w_up_all
        self.w_shared_down: Optional[torch.Tensor] = None  # a copy of its own (the products want whole rows)

    def expected_tensors(self) -> Dict[str, ExpectedTensor]:
        out = {"router.weight": ExpectedTensor((self.n_experts, self.dim))}
        if self.choice_correction:
            out["correction"] = ExpectedTensor((self.n_experts,))
        if self.router_bias:
            out["router.bias"] = ExpectedTensor((self.n_experts,))
        for e in range(self.n_experts):
            if self.gated:
                out[f"experts.{e}.gate.weight"] = ExpectedTensor((self.hidden, self.dim))
            out[f"experts.{e}.up.weight"] = ExpectedTensor((self.hidden, self.dim))
            out[f"experts.{e}.down.weight"] = ExpectedTensor((self.dim, self.hidden))
        if self.shared_hidden:
            if self.gated:
                out["shared.w_gate.weight"] = ExpectedTensor((self.shared_hidden, self.dim))
            out["shared.up.weight"] = ExpectedTensor((self.shared_hidden, self.dim))
            out["shared.down.weight"] = ExpectedTensor((self.dim, self.shared_hidden))
            if self.shared_gate:
                out["shared.gate.weight"] = ExpectedTensor((1, self.dim))
        return out

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        f32 = dict(device=self.env.device, dtype=torch.float32)
        rows = [tensors["router.weight"].to(**f32)]
        if self.shared_gate:
            rows.append(tensors["shared.gate.weight"].to(**f32))
        self.w_router = torch.cat(rows).contiguous()
        if self.choice_correction:
            self.correction = tensors["correction"].to(**f32).contiguous()
        if self.router_bias:
            self.logit_bias = tensors["router.bias"].to(**f32).contiguous()
        ups = [as_compute(tensors[f"experts.{e}.up.weight"], self.env) for e in range(self.n_experts)]
        if self.gated:        # an expert's rows are [gate; up], so that one product yields both
            ups = [torch.cat([as_compute(tensors[f"experts.{e}.gate.weight"], self.env), up]) for e, up in enumerate(ups)]
        downs = [as_compute(tensors[f"experts.{e}.down.weight"], self.env) for e in range(self.n_experts)]
        if self.shared_hidden:
            if self.gated:       # the shared expert's rows are [gate; up] as an expert's are
                ups.append(as_compute(tensors["shared.w_gate.weight"], self.env))
            ups.append(as_compute(tensors["shared.up.weight"], self.env))
            downs.append(as_compute(tensors["shared.down.weight"], self.env))
            self.w_shared_down = downs[-1]
        self.w_up_all = torch.cat(ups).contiguous()
        self.w_down_all = torch.cat(downs, dim=1).contiguous()
        n = self.n_experts * self.up_rows
        self.w_up = self.w_up_all[:n].view(self.n_experts, self.up_rows, self.dim)
        if self.shared_hidden:
            self.w_shared_up = self.w_up_all[n:]

    def weight_bytes(self) -> int:
        """What a step reads at most: the router and every expert (a step of few tokens leaves most
        experts alone; this counts all of them)."""
        return sum(t.numel() * t.element_size() for t in (self.w_router, self.w_up_all, self.w_down_all))

    def forward(self, x: torch.Tensor, ctx):
        ops = self.env.ops
        chosen, weights, gate = ops.moe_route(x, self.w_router, self.correction, n_experts=self.n_experts, top=self.top,
                                              scale=self.router_scale, renormalize=self.renormalize,
                                              shared_gate=self.shared_gate, logit_bias=self.logit_bias, score=self.score,
                                              n_groups=self.n_groups, keep_groups=self.keep_groups,
                                              group_score_top=self.group_score_top, renorm_eps=self.renorm_eps)
        if ops.moe_prefers_dense(x.shape[0], self.top, self.n_experts, x.dtype):
            # few tokens that touch most experts between them: every expert (and the shared one) as one
            # matrix each way, the rows of experts a token did not choose multiplied by zero
            u = ops.moe_dense_hidden(x, chosen, weights, gate, self.w_up_all, n_experts=self.n_experts, hidden=self.hidden, gated=self.gated,
                                     activation=self.activation, act_params=self.act_params, extra_act_params=self.shared_act_params)
            return PendingProduct(u, self.w_down_all)
        shared = None
        if self.shared_hidden and self.clamped:
            limit, alpha, offset = self.shared_act_params
            u = ops.linear_glu(x, self.w_shared_up, limit=limit, alpha=alpha, up_offset=offset)
            shared = ops.linear(u, self.w_shared_down, partials_ok=True)
        elif self.shared_hidden:
            u = ops.activation(ops.linear(x, self.w_shared_up, partials_ok=True), self.activation, out_dtype=self.env.dtype)
            shared = ops.linear(u, self.w_shared_down, partials_ok=True)
        return ops.moe_experts(x, chosen, weights, self.w_up, self.w_down_all, activation=self.activation,
                               shared=shared, shared_gate=gate, gated=self.gated, act_params=self.act_params)
