"""Recurrent mixers: a state of fixed size per request instead of a cache that grows.

The state lives in the cache manager's state rows (one row per live request, zeroed when the
request is admitted), in 32-bit floats whatever the activation dtype; a prompt portion runs the
recurrence over its tokens inside one kernel and leaves the state for the next step.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..kernels.lazy import PendingProduct
from ..weights.loader import ExpectedTensor
from .base import BuildEnv, Mixer, StateNeed, as_compute, join_states, register_mixer, state_field
from .rope import precise_rotary_table


@register_mixer("mingru")
class MinGRU(Mixer):
    """A gated recurrence whose gates read only the current token:

        ``z_t = sigmoid(Wz x_t + bz)``,  ``u_t = Wx x_t + bx``,
        ``c_t = u_t + 1/2`` where ``u_t >= 0``, ``sigmoid(u_t)`` elsewhere,
        ``S_t = (1 - z_t) S_(t-1) + z_t c_t``   (element by element, ``S`` of size ``width``),
        output ``Wo (S_t * silu(Wg x_t))``.

    The three projections of the input are one stacked product; the gates, the candidate, the
    recurrence and the output gate are one kernel in float32; ``Wo`` is left to whoever adds the
    result to the stream."""

    graph_safe = True

    def __init__(self, env: BuildEnv, *, dim: int, width: int):
        self.env = env
        self.dim, self.width = int(dim), int(width)
        if self.width <= 0:
            raise ValueError(f"the width of a recurrent state must be positive, got {width}")
        self.w_in: Optional[torch.Tensor] = None
        self.b_in: Optional[torch.Tensor] = None
        self.wo: Optional[torch.Tensor] = None

    def state_need(self) -> StateNeed:
        return StateNeed((self.width,), torch.float32)

    def expected_tensors(self) -> Dict[str, ExpectedTensor]:
        w, d = self.width, self.dim
        return {
            "wz.weight": ExpectedTensor((w, d)), "wz.bias": ExpectedTensor((w,)),
            "wx.weight": ExpectedTensor((w, d)), "wx.bias": ExpectedTensor((w,)),
            "wg.weight": ExpectedTensor((w, d)), "wo.weight": ExpectedTensor((d, w)),
        }

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        f32 = dict(device=self.env.device, dtype=torch.float32)
        self.w_in = torch.cat([as_compute(tensors[n], self.env) for n in ("wz.weight", "wx.weight", "wg.weight")])   # rows [wz; wx; wg]
        self.b_in = torch.cat([tensors["wz.bias"].to(**f32), tensors["wx.bias"].to(**f32),
                               torch.zeros(self.width, **f32)]).contiguous()
        self.wo = as_compute(tensors["wo.weight"], self.env)

    def forward(self, x: torch.Tensor, ctx, cache) -> PendingProduct:
        ops = self.env.ops
        proj = ops.linear(x, self.w_in, partials_ok=True)
        y = ops.mingru_scan(proj, self.b_in, cache.state, ctx.q_start, ctx.state_slot, ctx.fresh,
                            n_seqs=ctx.n_seqs, max_q_len=ctx.max_q_len, out_dtype=self.env.dtype)
        return PendingProduct(y, self.wo)


def _matrix_state_scan(ops, q, k, v, state, ctx, **how):
    return ops.linear_recurrence(q, k, v, state, ctx.q_start, ctx.state_slot, ctx.fresh, n_seqs=ctx.n_seqs,
                                 max_q_len=ctx.max_q_len, **how)


@register_mixer("retention")
class Retention(Mixer):
    """Linear attention with one fixed decay per head and neither softmax nor denominator:

        ``S_t = decay_h S_(t-1) + k_t v_t^T``,  ``o_t = S_t^T q_t``   (``S`` is ``head_dim x v_head_dim`` per head),

    q and k rotated by the position's angles on their first ``rot_dims`` coordinates (``rot_pairing``
    ``"half"``: coordinate ``i`` with ``i + rot_dims / 2``), k then multiplied by ``k_scale``.  Each
    head's ``o`` is divided by its root mean square (no weight), multiplied by ``silu(wg x)`` and
    projected by ``wo``.  Rotation, recurrence, state and the head norm are float32; one stacked
    product gives ``[q | k | v | g]``.  The state rows hold ``S^T`` (``[heads, v_head_dim, head_dim]``:
    a column's keys side by side, as the kernel's lanes read them)."""

    graph_safe = True

    def __init__(self, env: BuildEnv, *, dim: int, n_heads: int, head_dim: int, v_head_dim: int, decay, k_scale: float,
                 rot_dims: int, rot_base: float, norm_eps: float, rot_pairing: str = "half"):
        decay = tuple(float(x) for x in decay)
        if len(decay) != n_heads:
            raise ValueError(f"one decay per head: {n_heads} heads, {len(decay)} decays")
        if rot_dims < 0 or rot_dims % 2 or rot_dims > head_dim:
            raise ValueError(f"rot_dims must be even and at most head_dim ({head_dim}), got {rot_dims}")
        if rot_pairing != "half":
            raise ValueError(f"retention rotates in the 'half' pairing, got {rot_pairing!r}")
        self.env = env
        self.dim, self.n_heads, self.head_dim, self.v_head_dim = int(dim), int(n_heads), int(head_dim), int(v_head_dim)
        self.k_scale, self.rot_dims, self.norm_eps = float(k_scale), int(rot_dims), float(norm_eps)
        self.n_qk, self.n_v = self.n_heads * self.head_dim, self.n_heads * self.v_head_dim
        self.table = precise_rotary_table(max(self.rot_dims, 2), rot_base, 1.0, env.max_positions, env.device)
        self.decay = torch.tensor(decay, dtype=torch.float32, device=env.device)
        self.w_in: Optional[torch.Tensor] = None
        self.wo: Optional[torch.Tensor] = None

    def state_need(self) -> StateNeed:
        return StateNeed((self.n_heads, self.v_head_dim, self.head_dim), torch.float32)      # S^T: a column's keys side by side

    def expected_tensors(self) -> Dict[str, ExpectedTensor]:
        d = self.dim
        return {"wq.weight": ExpectedTensor((self.n_qk, d)), "wk.weight": ExpectedTensor((self.n_qk, d)),
                "wv.weight": ExpectedTensor((self.n_v, d)), "wg.weight": ExpectedTensor((self.n_v, d)),
                "wo.weight": ExpectedTensor((d, self.n_v))}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.w_in = torch.cat([as_compute(tensors[n], self.env) for n in ("wq.weight", "wk.weight", "wv.weight", "wg.weight")])
        self.wo = as_compute(tensors["wo.weight"], self.env)

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.wo))

    def forward(self, x: torch.Tensor, ctx, cache) -> PendingProduct:
        ops = self.env.ops
        proj = ops.linear(x, self.w_in)
        n, nv = self.n_qk, self.n_v
        turn = dict(n_heads=self.n_heads, head_dim=self.head_dim, positions=ctx.positions, table=self.table, rot_dims=self.rot_dims)
        q = ops.recurrence_prep(proj[:, :n], scale=1.0, **turn)
        k = ops.recurrence_prep(proj[:, n:2 * n], scale=self.k_scale, **turn)
        o = _matrix_state_scan(ops, q, k, proj[:, 2 * n:2 * n + nv], cache.state, ctx, decay=self.decay)
        y = ops.head_norm_gate(o, proj[:, 2 * n + nv:], None, self.norm_eps, head_dim=self.v_head_dim, out_dtype=self.env.dtype)
        return PendingProduct(y, self.wo)


@register_mixer("gated_delta")
class GatedDelta(Mixer):
    """The gated delta rule: per head a matrix state that forgets, then corrects what it holds
    under the current key towards the current value:

        ``S <- g_t S``;  ``u = beta_t (v_t - S^T k_t)``;  ``S <- S + k_t u^T``;  ``o_t = S^T q_t``

    with ``beta = sigmoid(wb x)`` and ``g = exp(-exp(A_log) softplus(wa x + dt_bias))`` per head.  q
    and k (``n_qk_heads`` heads, shared by ``n_heads / n_qk_heads`` value heads each) and v pass a
    short causal convolution over time (``conv_taps`` taps per channel, the last one the current
    token's) and ``silu``; q and k become unit vectors (``x / sqrt(sum(x^2) + unit_eps)``) and q is
    multiplied by ``q_scale``.  Each head's ``o`` is RMS-normed over its values with the weight
    ``norm.weight`` (shared by heads), multiplied by ``silu(wg x)`` and projected by ``wo``.

    State per request: the convolutions' last ``conv_taps - 1`` inputs and the heads' matrices (kept
    as ``S^T``, ``[heads, v_head_dim, head_dim]``), all float32.  One stacked product gives ``[q | k | v | b | a | g]``."""

    graph_safe = True

    def __init__(self, env: BuildEnv, *, dim: int, n_heads: int, n_qk_heads: int, head_dim: int, v_head_dim: int,
                 conv_taps: int, q_scale: float, norm_eps: float, unit_eps: float = 1e-6):
        if n_heads % n_qk_heads != 0:
            raise ValueError(f"n_heads ({n_heads}) must be a multiple of n_qk_heads ({n_qk_heads})")
        if conv_taps < 1:
            raise ValueError(f"a convolution has at least one tap, got {conv_taps}")
        self.env = env
        self.dim, self.n_heads, self.n_qk_heads = int(dim), int(n_heads), int(n_qk_heads)
        self.head_dim, self.v_head_dim, self.taps = int(head_dim), int(v_head_dim), int(conv_taps)
        self.q_scale, self.norm_eps, self.unit_eps = float(q_scale), float(norm_eps), float(unit_eps)
        self.n_qk, self.n_v = self.n_qk_heads * self.head_dim, self.n_heads * self.v_head_dim
        self.n_conv = 2 * self.n_qk + self.n_v
        self._need = join_states([("conv", StateNeed((self.taps - 1, self.n_conv)) if self.taps > 1 else None),
                                  ("matrix", StateNeed((self.n_heads, self.v_head_dim, self.head_dim)))])      # S^T per head
        self.w_in = self.w_conv = self.decay_rate = self.decay_bias = self.norm_w = self.wo = None

    def state_need(self) -> StateNeed:
        return self._need

    def expected_tensors(self) -> Dict[str, ExpectedTensor]:
        d, H = self.dim, self.n_heads
        return {"wq.weight": ExpectedTensor((self.n_qk, d)), "wk.weight": ExpectedTensor((self.n_qk, d)),
                "wv.weight": ExpectedTensor((self.n_v, d)), "wq.conv": ExpectedTensor((self.n_qk, self.taps)),
                "wk.conv": ExpectedTensor((self.n_qk, self.taps)), "wv.conv": ExpectedTensor((self.n_v, self.taps)),
                "wb.weight": ExpectedTensor((H, d)), "wa.weight": ExpectedTensor((H, d)), "A_log": ExpectedTensor((H,)),
                "dt_bias": ExpectedTensor((H,)), "norm.weight": ExpectedTensor((self.v_head_dim,)),
                "wg.weight": ExpectedTensor((self.n_v, d)), "wo.weight": ExpectedTensor((d, self.n_v))}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        f32 = dict(device=self.env.device, dtype=torch.float32)
        names = ("wq.weight", "wk.weight", "wv.weight", "wb.weight", "wa.weight", "wg.weight")
        self.w_in = torch.cat([as_compute(tensors[n], self.env) for n in names])
        self.w_conv = torch.cat([tensors[n].to(**f32) for n in ("wq.conv", "wk.conv", "wv.conv")]).contiguous()
        self.decay_rate = torch.exp(tensors["A_log"].to(**f32)).contiguous()       # exp(A_log), taken once
        self.decay_bias = tensors["dt_bias"].to(**f32).contiguous()
        self.norm_w = tensors["norm.weight"].to(**f32).contiguous()
        self.wo = as_compute(tensors["wo.weight"], self.env)

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.wo))

    def forward(self, x: torch.Tensor, ctx, cache) -> PendingProduct:
        ops = self.env.ops
        H, n, nv, nc = self.n_heads, self.n_qk, self.n_v, self.n_conv
        proj = ops.linear(x, self.w_in)
        if self.taps > 1:
            c = ops.short_conv(proj[:, :nc], self.w_conv, state_field(cache.state, self._need, "conv"), ctx.q_start,
                               ctx.state_slot, ctx.fresh, n_seqs=ctx.n_seqs, max_q_len=ctx.max_q_len, activation="silu",
                               residual=False, out_dtype=self.env.dtype)
        else:
            c = ops.short_conv(proj[:, :nc], self.w_conv, None, ctx.q_start, ctx.state_slot, ctx.fresh, n_seqs=ctx.n_seqs,
                               max_q_len=ctx.max_q_len, activation="silu", residual=False, out_dtype=self.env.dtype)
        unit = dict(n_heads=self.n_qk_heads, head_dim=self.head_dim, unit_eps=self.unit_eps)
        q = ops.recurrence_prep(c[:, :n], scale=self.q_scale, **unit)
        k = ops.recurrence_prep(c[:, n:2 * n], scale=1.0, **unit)
        o = _matrix_state_scan(ops, q, k, c[:, 2 * n:], state_field(cache.state, self._need, "matrix"), ctx,
                               beta_logits=proj[:, nc:nc + H], decay_logits=proj[:, nc + H:nc + 2 * H],
                               decay_rate=self.decay_rate, decay_bias=self.decay_bias)
        y = ops.head_norm_gate(o, proj[:, nc + 2 * H:], self.norm_w, self.norm_eps, head_dim=self.v_head_dim, out_dtype=self.env.dtype)
        return PendingProduct(y, self.wo)


@register_mixer("selective_scan")
class SelectiveScan(Mixer):
    """A selective state-space mixer: every channel keeps ``state`` numbers that decay and are fed
    at rates the token itself chooses.

        ``[x | z] = W_in h``;  ``x <- silu(conv(x) + conv_bias)`` (causal, ``conv_taps`` taps per channel);
        ``[r | B | C] = W_x x`` (``dt_rank``, ``state``, ``state`` numbers);  ``dt = softplus(W_dt r + dt_bias)``;
        ``S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n``,  ``A = -exp(A_log)``;
        ``y_c = sum_n S[c, n] C_n + D_c x_c``;  output ``W_o (y * silu(z))``.

    State per request: the convolution's last ``conv_taps - 1`` inputs and ``S`` (``[inner, state]``),
    float32.  The step sizes with their softplus, the decays with their exponentials, ``S`` and
    everything multiplied into it are float32 inside one kernel that walks a request's tokens in
    order, so a result does not depend on how a prompt was cut.  ``W_dt`` is stored padded with zero
    columns to the width of ``W_x``'s rows, so that it multiplies those rows as they lie."""

    graph_safe = True

    def __init__(self, env: BuildEnv, *, dim: int, inner: int, state: int, dt_rank: int, conv_taps: int):
        if min(inner, state, dt_rank, conv_taps) < 1:
            raise ValueError("the sizes of a selective scan must be positive")
        self.env = env
        self.dim, self.inner, self.state, self.dt_rank, self.taps = int(dim), int(inner), int(state), int(dt_rank), int(conv_taps)
        self.n_x = self.dt_rank + 2 * self.state
        self._need = join_states([("conv", StateNeed((self.taps - 1, self.inner)) if self.taps > 1 else None),
                                  ("scan", StateNeed((self.inner, self.state)))])
        self.w_in = self.w_conv = self.b_conv = self.w_x = self.w_dt = self.b_dt = self.A = self.D = self.wo = None

    def state_need(self) -> StateNeed:
        return self._need

    def expected_tensors(self) -> Dict[str, ExpectedTensor]:
        d, c = self.dim, self.inner
        return {"w_in.weight": ExpectedTensor((2 * c, d)), "conv.weight": ExpectedTensor((c, self.taps)),
                "conv.bias": ExpectedTensor((c,)), "w_x.weight": ExpectedTensor((self.n_x, c)),
                "w_dt.weight": ExpectedTensor((c, self.dt_rank)), "w_dt.bias": ExpectedTensor((c,)),
                "A_log": ExpectedTensor((c, self.state)), "D": ExpectedTensor((c,)), "wo.weight": ExpectedTensor((d, c))}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        f32 = dict(device=self.env.device, dtype=torch.float32)
        self.w_in = as_compute(tensors["w_in.weight"], self.env)
        self.w_conv = tensors["conv.weight"].to(**f32).contiguous()
        self.b_conv = tensors["conv.bias"].to(**f32).contiguous()
        self.w_x = as_compute(tensors["w_x.weight"], self.env)
        w_dt = torch.zeros((self.inner, self.n_x), dtype=tensors["w_dt.weight"].dtype)
        w_dt[:, :self.dt_rank] = tensors["w_dt.weight"]
        self.w_dt = as_compute(w_dt, self.env)
        self.b_dt = tensors["w_dt.bias"].to(**f32).contiguous()
        self.A = (-torch.exp(tensors["A_log"].to(**f32))).contiguous()           # taken once
        self.D = tensors["D"].to(**f32).contiguous()
        self.wo = as_compute(tensors["wo.weight"], self.env)

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_x, self.w_dt, self.A, self.wo))

    def forward(self, x: torch.Tensor, ctx, cache) -> PendingProduct:
        ops = self.env.ops
        c = self.inner
        xz = ops.linear(x, self.w_in)
        conv_state = state_field(cache.state, self._need, "conv") if self.taps > 1 else None
        u = ops.short_conv(xz[:, :c], self.w_conv, conv_state, ctx.q_start, ctx.state_slot, ctx.fresh, n_seqs=ctx.n_seqs,
                           max_q_len=ctx.max_q_len, activation="silu", residual=False, out_dtype=self.env.dtype, bias=self.b_conv)
        p = ops.linear(u, self.w_x)                       # [T, dt_rank + 2 state]
        dt = ops.linear(p, self.w_dt)                     # [T, inner]: the zero columns skip B and C
        y = ops.selective_scan(u, dt, p[:, self.dt_rank:self.dt_rank + self.state], p[:, self.dt_rank + self.state:], xz[:, c:],
                               self.A, self.D, self.b_dt, state_field(cache.state, self._need, "scan"), ctx.q_start,
                               ctx.state_slot, ctx.fresh, n_seqs=ctx.n_seqs, max_q_len=ctx.max_q_len, out_dtype=self.env.dtype)
        return PendingProduct(y, self.wo)
