"""Plain PyTorch twins of the CUDA kernels, one function per kernel, same signatures.

They serve two purposes in the tests: each kernel is compared with its twin on
the GPU, and the engine's host-side logic (cache, step function, scheduler,
replay) is exercised on the CPU by building an engine over a :class:`TorchOps`.
Nothing in the package imports this file.
"""

from __future__ import annotations

import math
from typing import Optional

import numpy as np
import torch

from torchllms_b200.kernels.lazy import PendingProduct, RowScaled      # two value types, no kernels

MASK64 = (1 << 64) - 1


def mix64(z: int) -> int:
    z &= MASK64
    z ^= z >> 30
    z = (z * 0xBF58476D1CE4E5B9) & MASK64
    z ^= z >> 27
    z = (z * 0x94D049BB133111EB) & MASK64
    z ^= z >> 31
    return z


def _mix64_np(z: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = z ^ (z >> np.uint64(30))
        z = z * np.uint64(0xBF58476D1CE4E5B9)
        z = z ^ (z >> np.uint64(27))
        z = z * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    return z


def noise_row(key: int, vocab: int) -> np.ndarray:
    """-log(-log(u)) for every vocabulary index, as float32, from the 64-bit row key."""
    with np.errstate(over="ignore"):
        i = np.arange(1, vocab + 1, dtype=np.uint64)
        bits = _mix64_np(np.uint64(key & MASK64) + i * np.uint64(0x9E3779B97F4A7C15))
    u = ((bits >> np.uint64(41)).astype(np.float32) + np.float32(0.5)) * np.float32(2.0 ** -23)
    return (-np.log(-np.log(u))).astype(np.float32)


class TorchOps:
    name = "torch-twin"

    def prepare(self, dtype, sampling=True):
        pass

    def check_attention_sizes(self, n_heads, n_kv_heads, head_dim, dtype, v_head_dim=None):
        assert n_heads % n_kv_heads == 0 and head_dim > 0

    def embed(self, token_ids, table, scale=1.0, positions=None, position_table=None, rows_dtype=None):
        h = table[token_ids.long()].float() * np.float32(scale)
        if position_table is not None:
            h = h + position_table[positions.long()].float()
        return h if rows_dtype is None else (h, self.stream_rows(h, rows_dtype))

    def stream_rows(self, h, dtype):
        return h if dtype == torch.float32 else h.to(dtype)

    def stream_inject(self, h, rows, row):
        """h += rows (float32 [T, dim] or None) + row (float32 [dim] or None), in place."""
        if rows is not None:
            h += rows
        if row is not None:
            h += row

    def norm_add(self, h, delta, weight, eps, out_dtype, then_weight=None, then_eps=0.0):
        """h += delta / sqrt(mean(delta^2) + eps) * weight (in place, float32); the new rows in out_dtype,
        or, with then_weight, their RMS norm under that weight."""
        bias = None
        if isinstance(delta, PendingProduct):
            bias = delta.bias
            delta = self.linear(delta.x, delta.w, partials_ok=True)
        d = delta.float().sum(0) if delta.dim() == 3 else delta.float()
        if bias is not None:
            d = d + bias
        h += d * torch.rsqrt(d.pow(2).mean(-1, keepdim=True) + eps) * weight
        if then_weight is not None:
            return (h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + then_eps) * then_weight).to(out_dtype)
        return self.stream_rows(h, out_dtype)

    def depth_mix(self, history, coef, n, out, then_weight=None, then_eps=0.0, out_dtype=None):
        """out = sum_j coef[j] * history[j] over the first n levels (float32); with then_weight also the
        RMS norm of out under it, in out_dtype."""
        out.copy_((history[:n] * coef[:n, None, None]).sum(0))
        if then_weight is None:
            return None
        return (out * torch.rsqrt(out.pow(2).mean(-1, keepdim=True) + then_eps) * then_weight).to(out_dtype)

    @staticmethod
    def _act(x, kind):
        if kind == "relu2":
            return torch.relu(x) ** 2
        if kind == "silu":
            return x * torch.sigmoid(x)
        if kind == "gelu_tanh":
            return 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x ** 3)))
        raise ValueError(kind)

    def activation(self, x, kind, out_dtype=None):
        out_dtype = out_dtype or x.dtype
        x = x.float().sum(0) if x.dim() == 3 else x.float()
        return self._act(x, kind).to(out_dtype)

    def gated_act(self, gate_up, activation, out_dtype=None):
        out_dtype = out_dtype or gate_up.dtype
        if gate_up.dim() == 3:
            gate_up = gate_up.float().sum(0)
        hidden = gate_up.shape[1] // 2
        return (self._act(gate_up[:, :hidden].float(), activation) * gate_up[:, hidden:].float()).to(out_dtype)

    def linear_gated_act(self, x, w_gate_up, *, activation):
        return self.gated_act(self.linear(x, w_gate_up, partials_ok=True), activation, out_dtype=x.dtype)

    def rope_store(self, proj, positions, table, *, n_q_heads, n_k_heads, n_v_heads, head_dim, v_head_dim, rot_dims,
                   interleaved, n_extra, k_pages, v_pages, slot_mapping, page_size, out_dtype, bias=None):
        """A row of proj is [q heads | k heads | v heads | extra]: the first rot_dims coordinates of every q
        and k head rotated by the position's angles, k and v written to their pages, sigmoid of the extra
        columns."""
        x = proj.float().sum(0) if proj.dim() == 3 else proj.float()
        if bias is not None:
            x = x + bias
        T = x.shape[0]
        nq, nk, nv = n_q_heads * head_dim, n_k_heads * head_dim, n_v_heads * v_head_dim
        assert x.shape[1] == nq + nk + nv + n_extra
        q, k, v, e = x.split([nq, nk, nv, n_extra], dim=1)
        cs = table[positions.long()][:, None, :rot_dims // 2]        # [T, 1, rot/2, 2]

        def turn(y, heads):
            y = y.reshape(T, heads, head_dim).clone()
            if rot_dims:
                r = y[..., :rot_dims]
                a, b = (r[..., 0::2], r[..., 1::2]) if interleaved else (r[..., :rot_dims // 2], r[..., rot_dims // 2:])
                ya, yb = a * cs[..., 0] - b * cs[..., 1], b * cs[..., 0] + a * cs[..., 1]
                if interleaved:
                    y[..., 0:rot_dims:2], y[..., 1:rot_dims:2] = ya, yb
                else:
                    y[..., :rot_dims // 2], y[..., rot_dims // 2:rot_dims] = ya, yb
            return y

        q = turn(q, n_q_heads)
        if k_pages is not None and n_k_heads:
            sm = slot_mapping.long()
            page, slot = sm // page_size, sm % page_size
            k_pages[page, :, slot] = turn(k, n_k_heads).to(k_pages.dtype)
            v_pages[page, :, slot] = v.reshape(T, n_v_heads, v_head_dim).to(v_pages.dtype)
        return q.to(out_dtype).contiguous(), (torch.sigmoid(e).to(out_dtype).contiguous() if n_extra else None)

    def differential_combine(self, maps, lam, *, eps, out_scale, gate, out_dtype):
        """maps [T, 2 H, dv], map-major: (a1 - lam a2) / sqrt(mean(.^2) + eps) * out_scale * gate[T, H]."""
        T, H2, dv = maps.shape
        a = maps.float().view(T, 2, H2 // 2, dv)
        o = a[:, 0] - np.float32(lam) * a[:, 1]
        o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + eps) * np.float32(out_scale)
        if gate is not None:
            o = o * gate.float()[:, :, None]
        return o.reshape(T, -1).to(out_dtype).contiguous()

    def mingru_scan(self, proj, bias, state, q_start, state_slot, fresh, *, n_seqs, max_q_len, out_dtype):
        """proj [T, 3 W] = [z | u | g] (+ bias): S = (1 - sigmoid(z)) S + sigmoid(z) c(u), out = S * silu(g);
        every request's state row is read (zero for a fresh request) and left updated."""
        x = (proj.float().sum(0) if proj.dim() == 3 else proj.float()) + bias
        W = x.shape[1] // 3
        z, u, g = torch.sigmoid(x[:, :W]), x[:, W:2 * W], x[:, 2 * W:]
        cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
        og = g * torch.sigmoid(g)
        out = torch.empty((x.shape[0], W), dtype=torch.float32, device=x.device)
        qs = q_start.tolist()
        for b in range(n_seqs):
            slot = int(state_slot[b])
            s = torch.zeros(W, device=x.device) if int(fresh[b]) else state[slot].clone()
            for t in range(qs[b], qs[b + 1]):
                s = (1.0 - z[t]) * s + z[t] * cand[t]
                out[t] = s * og[t]
            state[slot] = s
        return out.to(out_dtype)

    def moe_route(self, x, w_router, correction, *, n_experts, top, scale, renormalize, shared_gate, logit_bias=None,
                  score="softmax", n_groups=1, keep_groups=1, group_score_top=2, renorm_eps=0.0):
        z = x.float() @ w_router.t()
        if logit_bias is not None:
            z[:, :n_experts] += logit_bias
        s = torch.softmax(z[:, :n_experts], dim=-1) if score == "softmax" else torch.sigmoid(z[:, :n_experts])
        choice = s if correction is None else s + correction
        if n_groups > 1:
            per = n_experts // n_groups
            g = choice.view(-1, n_groups, per).topk(min(group_score_top, per), dim=-1).values.sum(-1)
            kept = torch.zeros_like(g, dtype=torch.bool).scatter_(1, g.topk(keep_groups, dim=-1).indices, True)
            choice = choice.masked_fill(~kept[:, :, None].expand(-1, -1, per).reshape(choice.shape), float("-inf"))
        chosen = torch.topk(choice, top, dim=-1).indices
        w = torch.gather(s, 1, chosen)
        if renormalize:
            w = w / (w.sum(-1, keepdim=True) + np.float32(renorm_eps))
        gate = torch.sigmoid(z[:, n_experts]).contiguous() if shared_gate else None
        return chosen.to(torch.int32).contiguous(), (w * np.float32(scale)).contiguous(), gate

    def _gated(self, gate, up, activation, act_params):
        if activation == "clamped_swish":
            limit, alpha, offset = act_params
            g = gate.clamp(max=limit)
            return g * torch.sigmoid(alpha * g) * (up.clamp(min=-limit, max=limit) + offset)
        return self._act(gate, activation) * up

    def moe_experts(self, x, chosen, weights, w_up, w_down, *, activation, shared=None, shared_gate=None, gated=False,
                    act_params=None):
        """w_up [E, hidden, dim] (gated: [E, 2 * hidden, dim], rows [gate; up]); w_down [dim, >= E * hidden], expert e's
        matrix in columns e * hidden ..."""
        T, top = chosen.shape
        hidden = w_up.shape[1] // (2 if gated else 1)
        out = torch.zeros((T, w_down.shape[0]), dtype=torch.float32, device=x.device)
        for k in range(top):
            for e in chosen[:, k].unique().tolist():
                rows = (chosen[:, k] == e).nonzero().flatten()
                u = x[rows].float() @ w_up[e].float().t()
                if gated:
                    u = self._gated(u[:, :hidden].to(x.dtype).float(), u[:, hidden:].to(x.dtype).float(), activation, act_params).to(x.dtype)
                else:
                    u = self._act(u, activation).to(x.dtype)
                y = (u.float() @ w_down[:, e * hidden:(e + 1) * hidden].float().t()).to(x.dtype)
                out[rows] += weights[rows, k:k + 1] * y.float()
        if shared is not None:
            sh = shared.float().sum(0) if shared.dim() == 3 else shared.float()
            out += sh if shared_gate is None else sh * shared_gate[:, None]
        return out.to(x.dtype)

    dense_experts = False     # tests switch it on to run the all-experts form of a layer of experts

    def moe_prefers_dense(self, n_tokens, top, n_experts, dtype):
        return self.dense_experts

    def moe_dense_hidden(self, x, chosen, weights, gate, w_up_all, *, n_experts, hidden, activation, gated=False,
                         act_params=None, extra_act_params=None):
        T = x.shape[0]
        u = x.float() @ w_up_all.float().t()
        if gated:            # an expert's columns are [gate | up]; what follows the experts is a shared expert's [gate | up]
            rest = u[:, n_experts * 2 * hidden:]
            u = u[:, :n_experts * 2 * hidden].view(T, n_experts, 2, hidden)
            u = self._gated(u[:, :, 0], u[:, :, 1], activation, act_params).reshape(T, n_experts * hidden)
            if rest.shape[1]:
                sh = rest.shape[1] // 2
                u = torch.cat([u, self._gated(rest[:, :sh], rest[:, sh:], activation, extra_act_params or act_params)], dim=1)
        else:
            u = self._act(u, activation)
        scale = torch.zeros((T, n_experts), dtype=torch.float32, device=x.device)
        scale.scatter_(1, chosen.long(), weights)
        cols = scale.repeat_interleave(hidden, dim=1)
        extra = u.shape[1] - cols.shape[1]
        if extra:
            cols = torch.cat([cols, (gate[:, None] if gate is not None else torch.ones(T, 1)).expand(T, extra)], dim=1)
        return (u * cols).to(x.dtype)

    def glu(self, gate_up, out_dtype=None, *, limit, alpha, up_offset):
        out_dtype = out_dtype or gate_up.dtype
        if gate_up.dim() == 3:
            gate_up = gate_up.float().sum(0)
        hidden = gate_up.shape[1] // 2
        g = gate_up[:, :hidden].float().clamp(max=limit)
        u = gate_up[:, hidden:].float().clamp(min=-limit, max=limit)
        return (g * torch.sigmoid(alpha * g) * (u + up_offset)).to(out_dtype)

    def linear_glu(self, x, w_gate_up, *, limit, alpha, up_offset):
        return self.glu(self.linear(x, w_gate_up, partials_ok=True), out_dtype=x.dtype, limit=limit, alpha=alpha,
                        up_offset=up_offset)

    def project_and_store(self, proj, *, n_q, n_k, n_v, n_extra, bias, q_norm, k_norm, eps, k_pages, v_pages,
                          slot_mapping, page_size, out_dtype, norm_head_dim=None):
        """A row of proj is [q | k | v | extra].  Bias added, q and k each normalised over their whole
        width (where a weight is given), k and v written to their pages, sigmoid of the extra columns."""
        x = proj.float().sum(0) if proj.dim() == 3 else proj.float()
        assert x.shape[1] == n_q + n_k + n_v + n_extra
        if bias is not None:
            x = x + bias
        q, k, v, e = x.split([n_q, n_k, n_v, n_extra], dim=1)
        if norm_head_dim:            # every head by itself, one weight for all heads
            def per_head(y, w):
                y = y.unflatten(1, (-1, norm_head_dim))
                return (y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + eps) * w).flatten(1)
            q = per_head(q, q_norm) if q_norm is not None else q
            k = per_head(k, k_norm) if k_norm is not None and n_k else k
        else:
            if q_norm is not None:
                q = q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + eps) * q_norm
            if k_norm is not None and n_k:
                k = k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + eps) * k_norm
        if k_pages is not None and n_k:
            sm = slot_mapping.long()
            page, slot = sm // page_size, sm % page_size
            k_pages[page, :, slot] = k.reshape(k.shape[0], k_pages.shape[1], k_pages.shape[3]).to(k_pages.dtype)
            if v_pages is not None and n_v:
                v_pages[page, :, slot] = v.reshape(v.shape[0], v_pages.shape[1], v_pages.shape[3]).to(v_pages.dtype)
        return q.to(out_dtype).contiguous(), (torch.sigmoid(e).to(out_dtype).contiguous() if n_extra else None)

    # ---- sums, short convolutions and recurrences with a matrix state
    def stream_add(self, h, *, normed, coef, eps, plain, out_dtype):
        """h += coef * sum_i t_i / sqrt(mean(t_i^2) + eps) * w_i + sum_j p_j (in place, float32); the new rows in out_dtype."""
        for t, w in normed:
            t = t.float().sum(0) if t.dim() == 3 else t.float()
            h += np.float32(coef) * (t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps) * w)
        for p in plain:
            h += p.float().sum(0) if p.dim() == 3 else p.float()
        return self.stream_rows(h, out_dtype)

    def short_conv(self, x, w, state, q_start, state_slot, fresh, *, n_seqs, max_q_len, activation, residual, out_dtype,
                   bias=None):
        """Causal convolution over time per channel: out_t = sum_j w[:, j] x_(t - taps + 1 + j) (+ x_t with residual),
        then the activation.  state [slots, taps - 1, C] holds every request's last inputs (zeros for a fresh one)."""
        C, taps = w.shape
        xf = x.float()
        out = torch.empty((x.shape[0], C), dtype=torch.float32, device=x.device)
        qs = q_start.tolist()
        for b in range(n_seqs):
            slot = int(state_slot[b])
            rows = xf[qs[b]:qs[b + 1]]
            if taps > 1:
                before = torch.zeros((taps - 1, C)) if int(fresh[b]) else state[slot].clone()
                full = torch.cat([before, rows])
                state[slot] = full[-(taps - 1):]
            else:
                full = rows
            y = sum(full[j:j + rows.shape[0]] * w[:, j] for j in range(taps))
            out[qs[b]:qs[b + 1]] = y + rows if residual else y
        if bias is not None:
            out = out + bias
        if activation is not None:
            out = self._act(out, activation)
        return out.to(out_dtype)

    def recurrence_prep(self, x, *, scale, n_heads, head_dim, positions=None, table=None, rot_dims=0, unit_eps=None):
        """float32 [T, n_heads * head_dim]: rotated by position on the first rot_dims coordinates of every head
        (coordinate i with i + rot_dims / 2), or made unit vectors per head; then times scale."""
        y = x.float().unflatten(1, (n_heads, head_dim)).clone()
        if table is not None and rot_dims:
            half = rot_dims // 2
            cs = table[positions.long()][:, None, :half]
            a, b = y[..., :half].clone(), y[..., half:rot_dims].clone()
            y[..., :half] = a * cs[..., 0] - b * cs[..., 1]
            y[..., half:rot_dims] = b * cs[..., 0] + a * cs[..., 1]
        if unit_eps is not None:
            y = y * torch.rsqrt(y.pow(2).sum(-1, keepdim=True) + unit_eps)
        return (y * np.float32(scale)).flatten(1).contiguous()

    def linear_recurrence(self, q, k, v, state, q_start, state_slot, fresh, *, n_seqs, max_q_len, decay=None,
                          beta_logits=None, decay_logits=None, decay_rate=None, decay_bias=None):
        """state [slots, H, dv, dk] float32 (S transposed: a column's keys side by side); q, k float32 [T, G * dk] (G heads shared by H / G value heads each), v [T, H * dv].
        decay: S = decay_h S + k v^T.  Otherwise the gated delta rule: S = g S; u = beta (v - S^T k); S += k u^T.  o = S^T q."""
        H, dv, dk = state.shape[1:]
        G = q.shape[1] // dk
        T = q.shape[0]
        qh, kh = q.view(T, G, dk).float(), k.view(T, G, dk).float()
        vh = v.float().reshape(T, H, dv)
        if decay is None:
            beta = torch.sigmoid(beta_logits.float())
            g = torch.exp(-decay_rate * torch.nn.functional.softplus(decay_logits.float() + decay_bias))
        out = torch.empty((T, H, dv), dtype=torch.float32, device=q.device)
        qs = q_start.tolist()
        for b in range(n_seqs):
            slot = int(state_slot[b])
            S = torch.zeros((H, dk, dv)) if int(fresh[b]) else state[slot].transpose(1, 2).clone()
            for t in range(qs[b], qs[b + 1]):
                kt = kh[t].repeat_interleave(H // G, dim=0)
                qt = qh[t].repeat_interleave(H // G, dim=0)
                if decay is not None:
                    S = decay[:, None, None] * S + kt[:, :, None] * vh[t][:, None, :]
                else:
                    S = g[t][:, None, None] * S
                    u = beta[t][:, None] * (vh[t] - torch.einsum("hkv,hk->hv", S, kt))
                    S = S + kt[:, :, None] * u[:, None, :]
                out[t] = torch.einsum("hkv,hk->hv", S, qt)
            state[slot] = S.transpose(1, 2)
        return out.flatten(1)

    def head_norm_gate(self, o, gate, weight, eps, *, head_dim, out_dtype):
        """Every head of o (float32 [T, H * head_dim]) divided by its root mean square, times the weight (if any), times silu(gate)."""
        y = o.float().unflatten(1, (-1, head_dim))
        y = y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + eps)
        if weight is not None:
            y = y * weight
        g = gate.float()
        return (y.flatten(1) * g * torch.sigmoid(g)).to(out_dtype)

    def side_gate(self, u, token_ids, table, out_dtype):
        """gelu_tanh(u) * table[token]."""
        u = u.float().sum(0) if u.dim() == 3 else u.float()
        return (self._act(u, "gelu_tanh") * table[token_ids.long()].float()).to(out_dtype)

    def sum_partials(self, parts, out_dtype):
        return parts.float().sum(0).to(out_dtype)

    def polynorm(self, z, coef, eps, out_dtype):
        """a N(z) + b N(z^2) + c N(z^3) + e with N(y) = y / sqrt(mean(y^2) + eps) over a row; coef = (a, b, c, e)."""
        z = z.float().sum(0) if z.dim() == 3 else z.float()
        n = lambda y: y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + eps)
        return (coef[0] * n(z) + coef[1] * n(z * z) + coef[2] * n(z * z * z) + coef[3]).to(out_dtype)

    def head_linear(self, x, w, gate=None):
        """x [T, H, K] against w [H, N, K]: out[t, h] = w[h] @ x[t, h] (times gate [T, H * N] where given)."""
        out = torch.einsum("thk,hnk->thn", x.float(), w.float()).to(x.dtype)
        if gate is not None:
            out = (out.float() * gate.float().view(out.shape)).to(x.dtype)
        return out.contiguous()

    def latent_store(self, proj, positions, table, *, n_q, n_latent, n_rot, n_extra, q_norm, latent_norm, eps, interleaved,
                     k_pages, slot_mapping, page_size, out_dtype):
        """A row of proj is [q latent | kv latent | rotated key part | extra]: both latents RMS-normed under their
        weights, the key part rotated by the position, [kv latent | key part] written to the pages, the q latent and
        sigmoid(extra) returned."""
        x = proj.float().sum(0) if proj.dim() == 3 else proj.float()
        assert x.shape[1] == n_q + n_latent + n_rot + n_extra
        q, c, r, e = x.split([n_q, n_latent, n_rot, n_extra], dim=1)
        q = q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + eps) * q_norm
        c = c * torch.rsqrt(c.pow(2).mean(-1, keepdim=True) + eps) * latent_norm
        r = self._turn(r[:, None, :], positions, table, n_rot, interleaved)[:, 0]
        sm = slot_mapping.long()
        k_pages[sm // page_size, 0, sm % page_size] = torch.cat([c, r], dim=1).to(k_pages.dtype)
        return q.to(out_dtype).contiguous(), (torch.sigmoid(e).to(out_dtype).contiguous() if n_extra else None)

    @staticmethod
    def _turn(y, positions, table, rot, interleaved):
        """y [T, heads, >= rot] float32: its first rot coordinates rotated by the positions' angles."""
        y = y.clone()
        if rot:
            cs = table[positions.long()][:, None, :rot // 2]
            r = y[..., :rot]
            a, b = (r[..., 0::2], r[..., 1::2]) if interleaved else (r[..., :rot // 2], r[..., rot // 2:])
            ya, yb = a * cs[..., 0] - b * cs[..., 1], b * cs[..., 0] + a * cs[..., 1]
            if interleaved:
                y[..., 0:rot:2], y[..., 1:rot:2] = ya, yb
            else:
                y[..., :rot // 2], y[..., rot // 2:rot] = ya, yb
        return y

    def latent_query(self, q, w_uk_t, positions, table, *, rot_dim, interleaved):
        """q [T, H, d + rot_dim], w_uk_t [H, rank, d]: [w_uk_t[h] @ q[t, h, :d] | rotated q[t, h, d:]]."""
        d = q.shape[2] - rot_dim
        lat = torch.einsum("thk,hnk->thn", q[..., :d].float(), w_uk_t.float())
        rot = self._turn(q[..., d:].float(), positions, table, rot_dim, interleaved)
        return torch.cat([lat, rot], dim=-1).to(q.dtype).contiguous()

    def selective_scan(self, x, dt, B, C, z, A, D, dt_bias, state, q_start, state_slot, fresh, *, n_seqs, max_q_len, out_dtype):
        """S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n with dt = softplus(dt + dt_bias); y = S C + D x; out = y silu(z)."""
        xf, zf, Bf, Cf = x.float(), z.float(), B.float(), C.float()
        step = torch.nn.functional.softplus(dt.float() + dt_bias)
        out = torch.empty(xf.shape, dtype=torch.float32, device=x.device)
        qs = q_start.tolist()
        for b in range(n_seqs):
            slot = int(state_slot[b])
            S = torch.zeros_like(state[slot]) if int(fresh[b]) else state[slot].clone()
            for t in range(qs[b], qs[b + 1]):
                S = torch.exp(step[t][:, None] * A) * S + (step[t] * xf[t])[:, None] * Bf[t][None, :]
                out[t] = (S @ Cf[t] + D * xf[t]) * (zf[t] * torch.sigmoid(zf[t]))
            state[slot] = S
        return out.to(out_dtype)

    def rmsnorm(self, h, delta, weight, eps, out_dtype, rows=None, deferred=False):
        if isinstance(delta, PendingProduct):
            delta = delta.take(self)
        if delta is not None and delta.dim() == 3:
            delta = delta.float().sum(0)
        x = h if delta is None else h + delta.float()
        if rows is None:
            if delta is not None:
                h.copy_(x)
        else:
            x = x[rows.long()]
        if deferred:
            assert rows is None
            return RowScaled((x * weight).to(out_dtype), x.pow(2).sum(-1, keepdim=True), x.shape[1], float(eps))
        y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * weight
        return y.to(out_dtype)

    fuse_residual = True      # tests switch it off to compare the two ways

    def can_fuse_residual(self, pending, h):
        return (self.fuse_residual and isinstance(pending, PendingProduct) and pending.x.dtype == torch.bfloat16
                and pending.x.shape[0] <= 64 and pending.w.shape[0] % 4 == 0 and pending.x.shape[1] % 8 == 0)

    def linear_residual_norm(self, pending, h, weight, eps, slab=128):
        """h += bf16(x @ w.T) (float32, in place); rows bf16(h * weight) and the sum of squares in parts
        of ``slab`` columns, as the kernel leaves them."""
        h += (pending.x.float() @ pending.w.float().t()).to(torch.bfloat16).float()
        N = h.shape[1]
        parts = [h[:, c:c + slab].pow(2).sum(-1) for c in range(0, N, slab)]
        return RowScaled((h * weight).to(torch.bfloat16), torch.stack(parts, 1), N, float(eps))

    def swiglu(self, gate_up, out_dtype=None):
        scale = None
        if isinstance(gate_up, RowScaled):
            scale, gate_up = gate_up.scale(), gate_up.x
        out_dtype = out_dtype or gate_up.dtype
        if gate_up.dim() == 3:
            gate_up = gate_up.float().sum(0)
        hidden = gate_up.shape[1] // 2
        g, u = gate_up[:, :hidden].float(), gate_up[:, hidden:].float()
        if scale is not None:
            g, u = g * scale[:, None], u * scale[:, None]
        return (g / (1 + torch.exp(-g)) * u).to(out_dtype)

    def linear_swiglu(self, x, w13, fused=None):
        if isinstance(x, RowScaled):
            # gate and up pass through the activation dtype unscaled, as between the product and its epilogue
            return self.swiglu(x.follow(self.linear(x.x, w13)), out_dtype=x.x.dtype)
        return self.swiglu(self.linear(x, w13), out_dtype=x.dtype)

    def linear(self, x, w, out_dtype=None, partials_ok=False):
        if isinstance(x, RowScaled):
            return x.follow(self.linear(x.x, w, out_dtype, partials_ok))
        out_dtype = out_dtype or x.dtype
        if x.dtype == torch.float32:
            return (x @ w.t()).to(out_dtype)
        return (x.float() @ w.float().t()).to(out_dtype)

    def gemm_simt(self, x, w, out_dtype):
        return (x.float() @ w.float().t()).to(out_dtype)

    def rope_kv_write(self, qkv, positions, table, *, n_heads, n_kv_heads, head_dim, interleaved,
                      k_pages, v_pages, slot_mapping, page_size, out_dtype=None):
        scale = None
        if isinstance(qkv, RowScaled):
            scale, qkv = qkv.scale(), qkv.x
        out_dtype = out_dtype or qkv.dtype
        if qkv.dim() == 3:
            qkv = qkv.float().sum(0)
        T = qkv.shape[0]
        x = qkv.float().view(T, n_heads + 2 * n_kv_heads, head_dim)
        if scale is not None:
            x = x * scale[:, None, None]
        cs = table[positions.long()]            # [T, hd/2, 2]
        c, s = cs[:, None, :, 0], cs[:, None, :, 1]
        rot = x[:, : n_heads + n_kv_heads]
        if interleaved:
            a, b = rot[..., 0::2], rot[..., 1::2]
        else:
            a, b = rot[..., : head_dim // 2], rot[..., head_dim // 2:]
        ya, yb = a * c - b * s, b * c + a * s
        out = torch.empty_like(rot)
        if interleaved:
            out[..., 0::2], out[..., 1::2] = ya, yb
        else:
            out[..., : head_dim // 2], out[..., head_dim // 2:] = ya, yb
        q = out[:, :n_heads].to(out_dtype).contiguous()
        if k_pages is not None:
            k = out[:, n_heads:].to(out_dtype)
            v = x[:, n_heads + n_kv_heads:].to(out_dtype)
            sm = slot_mapping.long()
            page, slot = sm // page_size, sm % page_size
            k_pages[page, :, slot] = k
            v_pages[page, :, slot] = v
        return q

    def paged_attention(self, q, k_pages, v_pages, block_table, q_start, kv_len, *, n_seqs, max_q_len,
                        max_kv_len, scale, window, page_size, allow_split=True, impl="auto", n_tokens=None, out=None,
                        keep_first=0, distance_bias=None, distance_buckets=None, gate=None, n_v_heads=None,
                        out_dtype=None, softcap=0.0, sinks=None, value_dim=None):
        T, H, hd = q.shape
        KV = k_pages.shape[1]
        group = H // KV
        if keep_first or distance_bias is not None or gate is not None or v_pages.shape[3] != hd \
                or v_pages.shape[1] != KV or out_dtype not in (None, q.dtype) or softcap or sinks is not None or value_dim:
            assert out is None and n_tokens is None and (n_v_heads or KV) == v_pages.shape[1]
            return self._attention_general(q, k_pages, v_pages, block_table, q_start, kv_len, n_seqs, scale, window,
                                           page_size, keep_first, distance_bias, distance_buckets, gate, out_dtype,
                                           softcap, sinks, value_dim)
        # the same contract as the kernels' front end: the step's bounds cover its requests and fit the table
        assert block_table.shape[1] * page_size >= max_kv_len, "block_table is too narrow for max_kv_len"
        assert int(kv_len[:n_seqs].max()) <= max_kv_len and n_seqs <= block_table.shape[0]
        out = torch.zeros_like(q) if out is None else out
        qs = q_start.tolist()
        kl = kv_len.tolist()
        for b in range(n_seqs):
            ql, L = qs[b + 1] - qs[b], kl[b]
            lo = 0
            if window:
                lo = max(0, (L - ql) - window + 1)
            pos = torch.arange(lo, L, device=q.device)
            pages = block_table[b].long()[pos // page_size]
            assert (pages >= 0).all(), "attention would read a page that was given back"
            k = k_pages[pages, :, pos % page_size].float()     # [n, KV, hd]
            v = v_pages[pages, :, pos % page_size].float()
            qq = q[qs[b]:qs[b + 1]].float()                    # [ql, H, hd]
            qpos = torch.arange(L - ql, L, device=q.device)
            hidden = pos[None, :] > qpos[:, None]
            if window:
                hidden = hidden | (pos[None, :] <= qpos[:, None] - window)
            for h in range(H):
                s = (qq[:, h] @ k[:, h // group].T) * scale
                s = s.masked_fill(hidden, float("-inf"))
                out[qs[b]:qs[b + 1], h] = (torch.softmax(s, -1) @ v[:, h // group]).to(q.dtype)
        return out

    def _attention_general(self, q, k_pages, v_pages, block_table, q_start, kv_len, n_seqs, scale, window, page_size,
                           keep_first, distance_bias, distance_buckets, gate, out_dtype=None, softcap=0.0, sinks=None,
                           value_dim=None):
        """Everything the general kernel can do, key by visible key: kept first tokens behind a
        window, a bias by bucketed distance, values of another size, an output gate per head
        ([T, H]) or per element ([T, H * dv])."""
        T, H, hd = q.shape
        KV, dv, VH = k_pages.shape[1], v_pages.shape[3], v_pages.shape[1]
        if value_dim:        # a stored value is the first so many coordinates of a stored vector
            dv = int(value_dim)
        group = H // KV
        out = torch.zeros((T, H, dv), dtype=out_dtype or q.dtype, device=q.device)
        qs, kl = q_start.tolist(), kv_len.tolist()
        for b in range(n_seqs):
            ql, L = qs[b + 1] - qs[b], kl[b]
            qpos = torch.arange(L - ql, L, device=q.device)
            lo = max(0, (L - ql) - window + 1) if window else 0
            pos = torch.cat([torch.arange(0, min(keep_first, lo), device=q.device), torch.arange(lo, L, device=q.device)])
            pages = block_table[b].long()[pos // page_size]
            assert (pages >= 0).all(), "attention would read a page that was given back"
            k = k_pages[pages, :, pos % page_size].float()
            v = v_pages[pages, :, pos % page_size].float()[..., :dv]
            qq = q[qs[b]:qs[b + 1]].float()
            dist = qpos[:, None] - pos[None, :]
            hidden = dist < 0
            if window:
                hidden = hidden | ((dist >= window) & (pos[None, :] >= keep_first))
            for h in range(H):
                s = (qq[:, h] @ k[:, h // group].T) * scale
                if distance_bias is not None:
                    s = s + distance_bias[distance_buckets[dist.clamp(min=0)].long(), h]
                if softcap:
                    s = np.float32(softcap) * torch.tanh(s / np.float32(softcap))
                s = s.masked_fill(hidden, float("-inf"))
                if sinks is not None:        # one more term in the denominator, without a value
                    s = torch.cat([s, sinks[h].expand(ql, 1)], dim=1)
                    o = torch.softmax(s, -1)[:, :-1] @ v[:, (h // group) % VH]
                else:
                    o = torch.softmax(s, -1) @ v[:, (h // group) % VH]
                if gate is not None:
                    g = gate[qs[b]:qs[b + 1]].float()
                    o = o * (g[:, h:h + 1] if gate.shape[1] == H else g.view(ql, H, dv)[:, h])
                out[qs[b]:qs[b + 1], h] = o.to(out.dtype)
        return out

    def sample(self, logits, temperature=None, top_k=None, row_keys=None):
        n, vocab = logits.shape
        out = torch.empty(n, dtype=torch.int32, device=logits.device)
        for r in range(n):
            row = logits[r].float().cpu()
            t = 0.0 if temperature is None else float(temperature[r])
            if not t > 0:
                out[r] = int(torch.argmax(row))
                continue
            score = row / np.float32(max(t, 1e-5))
            k = 0 if top_k is None else int(top_k[r])
            if 0 < k < vocab:
                pivot = torch.topk(row, k).values[-1]
                score = score.masked_fill(row < pivot, float("-inf"))
            key = int(row_keys[r]) & MASK64
            score = score + torch.from_numpy(noise_row(key, vocab))
            out[r] = int(torch.argmax(score))
        return out
