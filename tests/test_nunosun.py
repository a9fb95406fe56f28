"""Nunosun through the engine against the plain implementation (``plain_nunosun``).

Every test runs three ways: over the kernels' plain PyTorch twins on the CPU (the package's
parts, cache manager, step function and scheduler are the ones under test there), and on the GPU
over the CUDA kernels in float32 and in bfloat16.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

import nunosun_cases as nc
import plain_nunosun as plain
from nunosun_cases import BACKENDS


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("name", list(nc.CASES))
def test_whole_prompt_decoding_and_portions(tmp_path, backend, name):
    """A whole prompt in one step, the same tokens one by one from the first on, and portions of
    several sizes down to two tokens (cut inside pages, windows and the kernels' chunks) all give
    the plain logits."""
    cfg, tensors, folder, page = nc.case_folder(tmp_path, name, dtype=nc.stored_dtype(backend))
    n = 70 if name != "wide" else 200
    tokens = nc.clear_tokens(cfg, tensors, n, seed=1, dtype=backend[1])
    want = nc.plain_logits(cfg, tensors, tokens, backend[1])
    rp = nc.make_replayer(folder, backend, 4 * 256, page)
    want.check(nc.feed(rp, "whole", tokens, [n]), "whole prompt")
    want.check(nc.feed(rp, "single", tokens, [] if n <= 70 else [n - 60]), "token by token")
    want.check(nc.feed(rp, "cut", tokens, [2, 3, 2, 7, 16, 2, 5, 9, 2, 11]), "portions")
    want.check(nc.feed(rp, "cut2", tokens, [page + 1, 2 * page - 1, 2, 2, 33]), "portions across pages")
    if n > 130:
        want.check(nc.feed(rp, "cut3", tokens, [47, 2, 49, 16, 17, 2, 63]), "portions at the edges of windows and chunks")
    assert rp.engine.cache.n_live() == 0


@pytest.mark.parametrize("backend", BACKENDS)
def test_batches_of_unequal_requests(tmp_path, backend):
    """Four live requests of different lengths, portions beside single tokens, in a pool so small
    that pages and state slots are used again: every request's logits are those it gets alone."""
    cfg, tensors, folder, page = nc.case_folder(tmp_path, "mixed", dtype=nc.stored_dtype(backend))
    lengths = [61, 9, 34, 1, 47, 22, 80]
    reqs = {f"r{i}": nc.clear_tokens(cfg, tensors, n, seed=10 + i, dtype=backend[1]) for i, n in enumerate(lengths)}
    want = {rid: nc.plain_logits(cfg, tensors, toks, backend[1]) for rid, toks in reqs.items()}
    rp = nc.make_replayer(folder, backend, 4 * 128, page, max_num_seqs=4)
    rng = np.random.default_rng(0)
    waiting, live, at, got = list(reqs), [], {}, {rid: [] for rid in reqs}
    step = 0
    while waiting or live:
        while waiting and len(live) < 4:
            rid = waiting.pop(0)
            live.append(rid)
            at[rid] = 0
        entries, end = [], []
        for rid in live:
            if len(live) > 1 and rng.random() < 0.2:
                continue                                     # left out of this step
            left = len(reqs[rid]) - at[rid]
            n = 1 if (at[rid] > len(reqs[rid]) // 2) else int(min(left, rng.choice([2, 3, 5, 8, 13, 24])))
            entries.append({"id": rid, "tokens": reqs[rid][at[rid]:at[rid] + n], "want": list(range(n))})
            at[rid] += n
            if at[rid] == len(reqs[rid]):
                end.append(rid)
        if not entries:
            continue
        out = rp.run_step({"step": step, "entries": entries, "end": end})
        rp.engine.cache.check_invariants()
        row = 0
        for e in entries:
            got[e["id"]].append(out[row:row + len(e["tokens"])])
            row += len(e["tokens"])
        live = [rid for rid in live if rid not in end]
        step += 1
    for rid in reqs:
        want[rid].check(np.concatenate(got[rid]), rid)
    assert rp.engine.cache.n_live() == 0


@pytest.mark.parametrize("backend", BACKENDS)
def test_long_decoding_and_a_slot_used_again(tmp_path, backend):
    """A short prompt and 250 tokens decoded one by one (recorded steps on the GPU), then another
    request in the same state slot and pages: its first tokens must not feel the matrices and the
    convolutions' inputs that the first one left behind."""
    cfg, tensors, folder, page = nc.case_folder(tmp_path, "awkward", dtype=nc.stored_dtype(backend))
    tokens = nc.clear_tokens(cfg, tensors, 255, seed=3, dtype=backend[1])
    rp = nc.make_replayer(folder, backend, 256, page, max_num_seqs=1)
    nc.plain_logits(cfg, tensors, tokens, backend[1]).check(nc.feed(rp, "long", tokens, [5]), "long decoding")
    again = nc.clear_tokens(cfg, tensors, 20, seed=4, dtype=backend[1])
    nc.plain_logits(cfg, tensors, again, backend[1]).check(nc.feed(rp, "again", again, [1, 1, 3]), "the slot's next request")
    rp.engine.cache.check_invariants()


def test_layers_of_experts_as_one_matrix(tmp_path):
    """The form a decode batch takes on the GPU (every expert's [gate; up] as one matrix, zeros where a
    token did not choose an expert), forced for every step over the kernels' twins: the same logits."""
    from torch_ops import TorchOps
    from torchllms_b200.engine.replay import Replayer
    cfg, tensors, folder, page = nc.case_folder(tmp_path, "mixed")
    tokens = nc.tokens_for(cfg, 40, seed=2)
    ops = TorchOps()
    ops.dense_experts = True
    rp = Replayer(folder, "float32", 256, page_size=page, device="cpu", ops=ops, max_num_seqs=2)
    nc.plain_logits(cfg, tensors, tokens, "float32").check(nc.feed(rp, "a", tokens, [17, 2]), "all experts as one matrix")


# ---------------------------------------------------------------- one mechanism at a time

def _one_layer(layer, **kw):
    return nc.config([layer], **kw)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("kind", ["parallel", "delta", "delta-one-tap", "parallel-whole-rotation"])
def test_each_mixer_alone(tmp_path, backend, kind):
    """One layer without a feed-forward: the mixer, the convolution in front of it and the token's
    side input are all there is between the embedding and the head."""
    layer = {"parallel": nc.parallel_layer(window=5, bias_rows=8, bias_max=30.0),
             "parallel-whole-rotation": nc.parallel_layer(heads=2, kv_heads=2, dim=8, vdim=8, window=33, r_heads=2, r_dim=8, r_vdim=8,
                                                          decay=(0.5, 1.0), rot_dims=8, base=7.0, bias_rows=4, bias_max=3.0),
             "delta": nc.delta_layer(),
             "delta-one-tap": nc.delta_layer(heads=1, kv_heads=1, dim=4, vdim=4, conv=1)}[kind]
    cfg = _one_layer(layer, width=40, vocab=53, taps=2 if kind == "delta" else 5, side=1 if kind == "delta" else 7)
    dtype = nc.stored_dtype(backend)
    tensors = nc.stored(nc.tensors_for(cfg, seed=len(kind), sharp=3.0 if backend[1] == "float32" else 1.0), dtype)
    tokens = nc.tokens_for(cfg, 90, seed=5)
    want = nc.plain_logits(cfg, tensors, tokens, backend[1])
    rp = nc.make_replayer(nc.write_folder(tmp_path, kind, cfg, tensors, dtype), backend, 256, 8)
    want.check(nc.feed(rp, "p", tokens, [90]), "prompt")
    want.check(nc.feed(rp, "d", tokens, [3]), "decoded")
    want.check(nc.feed(rp, "c", tokens, [2, 2, 31, 2, 9, 17, 2]), "portions")


@pytest.mark.parametrize("backend", BACKENDS)
def test_keys_at_the_windows_edge(tmp_path, backend):
    """The table of distances is made so that the key at the window's last place outweighs all nearer
    ones, and so that a key one place further would outweigh even that one if it were seen: a
    window that is one key too wide or too narrow moves every row by far more than rounding.  The
    windows are shorter than, equal to and longer than a page, in prompts, decoded alone and in
    portions that start at every offset to the window's edge."""
    for window, rows, far in ((5, 6, 5.0), (8, 12, 8.0), (21, 44, 40.0)):
        layer = nc.parallel_layer(heads=2, kv_heads=1, dim=8, vdim=8, window=window, bias_max=far, bias_rows=rows, r_heads=1, r_dim=4,
                                  r_vdim=4, decay=(0.5,), rot_dims=4)
        cfg = _one_layer(layer, width=32, vocab=50)
        dtype = nc.stored_dtype(backend)
        tensors = nc.tensors_for(cfg, seed=window, sharp=1.0)
        rel = torch.zeros(rows, 2)
        inside, outside = plain.distance_row(window - 1, rows, far), plain.distance_row(window, rows, far)
        assert inside != outside, "the test's table cannot tell the window's last key from the next one"
        rel[inside], rel[outside:] = 6.0, 12.0
        tensors["l0.mix.left.rel"] = rel
        tensors["l0.mix.right.out"] = 0.05 * tensors["l0.mix.right.out"]          # the window's side carries the result
        tensors = nc.stored(tensors, dtype)
        tokens = nc.tokens_for(cfg, 75, seed=window)
        want = nc.plain_logits(cfg, tensors, tokens, backend[1])
        wider = dict(cfg, layers=[nc.parallel_layer(heads=2, kv_heads=1, dim=8, vdim=8, window=window + 1, bias_max=far, bias_rows=rows,
                                                    r_heads=1, r_dim=4, r_vdim=4, decay=(0.5,), rot_dims=4)])
        assert np.abs(nc.plain_logits(wider, tensors, tokens, backend[1])[window + 3:] - want[window + 3:]).max() > 0.05, \
            "the test's inputs do not show a window that is one key too wide"
        rp = nc.make_replayer(nc.write_folder(tmp_path, f"edge{window}", cfg, tensors, dtype), backend, 256, 8)
        want.check(nc.feed(rp, "p", tokens, [75]), f"prompt, window {window}")
        want.check(nc.feed(rp, "d", tokens, [window - 2]), f"decoded, window {window}")
        want.check(nc.feed(rp, "c", tokens, [window - 1, 2, window, 2, window + 1, 3]), f"portions, window {window}")


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("kind", ["retention", "delta"])
def test_a_state_that_remembers_the_first_token(tmp_path, backend, kind):
    """A matrix state that hardly forgets keeps its first token for hundreds of steps: the last logits
    depend on token 0 (proved on the plain implementation), so a state that is lost, zeroed or
    mixed up at the start of a portion or between steps shows."""
    dtype = nc.stored_dtype(backend)
    if kind == "retention":
        layer = nc.parallel_layer(heads=1, kv_heads=1, dim=4, vdim=4, window=3, bias_rows=4, bias_max=5.0, r_heads=2, r_dim=8, r_vdim=16,
                                  decay=(1.0, 0.999), rot_dims=6, base=100.0)
    else:
        layer = nc.delta_layer(heads=2, kv_heads=1, dim=64, vdim=12, conv=2)      # (many directions: later keys hardly touch the first)
    cfg = _one_layer(layer, width=32, vocab=50, taps=2)
    tensors = nc.tensors_for(cfg, seed=2)
    marked = cfg["vocab"] - 1            # a token that only position 0 has, and that writes a large value into the state
    if kind == "retention":
        tensors["l0.mix.left.out"] = 0.05 * tensors["l0.mix.left.out"]
        tensors["l0.mix.right.v"] = tensors["l0.mix.right.v"] * 0.3
        x = plain.rms(tensors["embed"][marked].double(), cfg["norm"]["eps"])
        tensors["l0.mix.right.v"] = (tensors["l0.mix.right.v"].double() + 4.0 * torch.outer(torch.ones(32, dtype=torch.float64), x / (x @ x) ** 0.5)).float()
    else:
        tensors["l0.mix.A_log"].fill_(-9.0)          # decays of all but one
        tensors["l0.mix.b"] = 0.05 * tensors["l0.mix.b"]
    tensors = nc.stored(tensors, dtype)
    n = 200
    tokens = [marked] + np.random.default_rng(5).integers(0, marked, size=n - 1).tolist()
    want = nc.plain_logits(cfg, tensors, tokens, backend[1])
    other = [0] + tokens[1:]
    assert np.abs(nc.plain_logits(cfg, tensors, other, backend[1])[n - 1] - want[n - 1]).max() > 0.05, \
        "the test's inputs do not show the first token at the end"
    rp = nc.make_replayer(nc.write_folder(tmp_path, "memory" + kind, cfg, tensors, dtype), backend, 512, 16)
    want.check(nc.feed(rp, "p", tokens, [n]), "prompt")
    want.check(nc.feed(rp, "d", tokens, [1]), "decoded from the second token on")
    want.check(nc.feed(rp, "c", tokens, [15, 2, 16, 17, 64, 2]), "portions around the chunk size")


def _ops_for(backend):
    if backend[0] == "cpu":
        from torch_ops import TorchOps
        return TorchOps(), "cpu", torch.float32
    from torchllms_b200.kernels import get_ops
    return get_ops(), "cuda", (torch.float32 if backend[1] == "float32" else torch.bfloat16)


@pytest.mark.parametrize("backend", BACKENDS)
def test_small_kernels_against_the_plain_functions(backend):
    """The sum of normed and plain terms, PolyNorm, the side input's gate, the short convolution with its
    state, the rotation and the unit vectors, both recurrences, the head norm with its gate, the router
    with a bias and gated experts, each against the plain implementation's function or the
    equations written out here in float64, at sizes that are and are not multiples of four."""
    ops, dev, dtype = _ops_for(backend)
    g = torch.Generator().manual_seed(3)
    tol = dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)
    rnd = lambda *shape: torch.randn(*shape, generator=g)
    i32 = lambda xs: torch.tensor(xs, dtype=torch.int32, device=dev)
    close = lambda got, want, **kw: torch.testing.assert_close(got.float().cpu(), want.float(), **(kw or tol))
    for T, dim in ((1, 64), (7, 42), (150, 256)):
        # the sum: two normed terms and two plain ones onto the stream
        h, a, b, c, d = rnd(T, dim), rnd(T, dim).to(dtype), rnd(T, dim).to(dtype), rnd(T, dim).to(dtype), rnd(T, dim).to(dtype)
        wa, wb = rnd(dim), rnd(dim)
        want = h.double() + 0.5 * (plain.rms(a.double(), 1e-5) * wa + plain.rms(b.double(), 1e-5) * wb) + c.double() + d.double()
        hd = h.clone().to(dev)
        rows = ops.stream_add(hd, normed=((a.to(dev), wa.to(dev)), (b.to(dev), wb.to(dev))), coef=0.5, eps=1e-5,
                              plain=(c.to(dev), d.to(dev)), out_dtype=dtype)
        close(hd, want, atol=2e-5, rtol=2e-5)
        close(rows, want)
        # the same with a normed and a plain term that arrive as partial sums of a split-K product
        pa, pc = rnd(3, T, dim), rnd(2, T, dim)
        want = h.double() + 0.5 * (plain.rms(pa.double().sum(0), 1e-5) * wa + plain.rms(b.double(), 1e-5) * wb) + pc.double().sum(0)
        hd = h.clone().to(dev)
        ops.stream_add(hd, normed=((pa.to(dev), wa.to(dev)), (b.to(dev), wb.to(dev))), coef=0.5, eps=1e-5, plain=(pc.to(dev),), out_dtype=dtype)
        close(hd, want, atol=3e-5, rtol=3e-5)
        close(ops.sum_partials(pa.to(dev), dtype), pa.double().sum(0))
        # PolyNorm
        z, coef = rnd(T, dim).to(dtype), torch.tensor([0.9, -0.4, 0.3, 0.2])
        zd = z.double()
        want = 0.9 * plain.rms(zd, 1e-6) - 0.4 * plain.rms(zd ** 2, 1e-6) + 0.3 * plain.rms(zd ** 3, 1e-6) + 0.2
        close(ops.polynorm(z.to(dev), coef.to(dev), 1e-6, dtype), want)
        zp = torch.stack([0.25 * z.float(), 0.75 * z.float()])
        close(ops.polynorm(zp.to(dev), coef.to(dev), 1e-6, dtype), want)
        # the side input's gate
        s = 5 if dim % 4 else 24
        u, table, ids = rnd(T, s).to(dtype), rnd(11, s).to(dtype), torch.randint(0, 11, (T,), generator=g)
        close(ops.side_gate(u.to(dev), i32(ids.tolist()), table.to(dev), dtype), plain.gelu_tanh(u.double()) * table.double()[ids])
        up = torch.stack([0.5 * u.float(), 0.25 * u.float(), 0.25 * u.float()])
        close(ops.side_gate(up.to(dev), i32(ids.tolist()), table.to(dev), dtype), plain.gelu_tanh(u.double()) * table.double()[ids])
        # the head norm with its gate: heads inside a wider row of gates
        H, hd_ = (3, 10) if dim % 4 else (4, 32)
        o, wide, w = rnd(T, H * hd_), rnd(T, H * hd_ + 6).to(dtype), rnd(hd_)
        gate = wide[:, 3:3 + H * hd_]
        want = (plain.rms(o.double().view(T, H, hd_), 1e-5) * w.double()).flatten(1) * plain.silu(gate.double())
        close(ops.head_norm_gate(o.to(dev), wide.to(dev)[:, 3:3 + H * hd_], w.to(dev), 1e-5, head_dim=hd_, out_dtype=dtype), want)
        want = plain.rms(o.double().view(T, H, hd_), 1e-5).flatten(1) * plain.silu(gate.double())
        close(ops.head_norm_gate(o.to(dev), wide.to(dev)[:, 3:3 + H * hd_], None, 1e-5, head_dim=hd_, out_dtype=dtype), want)
        # rotation (a part of the head, positions far from zero) and unit vectors
        rot = 6 if dim % 4 else 16
        from torchllms_b200.parts.rope import precise_rotary_table
        table = precise_rotary_table(rot, 1000.0, 1.0, 600, dev)
        x = rnd(600, H * hd_).to(dtype)
        want = plain.rotate_half(x.double().view(600, H, hd_), rot, 1000.0).flatten(1) * 0.25
        got = ops.recurrence_prep(x.to(dev), scale=0.25, n_heads=H, head_dim=hd_, positions=i32(list(range(600))), table=table, rot_dims=rot)
        close(got, want, atol=2e-5, rtol=2e-5)
        xh = x.double().view(600, H, hd_)
        want = (xh / torch.sqrt(xh.pow(2).sum(-1, keepdim=True) + 1e-6)).flatten(1) * 0.5
        close(ops.recurrence_prep(x.to(dev), scale=0.5, n_heads=H, head_dim=hd_, unit_eps=1e-6), want, atol=2e-5, rtol=2e-5)
    # the short convolution: three requests, one of them going on from a state, in slots of their own; x is a column
    # range of a wider row and the state a field of a wider row
    for taps, C, act, residual in ((4, 44, "silu", False), (3, 30, None, True), (1, 9, "silu", False), (8, 130, None, True)):
        lens, slots = [19, 1, 6], [2, 0, 3]
        wide = rnd(sum(lens), C + 5).to(dtype)
        x, w = wide[:, 2:2 + C], rnd(C, taps)
        before = rnd(taps - 1, C)                      # what the second request's earlier inputs were
        state_all = torch.zeros(4, (taps - 1) * C + 7)
        state = state_all[:, 4:4 + (taps - 1) * C].unflatten(1, (taps - 1, C)) if taps > 1 else None
        if taps > 1:
            state[0] = before
            state[2] = 7.0                             # left behind by an earlier request: a fresh one must not read it
        want, new_state, at = [], {}, 0
        for n, slot, fresh in zip(lens, slots, (True, False, True)):
            full = torch.cat([torch.zeros(taps - 1, C) if fresh else before, x[at:at + n].float()]).double()
            y = plain.causal_conv(full, w.double())[taps - 1:]
            y = y + full[taps - 1:] if residual else y
            want.append(plain.silu(y) if act else y)
            new_state[slot] = full[full.shape[0] - (taps - 1):]
            at += n
        sd = state_all.to(dev)
        sv = sd[:, 4:4 + (taps - 1) * C].unflatten(1, (taps - 1, C)) if taps > 1 else None
        got = ops.short_conv(wide.to(dev)[:, 2:2 + C], w.to(dev), sv, i32([0, 19, 20, 26]), i32(slots), i32([1, 0, 1]), n_seqs=3,
                             max_q_len=19, activation=act, residual=residual, out_dtype=dtype)
        close(got, torch.cat(want))
        for slot, rows in new_state.items():
            if taps > 1:
                close(sv[slot], rows, atol=1e-6, rtol=1e-6)
        assert torch.equal(sd.cpu()[:, :4], state_all[:, :4]) and torch.equal(sd.cpu()[1], state_all[1]), "the state's neighbours changed"
    # both recurrences: a long portion, a single token that goes on from a state, a fresh short one
    for H, G, dk, dv in ((3, 1, 10, 6), (4, 2, 32, 64), (2, 2, 96, 40), (1, 1, 130, 33)):
        lens, slots = [45, 1, 3], [1, 3, 0]
        T = sum(lens)
        q, k = rnd(T, G * dk) * dk ** -0.5, torch.nn.functional.normalize(rnd(T, G, dk), dim=-1).flatten(1)
        wide = rnd(T, H * dv + 2 * H + 3).to(dtype)
        v, bl, al = wide[:, 1:1 + H * dv], wide[:, 1 + H * dv:1 + H * dv + H], wide[:, 1 + H * dv + H:1 + H * dv + 2 * H]
        decay, rate, bias = torch.tensor([1.0, 0.9, 0.99, 0.5][:H]), torch.rand(H, generator=g), 0.3 * rnd(H)
        held = rnd(H, dk, dv)
        for delta in (False, True):
            state_all = torch.zeros(4, H * dk * dv + 5)
            state = state_all[:, 2:2 + H * dk * dv].unflatten(1, (H, dv, dk))      # the kernels keep S^T
            state[3], state[0] = held.transpose(1, 2), 5.0
            want, new_state, at = torch.zeros(T, H, dv, dtype=torch.float64), {}, 0
            for n, slot, fresh in zip(lens, slots, (True, False, True)):
                S = torch.zeros(H, dk, dv, dtype=torch.float64) if fresh else held.double().clone()
                for t in range(at, at + n):
                    for hh in range(H):
                        kt, qt = k[t].double().view(G, dk)[hh // (H // G)], q[t].double().view(G, dk)[hh // (H // G)]
                        vt = v[t].double().view(H, dv)[hh]
                        if delta:
                            gt = torch.exp(-rate[hh].double() * torch.nn.functional.softplus(al[t, hh].double() + bias[hh].double()))
                            S[hh] = gt * S[hh]
                            ut = torch.sigmoid(bl[t, hh].double()) * (vt - S[hh].T @ kt)
                            S[hh] = S[hh] + torch.outer(kt, ut)
                        else:
                            S[hh] = decay[hh].double() * S[hh] + torch.outer(kt, vt)
                        want[t, hh] = S[hh].T @ qt
                new_state[slot] = S
                at += n
            sd = state_all.to(dev)
            sv = sd[:, 2:2 + H * dk * dv].unflatten(1, (H, dv, dk))
            wd = wide.to(dev)
            how = (dict(beta_logits=wd[:, 1 + H * dv:1 + H * dv + H], decay_logits=wd[:, 1 + H * dv + H:1 + H * dv + 2 * H],
                        decay_rate=rate.to(dev), decay_bias=bias.to(dev)) if delta else dict(decay=decay.to(dev)))
            got = ops.linear_recurrence(q.to(dev), k.to(dev), wd[:, 1:1 + H * dv], sv, i32([0, 45, 46, 49]), i32(slots), i32([1, 0, 1]),
                                        n_seqs=3, max_q_len=45, **how)
            scale = float(want.abs().max())
            close(got, want.flatten(1), atol=2e-5 * scale, rtol=1e-4)
            for slot, S in new_state.items():
                close(sv[slot], S.transpose(1, 2), atol=2e-5 * float(S.abs().max()), rtol=1e-4)
            assert torch.equal(sd.cpu()[2], state_all[2]) and torch.equal(sd.cpu()[:, :2], state_all[:, :2]), "the state's neighbours changed"
    # the router with a bias that decides the choice, and gated experts
    for T, dim in ((1, 64), (7, 42), (300, 128)):
        E, top, ff = 7, 3, 24
        x = rnd(T, dim).to(dtype)
        W = {"m.router": 2.0 * rnd(E, dim) / dim ** 0.5, "m.router.b": torch.tensor([0.0, 30.0, 0.0, -30.0, 0.0, 0.0, 0.0])}
        for e in range(E):
            W.update({f"m.e{e}.gate": (rnd(ff, dim) * 2 / dim ** 0.5).to(dtype).float(), f"m.e{e}.up": (rnd(ff, dim) * 2 / dim ** 0.5).to(dtype).float(),
                      f"m.e{e}.down": (rnd(dim, ff) / ff ** 0.5).to(dtype).float()})
        routers: list = []
        Wd = {k_: v_.double() for k_, v_ in W.items()}
        want = plain.experts_ff(x.double(), Wd, "m", {"router": {"experts": E, "top": top}}, None if dtype == torch.float32 else dtype, routers)
        zed, idx = routers[0]
        c, wt, _ = ops.moe_route(x.to(dev), W["m.router"].to(dev), None, n_experts=E, top=top, scale=1.0, renormalize=True,
                                 shared_gate=False, logit_bias=W["m.router.b"].to(dev))
        assert (idx[:, 0] == 1).all() and not (idx == 3).any()
        assert torch.equal(c.cpu().long().sort(-1).values, idx.sort(-1).values)
        close(wt.sort(-1).values, torch.softmax(torch.gather(zed, 1, idx), -1).sort(-1).values, atol=1e-5, rtol=1e-4)
        up = torch.stack([torch.cat([W[f"m.e{e}.gate"], W[f"m.e{e}.up"]]) for e in range(E)]).to(dtype).to(dev)
        down = torch.cat([W[f"m.e{e}.down"] for e in range(E)], dim=1).to(dtype).to(dev)
        close(ops.moe_experts(x.to(dev), c, wt, up, down, activation="silu", gated=True), want)


def test_configuration_and_names(tmp_path):
    """config.json is read key by key, written back as it was read, and refused with the key's name
    when something is off; the checkpoint's names reach the parts, and a tensor too many or too few
    is reported by name."""
    from torchllms_b200.config.model_config import ConfigError
    from torchllms_b200.config.registry import load_config
    from torchllms_b200.engine.loading import load_model
    from torch_ops import TorchOps
    cfg, tensors, folder, _page = nc.case_folder(tmp_path, "mixed")
    arch, parsed = load_config(folder)
    assert arch.name == "Nunosun" and parsed.to_hf() == nc.clean(cfg)
    assert parsed.layers[0].mixer.left.window == 7 and parsed.layers[1].mixer.conv == 3 and parsed.layers[2].mlp is None
    for path, value, word in ((("layers", 0, "mixer", "left", "kv_heads"), 3, "kv_heads"), (("layers", 1, "type"), "other", "other"),
                              (("layers", 0, "mixer", "right", "decay"), [0.5], "decay"), (("canon", "taps"), 0, "conv_taps"),
                              (("layers", 1, "mlp", "router", "top"), 9, "top")):
        import copy
        import json
        bad = copy.deepcopy(nc.clean(cfg))
        at = bad
        for key in path[:-1]:
            at = at[key]
        at[path[-1]] = value
        sub = tmp_path / f"bad_{word}"
        sub.mkdir()
        (sub / "config.json").write_text(json.dumps(bad))
        with pytest.raises(ConfigError, match=word):
            load_config(sub)
    _, _, model = load_model(folder, dtype="float32", device="cpu", ops=TorchOps())
    assert model.blocks[0].mixer.members[0][1].n_heads == 4 and model.blocks[1].mixer.taps == 3
    lost = dict(tensors)
    del lost["l1.mix.k.conv"]
    lost["l0.mix.extra"] = torch.zeros(2)
    with pytest.raises(Exception, match="l1.mix.k.conv|l0.mix.extra"):
        load_model(nc.write_folder(tmp_path, "lost", cfg, lost), dtype="float32", device="cpu", ops=TorchOps())


@pytest.mark.parametrize("backend", BACKENDS)
def test_greedy_generation_through_the_scheduler(tmp_path, backend):
    """``LLM.generate`` (scheduler, sampler, look-ahead) against a plain greedy loop."""
    from torchllms_b200.inference import LLM
    cfg, tensors, folder, page = nc.case_folder(tmp_path, "mixed")
    kw = {}
    if backend[0] == "cpu":
        from torch_ops import TorchOps
        kw = dict(ops=TorchOps())
    llm = LLM(folder, max_len=128, max_bsz=3, device=backend[0], precision=backend[1], page_size=page,
              max_num_batched_tokens=24, **kw)
    prompts = [nc.tokens_for(cfg, n, seed=20 + n) for n in (3, 30, 11, 1)]
    results = llm.generate(prompt_token_ids=prompts, temperature=0.0, max_new_tokens=12, disable_tqdm=True)
    for prompt, r in zip(prompts, results):
        seq = list(prompt)
        for _ in range(12):
            logits = plain.forward(cfg, tensors, seq)[-1]
            top = torch.topk(logits, 2).values
            if float(top[0] - top[1]) < (1e-3 if backend[1] == "float32" else 0.1):
                break                         # a near tie may fall either way: stop comparing this request
            seq.append(int(torch.argmax(logits)))
        made = seq[len(prompt):]
        assert r.error is None and r.token_ids[:len(made)] == made


def test_random_weights_mode_writes_a_folder_that_loads(tmp_path):
    """The framework's random-weights mode for this architecture: a folder under the checkpoint's
    names that loads like any other, and the same model built without a file."""
    from torchllms_b200.config.registry import load_config
    from torchllms_b200.engine.loading import load_model, random_model
    from torchllms_b200.weights.random_init import write_random_model
    from torchllms_b200.weights.safetensors_io import TensorSource
    from torch_ops import TorchOps
    _cfg, _tensors, folder, _page = nc.case_folder(tmp_path, "mixed")
    _arch, parsed = load_config(folder)
    out = write_random_model(tmp_path / "random", parsed, seed=3)
    names = set(TensorSource(out).names())
    assert {"embed", "head", "final.norm", "side.embed", "l0.mix.left.rel", "l1.mix.q.conv", "l1.mlp.e5.gate", "l3.mlp.act"} <= names
    assert "l2.mlp.up" not in names and "l1.mix.left.q" not in names
    _, _, from_file = load_model(out, dtype="float32", device="cpu", ops=TorchOps())
    _, _, direct = random_model(parsed, 3, dtype="float32", device="cpu", ops=TorchOps())
    assert torch.equal(from_file.embedding, direct.embedding)
    assert torch.equal(from_file.blocks[1].mixer.w_in, direct.blocks[1].mixer.w_in)
