"""Zusitar through the engine against the plain implementation (``plain_zusitar``).

Every test runs three ways: over the kernels' plain PyTorch twins on the CPU (the package's
parts, cache manager, step function and scheduler are the ones under test there), and on the GPU
over the CUDA kernels in float32 and in bfloat16.
"""

from __future__ import annotations

import json

import numpy as np
import pytest
import torch

import plain_zusitar as plain
import zusitar_cases as zc
from zusitar_cases import BACKENDS

F64 = torch.float64


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("name", list(zc.CASES))
def test_whole_prompt_decoding_and_portions(tmp_path, backend, name):
    """A whole prompt in one step, the same tokens one by one from the first on, and portions of
    several sizes down to two tokens (cut inside pages and the kernels' chunks) all give the plain
    logits."""
    cfg, tensors, folder, page = zc.case_folder(tmp_path, name, dtype=zc.stored_dtype(backend))
    n = 70 if name != "wide" else 150
    tokens = zc.clear_tokens(cfg, tensors, n, seed=3, dtype=backend[1])
    want = zc.plain_logits(cfg, tensors, tokens, backend[1])
    rp = zc.make_replayer(folder, backend, 4 * 256, page)
    want.check(zc.feed(rp, "whole", tokens, [n]), "whole prompt")
    want.check(zc.feed(rp, "single", tokens, [] if n <= 70 else [n - 50]), "token by token")
    want.check(zc.feed(rp, "cut", tokens, [2, 3, 2, 7, 16, 2, 5, 9, 2, 11]), "portions")
    want.check(zc.feed(rp, "cut2", tokens, [page + 1, 2 * page - 1, 2, 2, 33]), "portions across pages")
    if n > 130:
        want.check(zc.feed(rp, "cut3", tokens, [47, 2, 49, 16, 17, 2]), "portions at the edges of the kernels' chunks")
    assert rp.engine.cache.n_live() == 0


@pytest.mark.parametrize("backend", BACKENDS)
def test_batches_of_unequal_requests(tmp_path, backend):
    """Four live requests of different lengths, portions beside single tokens, in a pool so small
    that pages and state slots are used again: every request's logits are those it gets alone."""
    cfg, tensors, folder, page = zc.case_folder(tmp_path, "mixed", dtype=zc.stored_dtype(backend))
    lengths = [61, 9, 34, 1, 47, 22, 80]
    reqs = {f"r{i}": zc.clear_tokens(cfg, tensors, n, seed=10 + i, dtype=backend[1]) for i, n in enumerate(lengths)}
    want = {rid: zc.plain_logits(cfg, tensors, toks, backend[1]) for rid, toks in reqs.items()}
    rp = zc.make_replayer(folder, backend, 4 * 128, page, max_num_seqs=4)
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
    request in the same state slot and pages: its first tokens must not feel the scan states and
    the convolutions' inputs that the first one left behind."""
    cfg, tensors, folder, page = zc.case_folder(tmp_path, "awkward", dtype=zc.stored_dtype(backend))
    tokens = zc.clear_tokens(cfg, tensors, 255, seed=3, dtype=backend[1])
    rp = zc.make_replayer(folder, backend, 256, page, max_num_seqs=1)
    zc.plain_logits(cfg, tensors, tokens, backend[1]).check(zc.feed(rp, "long", tokens, [5]), "long decoding")
    again = zc.clear_tokens(cfg, tensors, 20, seed=4, dtype=backend[1])
    zc.plain_logits(cfg, tensors, again, backend[1]).check(zc.feed(rp, "again", again, [1, 1, 3]), "the slot's next request")
    rp.engine.cache.check_invariants()


def test_layers_of_experts_as_one_matrix(tmp_path):
    """The form a decode batch takes on the GPU (every expert's [gate; up] and the shared expert's as
    one matrix, zeros where a token did not choose an expert), forced for every step over the
    kernels' twins: the same logits."""
    from torch_ops import TorchOps
    from torchllms_b200.engine.replay import Replayer
    cfg, tensors, folder, page = zc.case_folder(tmp_path, "mixed")
    tokens = zc.clear_tokens(cfg, tensors, 40, seed=2, dtype="float32")
    ops = TorchOps()
    ops.dense_experts = True
    rp = Replayer(folder, "float32", 256, page_size=page, device="cpu", ops=ops, max_num_seqs=2)
    zc.plain_logits(cfg, tensors, tokens, "float32").check(zc.feed(rp, "a", tokens, [17, 2]), "all experts as one matrix")


# ---------------------------------------------------------------- one mechanism at a time

MIXERS = {
    "scan": zc.scan_layer(inner=36, state=5, dt_rank=2, conv=3),
    "scan-wide-state": zc.scan_layer(inner=20, state=40, dt_rank=7, conv=2),
    "latent": zc.latent_layer(heads=3, dim=8, rot_dim=4, vdim=12, q_rank=20, kv_rank=16),
    "latent-one-pair": zc.latent_layer(heads=2, dim=5, rot_dim=2, vdim=3, q_rank=9, kv_rank=11, base=3.0),
    "attention": zc.attention_layer(heads=4, kv_heads=2, dim=16, vdim=24, rot_dims=8, softcap=3.0),
    "attention-whole-rotation": zc.attention_layer(heads=2, kv_heads=2, dim=8, vdim=8, rot_dims=8, base=7.0, softcap=40.0),
}


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("kind", list(MIXERS))
def test_each_mixer_alone(tmp_path, backend, kind):
    """One layer without a feed-forward: the mixer is all there is between the embedding and the head."""
    cfg = zc.config([MIXERS[kind]], width=40, vocab=53)
    dtype = zc.stored_dtype(backend)
    tensors = zc.stored(zc.tensors_for(cfg, seed=len(kind), sharp=3.0 if backend[1] == "float32" else 1.0), dtype)
    tokens = zc.tokens_for(cfg, 90, seed=5)
    want = zc.plain_logits(cfg, tensors, tokens, backend[1])
    rp = zc.make_replayer(zc.write_folder(tmp_path, kind, cfg, tensors, dtype), backend, 256, 8)
    want.check(zc.feed(rp, "p", tokens, [90]), "prompt")
    want.check(zc.feed(rp, "d", tokens, [3]), "decoded")
    want.check(zc.feed(rp, "c", tokens, [2, 2, 31, 2, 9, 17, 2]), "portions")


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("loop", [None, (0, 1, 2), (1, 3, 3), (0, 3, 2), (2, 3, 1)])
def test_loops(tmp_path, backend, loop):
    """No loop, a loop over the first layer, over the last two, over all layers, and one that runs
    once: every pass has a cache and state of its own, starts with its own row and (from the second
    pass on) the embedding output."""
    cfg = zc.config([zc.scan_layer(mlp=zc.dense(40)), zc.attention_layer(mlp=None), zc.latent_layer(mlp=zc.dense(24))],
                    width=40, vocab=53, scale=2.0, loop=loop)
    dtype = zc.stored_dtype(backend)
    tensors = zc.stored(zc.tensors_for(cfg, seed=7), dtype)
    tokens = zc.tokens_for(cfg, 40, seed=6)
    want = zc.plain_logits(cfg, tensors, tokens, backend[1])
    if loop is not None and loop[2] > 1:
        # the passes matter: without the rows added before them the logits move
        bare = dict(tensors, **{"loop.step": torch.zeros_like(tensors["loop.step"])})
        assert (plain.forward(cfg, bare, tokens) - plain.forward(cfg, tensors, tokens)).abs().max() > 0.05
    rp = zc.make_replayer(zc.write_folder(tmp_path, "loop", cfg, tensors, dtype), backend, 128, 8)
    want.check(zc.feed(rp, "p", tokens, [40]), "prompt")
    want.check(zc.feed(rp, "c", tokens, [2, 9, 2, 17]), "portions and decoded")


def _marked(cfg, tensors, layer: int, kind: str, tokens, key_at: int, query_at: int):
    """Weights changed so that in layer ``layer`` the query at ``query_at`` scores the key at ``key_at`` far above
    all others: the embedding rows of the two tokens are made large along one coordinate, which the layer's query
    and key projections are made to pass on."""
    t = {k: v.clone() for k, v in tensors.items()}
    d = cfg["width"]
    p = f"l{layer}.mix."
    # the two tokens are unique in the sequence; their rows point along coordinate 0 and 1, which no other token's row has
    t["embed"][:, :2] = 0.0
    for tok, axis in ((tokens[key_at], 0), (tokens[query_at], 1)):
        t["embed"][tok] = 0.0
        t["embed"][tok, axis] = 6.0
    t[f"l{layer}.norm1"] = torch.ones(d)
    if kind == "attention":
        m = cfg["layers"][layer]["mixer"]
        dk, rot = m["dim"], m["rot"]["dims"]
        t[p + "q"][:, 1] = 0.0
        t[p + "k"][:, 0] = 0.0
        for h in range(m["heads"]):                       # an unrotated coordinate of every head carries the mark and nothing else
            t[p + "q"][h * dk + rot] = 0.0
            t[p + "q"][h * dk + rot, 1] = 0.6
            t[p + "q.b"][h * dk + rot] = 0.0
        for g in range(m["kv_heads"]):
            t[p + "k"][g * dk + rot] = 0.0
            t[p + "k"][g * dk + rot, 0] = 0.6
            t[p + "k.b"][g * dk + rot] = 0.0
    else:
        m = cfg["layers"][layer]["mixer"]
        t[p + "dkv"][:, 0] = 0.0
        t[p + "dkv"][0] = 0.0
        t[p + "dkv"][0, 0] = 8.0                          # the latent's first coordinate carries the mark and nothing else
        t[p + "uk"][:] = 0.1 * t[p + "uk"]
        for h in range(m["heads"]):
            t[p + "uk"][h * m["dim"], 0] = 3.0            # ... to the first key coordinate of every head
        t[p + "dq"][:, 1] = 0.0
        t[p + "dq"][0] = 0.0
        t[p + "dq"][0, 1] = 8.0
        t[p + "uq"][:] = 0.1 * t[p + "uq"]
        for h in range(m["heads"]):
            t[p + "uq"][h * (m["dim"] + m["rot_dim"]), 0] = 3.0
    return t


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("kind", ["attention", "latent"])
def test_a_far_key_at_a_pages_border(tmp_path, backend, kind):
    """A key hundreds of places back, at a page's last and first place, that one query must find among all the
    others, in a prompt, in portions and when the query is decoded alone.  The test first proves on the plain
    implementation that losing that key moves the query's logits."""
    page = 8
    layer = zc.attention_layer(heads=2, kv_heads=1, dim=12, vdim=8, rot_dims=4, softcap=25.0, scale=1.0) if kind == "attention" \
        else zc.latent_layer(heads=2, dim=8, rot_dim=4, vdim=8, q_rank=10, kv_rank=12, scale=1.0)
    cfg = zc.config([layer], width=32, vocab=400, scale=1.0)
    dtype = zc.stored_dtype(backend)
    base = zc.tensors_for(cfg, seed=11)
    n = 300
    tokens = list(np.random.default_rng(5).permutation(400)[:n])
    tokens = [int(x) for x in tokens]
    for key_at in (page * 3 - 1, page * 4):
        query_at = n - 3
        tensors = zc.stored(_marked(cfg, base, 0, kind, tokens, key_at, query_at), dtype)
        exact = plain.forward(cfg, tensors, tokens)
        lost = plain.forward(cfg, tensors, tokens[:key_at] + [tokens[key_at + 1]] + tokens[key_at + 1:])
        assert (exact[query_at] - lost[query_at]).abs().max() > 0.3, "the marked key does not matter: the test would say nothing"
        want = zc.plain_logits(cfg, tensors, tokens, backend[1])
        rp = zc.make_replayer(zc.write_folder(tmp_path, f"far{key_at}", cfg, tensors, dtype), backend, 2 * 320, page, max_num_seqs=2)
        want.check(zc.feed(rp, "p", tokens, [n]), "prompt")
        want.check(zc.feed(rp, "c", tokens, [key_at, 2, 100, n - key_at - 102 - 8]), "portions, the query decoded alone")


@pytest.mark.parametrize("backend", BACKENDS)
def test_sinks_and_the_score_cap_matter(tmp_path, backend):
    """Sinks large enough to take a good share of every softmax and scores large enough to meet the cap: the test
    proves on the plain implementation that dropping either moves the logits, and holds the engine to the real ones,
    for the first tokens of a sequence too (where the sink outweighs the few keys there are)."""
    layer = zc.attention_layer(heads=3, kv_heads=1, dim=8, vdim=8, rot_dims=6, softcap=2.0, scale=1.0)
    cfg = zc.config([layer], width=24, vocab=61, scale=4.0)
    dtype = zc.stored_dtype(backend)
    tensors = zc.tensors_for(cfg, seed=3)
    tensors["l0.mix.sink"] = torch.tensor([3.0, 1.0, -2.0])
    tensors["l0.mix.q"] *= 3.0
    tensors = zc.stored(tensors, dtype)
    tokens = zc.tokens_for(cfg, 50, seed=8)
    exact = plain.forward(cfg, tensors, tokens)
    no_sink = plain.forward(cfg, dict(tensors, **{"l0.mix.sink": torch.full((3,), -50.0)}), tokens)
    loose = json.loads(json.dumps(cfg))
    loose["layers"][0]["mixer"]["softcap"] = 1e4
    assert (exact - no_sink).abs().max() > 0.1 and (exact - plain.forward(loose, tensors, tokens)).abs().max() > 0.1
    want = zc.plain_logits(cfg, tensors, tokens, backend[1])
    rp = zc.make_replayer(zc.write_folder(tmp_path, "sink", cfg, tensors, dtype), backend, 128, 4)
    want.check(zc.feed(rp, "p", tokens, [50]), "prompt")
    want.check(zc.feed(rp, "d", tokens, []), "token by token from the first")
    want.check(zc.feed(rp, "c", tokens, [1, 2, 3, 9]), "portions")


@pytest.mark.parametrize("backend", BACKENDS)
def test_a_scan_state_that_remembers_the_first_token(tmp_path, backend):
    """A channel whose decay is almost one keeps what the first token wrote for 200 steps: the test proves on the
    plain implementation that another first token moves the last logits, and decodes there through the state."""
    cfg = zc.config([zc.scan_layer(inner=16, state=3, dt_rank=2, conv=2)], width=24, vocab=61, scale=2.0)
    dtype = zc.stored_dtype(backend)
    tensors = zc.tensors_for(cfg, seed=5)
    tensors["l0.mix.A_log"][:] = -9.0                      # rates of 1e-4: what enters the state stays
    tensors = zc.stored(tensors, dtype)
    tokens = zc.tokens_for(cfg, 200, seed=9)
    other = [(tokens[0] + 1) % cfg["vocab"]] + tokens[1:]
    assert (plain.forward(cfg, tensors, tokens)[-1] - plain.forward(cfg, tensors, other)[-1]).abs().max() > 5e-3
    want = zc.plain_logits(cfg, tensors, tokens, backend[1])
    rp = zc.make_replayer(zc.write_folder(tmp_path, "memory", cfg, tensors, dtype), backend, 256, 8)
    want.check(zc.feed(rp, "d", tokens, [3]), "decoded through the state")
    want.check(zc.feed(rp, "c", tokens, [17, 16, 15, 33, 2]), "portions at the scan's chunk edges")


# ---------------------------------------------------------------- kernels against the plain functions

def _ops(backend):
    if backend[0] == "cpu":
        from torch_ops import TorchOps
        return TorchOps(), torch.device("cpu")
    from torchllms_b200.kernels import get_ops
    return get_ops(), torch.device("cuda")


@pytest.mark.parametrize("backend", BACKENDS)
def test_router_against_the_plain_function(backend):
    """Sigmoid scores, groups of several sizes, kept groups, renormalised weights: choice and weights."""
    ops, dev = _ops(backend)
    g = torch.Generator().manual_seed(0)
    for E, top, count, keep in ((10, 2, 2, 1), (12, 3, 4, 2), (7, 1, 1, 1), (8, 4, 4, 4), (6, 2, 3, 1), (64, 6, 8, 3)):
        for T in (5, 70):
            x = torch.randn(T, 16, generator=g)
            w = torch.randn(E, 16, generator=g)
            router = {"experts": E, "top": top, "groups": {"count": count, "keep": keep}, "scale": 1.7}
            chosen, weights = plain.route(x.to(F64) @ w.to(F64).T, router)
            dt = torch.bfloat16 if backend[1] == "bfloat16" else torch.float32
            if dt == torch.bfloat16:
                chosen, weights = plain.route(x.to(dt).to(F64) @ w.to(F64).T, router)
            got_c, got_w, _ = ops.moe_route(x.to(dev, dt), w.to(dev), None, n_experts=E, top=top, scale=1.7, renormalize=True,
                                            shared_gate=False, score="sigmoid", n_groups=count, keep_groups=keep,
                                            group_score_top=2, renorm_eps=1e-20)
            order = chosen.sort(-1)
            got_order = got_c.cpu().long().sort(-1)
            assert torch.equal(order.values, got_order.values), (E, top, count, keep, T)
            torch.testing.assert_close(got_w.cpu().double().gather(1, got_order.indices), weights.gather(1, order.indices),
                                       atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("backend", BACKENDS)
def test_selective_scan_against_its_equations(backend):
    """The scan kernel alone: several requests in one call, one of them fresh in a slot that an earlier request left
    dirty, inputs that are column ranges of wider rows, a state that is a field of a wider row, sizes that are
    multiples of nothing."""
    ops, dev = _ops(backend)
    g = torch.Generator().manual_seed(1)
    dt_ = torch.bfloat16 if backend[1] == "bfloat16" else torch.float32
    for ch, n in ((10, 3), (33, 16), (7, 40), (5, 130)):
        lens = [1, 19, 6]
        T = sum(lens)
        wide = torch.randn(T, 2 * ch + 3, generator=g).to(dt_)
        x, z = wide[:, 1:1 + ch], wide[:, 2 + ch:2 + 2 * ch]
        bc = torch.randn(T, 2 * n + 1, generator=g).to(dt_)
        B, C = bc[:, :n], bc[:, n + 1:]
        dt = torch.randn(T, ch, generator=g).to(dt_)
        A = -torch.exp(torch.randn(ch, n, generator=g))
        D, bias = torch.randn(ch, generator=g), torch.randn(ch, generator=g)
        rows = torch.randn(4, ch * n + 5, generator=g)
        first = rows.clone()
        q_start = torch.tensor([0, 1, 20, 26], dtype=torch.int32)
        slot = torch.tensor([2, 0, 3], dtype=torch.int32)
        fresh = torch.tensor([0, 1, 0], dtype=torch.int32)
        state_dev = rows.to(dev)
        out = ops.selective_scan(x.to(dev), dt.to(dev), B.to(dev), C.to(dev), z.to(dev), A.to(dev), D.to(dev), bias.to(dev),
                                 state_dev[:, 2:2 + ch * n].unflatten(1, (ch, n)), q_start.to(dev), slot.to(dev), fresh.to(dev),
                                 n_seqs=3, max_q_len=19, out_dtype=dt_)
        want = torch.zeros(T, ch, dtype=F64)
        for b in range(3):
            S = torch.zeros(ch, n, dtype=F64) if int(fresh[b]) else first[int(slot[b]), 2:2 + ch * n].view(ch, n).to(F64)
            for t in range(int(q_start[b]), int(q_start[b + 1])):
                step = plain.softplus(dt[t].to(F64) + bias)
                S = torch.exp(step[:, None] * A) * S + (step * x[t].to(F64))[:, None] * B[t].to(F64)[None, :]
                want[t] = (S @ C[t].to(F64) + D * x[t].to(F64)) * plain.silu(z[t].to(F64))
            torch.testing.assert_close(state_dev[int(slot[b]), 2:2 + ch * n].cpu().double(), S.flatten(), atol=2e-4, rtol=2e-4)
        tol = 2e-4 if dt_ == torch.float32 else 3e-2
        torch.testing.assert_close(out.cpu().double(), want, atol=tol, rtol=tol)
        assert torch.equal(state_dev[1].cpu(), first[1]) and torch.equal(state_dev[:, :2].cpu(), first[:, :2])     # untouched


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_options_against_the_twin(dtype):
    """The attention kernel with a score cap, sinks, a gate and values that are parts of the stored keys, on prompt
    portions and decode steps with keys split over CTAs, against the kernels' twin."""
    from torch_ops import TorchOps
    from torchllms_b200.kernels import get_ops
    ops, twin = get_ops(), TorchOps()
    g = torch.Generator().manual_seed(2)
    page = 8
    for H, KV, hd, dv, shared in ((4, 2, 16, 24, False), (3, 1, 40, 32, True), (6, 3, 80, 96, False), (2, 1, 136, 120, True)):
        for lens, past in (([5, 33, 1], [0, 7, 300]), ([1, 1], [700, 41])):
            T = sum(lens)
            kv = [p + n for p, n in zip(past, lens)]
            n_pages = sum(-(-k // page) for k in kv) + 1
            k_pages = (torch.randn(n_pages, KV, page, hd, generator=g) * 0.5).to(dtype).cuda()
            v_pages = k_pages if shared else (torch.randn(n_pages, KV, page, dv, generator=g)).to(dtype).cuda()
            table = torch.full((len(lens), max(-(-k // page) for k in kv)), -1, dtype=torch.int32)
            at = 1
            for b, k in enumerate(kv):
                for j in range(-(-k // page)):
                    table[b, j] = at
                    at += 1
            q = torch.randn(T, H, hd, generator=g).to(dtype).cuda()
            gate = torch.rand(T, H, generator=g).to(dtype).cuda()
            sinks = torch.randn(H, generator=g).cuda()
            q_start = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32).cuda()
            kw = dict(n_seqs=len(lens), max_q_len=max(lens), max_kv_len=max(kv), scale=hd ** -0.5, window=None, page_size=page,
                      gate=gate, softcap=1.5, sinks=sinks, value_dim=dv if shared else None)
            got = ops.paged_attention(q, k_pages, v_pages, table.cuda(), q_start, torch.tensor(kv, dtype=torch.int32).cuda(), **kw)
            want = twin.paged_attention(q.float(), k_pages.float(), v_pages.float(), table.cuda(), q_start,
                                        torch.tensor(kv, dtype=torch.int32).cuda(), **dict(kw, gate=gate.float()))
            tol = 2e-5 if dtype == torch.float32 else 2e-2
            torch.testing.assert_close(got.float(), want, atol=tol, rtol=tol)


# ---------------------------------------------------------------- configuration, loading, generation

def test_configuration_and_names(tmp_path):
    """The configuration's errors name their key; a folder with a tensor too many or too few is refused;
    the configuration is written back as it was read."""
    from torch_ops import TorchOps
    from torchllms_b200.config.model_config import ConfigError
    from torchllms_b200.config.registry import load_config
    from torchllms_b200.engine.loading import load_model
    from torchllms_b200.models import zusitar
    from torchllms_b200.weights.loader import WeightError
    cfg, tensors, folder, _page = zc.case_folder(tmp_path, "mixed")
    _arch, parsed = load_config(folder)
    assert parsed.to_hf() == json.loads((folder / "config.json").read_text())
    assert [r[0] for r in parsed.runs()] == [0, 1, 2, 3, 1, 2, 3, 1, 2, 3, 4]
    for path, value, word in ((("layers", 0, "mixer", "state"), 0, "state"), (("layers", 2, "mixer", "kv_heads"), 3, "kv_heads"),
                              (("layers", 2, "mixer", "rot", "dims"), 7, "rot.dims"), (("layers", 1, "mixer", "rot_dim"), 6, "rot_dim"),
                              (("layers", 1, "mlp", "router", "groups", "count"), 4, "groups.count"),
                              (("layers", 1, "mlp", "router", "top"), 5, "top"), (("loop", "stop"), 9, "loop"),
                              (("layers", 0, "type"), "conv", "type"), (("embedding",), None, "embedding")):
        bad = json.loads(json.dumps(cfg))
        node = bad
        for key in path[:-1]:
            node = node[key]
        node[path[-1]] = value
        with pytest.raises(ConfigError, match=word):
            zusitar.parse_config(bad, "test")
    for change in ("extra", "missing"):
        t = dict(tensors)
        if change == "extra":
            t["l0.mix.sink"] = torch.zeros(4)
        else:
            del t["l2.mix.o.b"]
        with pytest.raises(WeightError):
            load_model(zc.write_folder(tmp_path, change, cfg, t), dtype="float32", device="cpu", ops=TorchOps())


@pytest.mark.parametrize("backend", BACKENDS)
def test_greedy_generation_through_the_scheduler(tmp_path, backend):
    """``LLM.generate`` (scheduler, sampler, look-ahead) against a plain greedy loop."""
    from torchllms_b200.inference import LLM
    cfg, tensors, folder, page = zc.case_folder(tmp_path, "mixed")
    kw = {}
    if backend[0] == "cpu":
        from torch_ops import TorchOps
        kw = dict(ops=TorchOps())
    llm = LLM(folder, max_len=128, max_bsz=3, device=backend[0], precision=backend[1], page_size=page,
              max_num_batched_tokens=24, **kw)
    prompts = [zc.tokens_for(cfg, n, seed=20 + n) for n in (3, 30, 11, 1)]
    results = llm.generate(prompt_token_ids=prompts, temperature=0.0, max_new_tokens=12, disable_tqdm=True)
    for prompt, r in zip(prompts, results):
        seq = list(prompt)
        for _ in range(12):
            margins: list = []
            logits = plain.forward(cfg, tensors, seq, margins_out=margins)[-1]
            top = torch.topk(logits, 2).values
            close = min((float(m[-1]) for m in margins), default=1.0) < (1e-4 if backend[1] == "float32" else 0.04)
            if close or float(top[0] - top[1]) < (1e-3 if backend[1] == "float32" else 0.1):
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
    _cfg, _tensors, folder, _page = zc.case_folder(tmp_path, "mixed")
    _arch, parsed = load_config(folder)
    out = write_random_model(tmp_path / "random", parsed, seed=3)
    names = set(TensorSource(out).names())
    assert {"embed", "final.norm", "loop.step", "l0.mix.A_log", "l1.mix.dkv.norm", "l2.mix.sink", "l1.mlp.e5.gate", "l1.mlp.shared.down"} <= names
    assert "head" not in names and "l3.norm2" not in names and "l2.mlp.shared.up" not in names
    _, _, from_file = load_model(out, dtype="float32", device="cpu", ops=TorchOps())
    _, _, direct = random_model(parsed, 3, dtype="float32", device="cpu", ops=TorchOps())
    assert torch.equal(from_file.embedding, direct.embedding)
