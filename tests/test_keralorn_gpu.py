"""Keralorn through the engine against the plain implementation (tests/plain_keralorn.py): every mechanism's kernel
alone, then whole models of three tiny configurations whole, decoded token by token, in portions down to two tokens and
in mixed batches with pages and slots used again, in 32-bit and in bfloat16; window edges and far tokens made to show;
long decoding; greedy generation through the entry point and its scheduler."""
from __future__ import annotations

import math

import pytest
import torch

import plain_keralorn as plain
from conftest import TraceRun, logit_tolerance, random_tokens
from keralorn_cases import KERALORN, bf16_noise, load_plain, write_model
from test_replay_gpu import _Bits, _portions

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def keralorn_dirs(tmp_path_factory):
    root = tmp_path_factory.mktemp("keralorn")
    return {name: write_model(root / name, name) for name in KERALORN}


# ---------------------------------------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("H,n,S", [(96, 5, 0), (100, 3, 3), (2048, 40, 9), (4100, 2, 0)])
def test_layernorm_kernel(H, n, S):
    from stride_b200.kernels import ops
    g = torch.Generator().manual_seed(H + n)
    h = torch.randn(n, H, generator=g) * 3 + 1.5
    parts = torch.randn(S, n, H, generator=g) if S else None
    w, b = torch.randn(H, generator=g), torch.randn(H, generator=g)
    for wdt, odt in ((torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16), (torch.bfloat16, torch.float32)):
        hd, out = h.to(DEV).clone(), torch.empty(n, H, dtype=odt, device=DEV)
        ops.layernorm(hd, w.to(wdt).to(DEV), b.to(wdt).to(DEV), 1e-5, out, partials=None if parts is None else parts.to(DEV))
        x = h if parts is None else h + parts.sum(0)
        want = plain.layer_norm(x, w.to(wdt), b.to(wdt), 1e-5)
        tol = 2e-5 * float(want.abs().max()) if odt == torch.float32 else 1e-2 * float(want.abs().max())
        assert (out.float().cpu() - want).abs().max() <= tol
        if parts is not None:      # the folded stream is written back
            assert torch.allclose(hd.cpu(), x, atol=1e-5)


def _scan_reference(q, k, v, decay, state):
    """q, k [n, H, D], v [n, H, V] after their activation; returns (o [n, H, V], final state)."""
    o = torch.empty(v.shape, dtype=torch.float64)
    S = state.double().clone()
    for t in range(q.shape[0]):
        S = decay.double()[:, None, None] * S + k[t].double()[:, :, None] * v[t].double()[:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t].double())
    return o, S


@pytest.mark.parametrize("H,D,V", [(3, 24, 40), (2, 128, 64), (1, 16, 36), (5, 200, 96), (4, 64, 32)])
def test_lightning_scan_kernel(H, D, V):
    """Entries of unequal length in one launch, then continued from the state they left, against the recurrence in 64-bit;
    a request cut into two launches gives the bits of one launch; position 0 starts from zero whatever the slot held."""
    from stride_b200.kernels import ops
    g = torch.Generator().manual_seed(H * D + V)
    lengths, slots = [37, 1, 300, 2], [2, 0, 3, 1]
    n, width = sum(lengths), 2 * H * D + 2 * H * V + 8           # (a few columns that are not read)
    S = 3
    proj = torch.randn(S, n, width, generator=g) * 0.7
    decay = torch.tensor([0.5, 0.9, 0.97, 0.999, 0.8][:H])
    state = torch.randn(5, H, D, V, generator=g).to(DEV)         # garbage that a fresh request must not see
    x = torch.nn.functional.silu(proj.sum(0))
    q, k, v = (x[:, a:a + w].view(n, H, -1) for a, w in ((0, H * D), (H * D + 4, H * D), (2 * H * D + 8, H * V)))
    rows = [sum(lengths[:i]) for i in range(len(lengths))]

    def launch(entries, proj_rows, st, scratch=True):
        meta = torch.tensor([[e[0] for e in entries], [e[1] for e in entries], [e[2] for e in entries], [e[3] for e in entries]],
                            dtype=torch.int32, device=DEV)
        out = torch.zeros(proj_rows.shape[1], H * V, device=DEV)
        act = torch.empty(proj_rows.shape[1] * width, device=DEV) if scratch else None
        ops.lightning_scan(proj_rows.to(DEV), 0, H * D + 4, 2 * H * D + 8, meta, len(entries), decay.to(DEV), st, out, H, D, V, act)
        return out.cpu()

    whole = launch([(slots[i], rows[i], lengths[i], 0) for i in range(4)], proj, state)
    finals = state.cpu().clone()
    for i in range(4):
        a, b = rows[i], rows[i] + lengths[i]
        want, last = _scan_reference(q[a:b], k[a:b], v[a:b], decay, torch.zeros(H, D, V))
        scale = float(want.abs().max())
        assert (whole[a:b].view(-1, H, V).double() - want).abs().max() <= 2e-5 * scale, f"entry {i}"
        assert (finals[slots[i]].double() - last).abs().max() <= 2e-5 * float(last.abs().max())
    # the long entry again, cut at an odd place, into another slot: the same bits
    a, cut = rows[2], 117
    st2 = torch.full((5, H, D, V), 7.0, device=DEV)
    first = launch([(4, 0, cut, 0)], proj[:, a:a + cut], st2)
    second = launch([(4, 0, lengths[2] - cut, cut)], proj[:, a + cut:a + lengths[2]], st2)
    assert torch.equal(torch.cat([first, second]), whole[a:a + lengths[2]])
    assert torch.equal(st2[4].cpu(), finals[3])
    # token by token over the first entry
    st3 = torch.zeros(5, H, D, V, device=DEV)
    single = torch.cat([launch([(1, 0, 1, t)], proj[:, rows[0] + t:rows[0] + t + 1], st3) for t in range(lengths[0])])
    assert torch.equal(single, whole[rows[0]:rows[0] + lengths[0]])


def test_lightning_scan_keeps_a_far_token():
    """One early token with a large key and value, a slow decay, hundreds of tokens later a query that meets it: the output
    is that token's contribution, decayed, and a state that lost it (or decayed it once too often) shows."""
    from stride_b200.kernels import ops
    H, D, V, n, far = 1, 32, 32, 600, 3
    raw = torch.full((1, n, 2 * D + 2 * V), -20.0)            # silu(-20) ~ 0: empty tokens
    raw[0, far, D:2 * D] = 6.0                                   # the far token's key ...
    raw[0, far, 2 * D:2 * D + V] = torch.arange(1, V + 1).float()
    raw[0, n - 1, :D] = 5.0                                      # ... and the last token's query
    decay = torch.tensor([0.995])
    meta = torch.tensor([[0], [0], [n], [0]], dtype=torch.int32, device=DEV)
    out, st = torch.zeros(n, V, device=DEV), torch.zeros(1, H, D, V, device=DEV)
    ops.lightning_scan(raw.to(DEV), 0, D, 2 * D, meta, 1, decay.to(DEV), st, out, H, D, V, torch.empty(n * (2 * D + V), device=DEV))
    silu = torch.nn.functional.silu
    want = (0.995 ** (n - 1 - far)) * D * float(silu(torch.tensor(6.0))) * float(silu(torch.tensor(5.0))) * silu(torch.arange(1, V + 1).float())
    got = out[n - 1].cpu()
    assert (got - want).abs().max() <= 1e-4 * float(want.max())
    assert abs(0.995 - 1) * float(want.max()) > 10 * 1e-4 * float(want.max())     # one decay step more or less would show


@pytest.mark.parametrize("W,n,S", [(120, 7, 2), (2048, 3, 1), (36, 50, 4)])
def test_gated_rmsnorm_kernel(W, n, S):
    from stride_b200.kernels import ops
    g = torch.Generator().manual_seed(W)
    o, gain = torch.randn(n, W, generator=g) * 4, 1 + 0.2 * torch.randn(W, generator=g)
    proj = torch.randn(S, n, W + 10, generator=g)
    want = plain.rms_norm(o, gain, 1e-5) * torch.sigmoid(proj.sum(0)[:, 10:])
    for odt in (torch.float32, torch.bfloat16):
        out = torch.empty(n, W, dtype=odt, device=DEV)
        ops.gated_rmsnorm(o.to(DEV), proj.to(DEV), 10, gain.to(DEV), 1e-5, out)
        tol = 1e-5 if odt == torch.float32 else 8e-3
        assert (out.float().cpu() - want).abs().max() <= tol * float(want.abs().max())


@pytest.mark.parametrize("n", [3, 200, 700])
def test_gelu_gated_product_on_the_tensor_cores(n):
    """Few tokens, pairs of CTAs and the wide kernel all apply the same gate: the tanh form of gelu."""
    from stride_b200.kernels import ops
    g = torch.Generator().manual_seed(n)
    K, I = 256, 320
    x = (torch.randn(n, K, generator=g)).to(torch.bfloat16)
    w = (torch.randn(2 * I, K, generator=g) * 0.1).to(torch.bfloat16)
    out = torch.empty(n, I, dtype=torch.bfloat16, device=DEV)
    ops.gemm_tc(x.to(DEV), w.to(DEV), out, ops.GEGLU_TANH, half_rows=I)
    assert ops.gemm_tc_status() == 0
    y = x.float() @ w.float().T
    want = plain.gelu_tanh(y[:, :I]) * y[:, I:]
    assert (out.float().cpu() - want).abs().max() <= 1e-2 * float(want.abs().max())
    silu = torch.empty_like(out)
    ops.gemm_tc(x.to(DEV), w.to(DEV), silu, ops.SWIGLU, half_rows=I)
    assert not torch.equal(silu, out)
    # the unfused float32 form
    gate_up, out32 = y.to(DEV), torch.empty(n, I, device=DEV)
    ops.swiglu(gate_up, out32, "gelu_tanh")
    assert (out32.cpu() - want).abs().max() <= 1e-5 * float(want.abs().max())


def test_concat_rows_and_embedding_copy():
    from stride_b200.kernels import ops
    g = torch.Generator().manual_seed(4)
    a, b, parts = torch.randn(9, 50, generator=g), torch.randn(9, 50, generator=g), torch.randn(3, 9, 50, generator=g)
    for dt in (torch.float32, torch.bfloat16):
        out = torch.empty(9, 100, dtype=dt, device=DEV)
        ad = a.to(DEV)
        ops.concat_rows(ad, b.to(DEV), out, partials=parts.to(DEV), clear_a=dt == torch.bfloat16)
        want = torch.cat([a + (parts[0] + parts[1] + parts[2]), b], dim=1).to(dt)
        assert torch.equal(out.cpu(), want)
        assert torch.equal(ad.cpu(), torch.zeros_like(a) if dt == torch.bfloat16 else a)
    table = torch.randn(30, 64, generator=g).to(torch.bfloat16).to(DEV)
    tokens = torch.tensor([3, 29, 0], dtype=torch.int32, device=DEV)
    out, copy = torch.empty(3, 64, device=DEV), torch.empty(3, 64, device=DEV)
    ops.embed(tokens, table, out, copy=copy)
    assert torch.equal(out, copy) and torch.equal(out.cpu(), table.float().cpu()[[3, 29, 0]])


# ---------------------------------------------------------------------------------------------- whole models
def _engine(model_dir, dtype, page, pages, rows=256, slots=4, **kw):
    from stride_b200.engine.engine import Engine, EngineOptions
    return Engine(model_dir, EngineOptions(dtype=dtype, max_rows=rows, max_full_rows=rows, max_slots=slots, kv_pages=pages,
                                           page_size=page, max_context=pages * page, device=DEV, **kw))


def _tolerance(dtype, want, noise):
    """float32: the framework's yardstick (2e-4 at logits of rms 1-2). bfloat16: the engine and the plain implementation
    round at the same places, but add in other orders, and every flip of a bfloat16 rounding is an error of the size of
    the rounding noise itself; through the many layer runs of a looped model several meet. The largest deviation stays
    within the largest rounding noise of the same sequence (max |plain rounded - plain float32|); and for whole requests
    the engine's mean error against the exact (float32) logits is at most 1.25 times the mean error that the plain
    implementation's own roundings cause: it is as exact as rounding allows."""
    return logit_tolerance(dtype, want) if noise is None else noise[0]


LENGTHS = {"P": [70, 130, 45, 33, 2], "Q": [300, 65, 140, 129, 40], "R": [48, 90, 17, 64, 5]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q", "R"])
def test_replay_modes(name, dtype, keralorn_dirs, tmp_path):
    """Through bin/trace_run: whole; all but the last 32 tokens, then token by token (the windows pass over decoded
    tokens); portions down to two tokens; mixed batches in a pool so small that pages are used again, four slots for five
    requests. Against the plain implementation, and all four in the same bits."""
    cfg, _, page = KERALORN[name]
    vocab = cfg["vocab"]
    reqs = [random_tokens(vocab, n, 300 + i) for i, n in enumerate(LENGTHS[name])]
    pcfg, w = load_plain(keralorn_dirs[name])
    rnd = None if dtype == "float32" else torch.bfloat16
    want = [plain.forward(pcfg, w, r, rnd) for r in reqs]
    exact = want if rnd is None else [plain.forward(pcfg, w, r, None) for r in reqs]
    noise = [None if rnd is None else bf16_noise(pcfg, w, r) for r in reqs]
    per = lambda n: -(-n // page) * page
    longest = sorted((per(len(r)) for r in reqs), reverse=True)
    pool = max(longest[0] + longest[1] + page, 4 * page)
    tr = TraceRun(keralorn_dirs[name], dtype, tmp_path, pool, page, extra=("--kv-shuffle", "5"))
    bits = _Bits()

    def compare(got, i, a, b, what):
        tol = _tolerance(dtype, want[i], noise[i])
        diff = (got - want[i][a:b]).abs()
        assert diff.max() <= tol, f"{name} {dtype} {what}: max |diff| {diff.max():.3e} > {tol:.3e} at {a + int(diff.max(dim=1).values.argmax())}"
        bits.check(i, a, got, f"{name} {what}")

    try:
        for i, r in enumerate(reqs):
            s = tr.run([(f"w{i}", r, range(len(r)))], end=[f"w{i}"])
            compare(tr.logits(s, vocab), i, 0, len(r), f"whole request {i}")
            if noise[i] is not None:
                mean = float((tr.logits(s, vocab) - exact[i]).abs().mean())
                assert mean <= 1.25 * noise[i][1], f"{name} whole request {i}: mean error {mean:.3e} > 1.25 x the mean rounding noise {noise[i][1]:.3e}"
        for i, r in enumerate(reqs):
            cut = max(1, len(r) - 32)
            s = tr.run([(f"d{i}", r[:cut], [cut - 1])], end=[f"d{i}"] if cut == len(r) else [])
            compare(tr.logits(s, vocab), i, cut - 1, cut, f"request {i} prefill end")
            for p in range(cut, len(r)):
                s = tr.run([(f"d{i}", r[p:p + 1], [0])], end=[f"d{i}"] if p == len(r) - 1 else [])
                compare(tr.logits(s, vocab), i, p, p + 1, f"request {i} decode at {p}")
        for i, r in enumerate(reqs):
            cuts = _portions(len(r), [7, 2, 19, 3, 2, 31, 5])
            for j, (a, b) in enumerate(cuts):
                s = tr.run([(f"p{i}", r[a:b], range(b - a))], end=[f"p{i}"] if j == len(cuts) - 1 else [])
                compare(tr.logits(s, vocab), i, a, b, f"request {i} portion {a}:{b}")
        fed, turn = [0] * len(reqs), [0] * len(reqs)
        sizes = [[9, 1, 1, 4, 1], [2, 13, 1, 1, 1, 6], [5, 1, 1, 1], [17, 1, 2, 1, 1], [3, 1, 8, 1]]
        live, waiting, steps = [], list(range(len(reqs))), 0
        while live or waiting:
            while waiting and len(live) < 4 and sum(per(len(reqs[i])) for i in live) + per(len(reqs[waiting[0]])) <= pool:
                live.append(waiting.pop(0))
            entries, ends, spans = [], [], []
            for k, i in enumerate(list(live)):
                if (steps + k) % 5 == 4 and len(live) > 1:
                    continue
                n = min(sizes[i][turn[i] % len(sizes[i])], len(reqs[i]) - fed[i])
                turn[i] += 1
                a, b = fed[i], fed[i] + n
                entries.append((f"m{i}", reqs[i][a:b], range(n)))
                spans.append((i, a, b))
                fed[i] = b
                if b == len(reqs[i]):
                    ends.append(f"m{i}")
                    live.remove(i)
            s = tr.run(entries, end=ends)
            got, at = tr.logits(s, vocab), 0
            for i, a, b in spans:
                compare(got[at:at + b - a], i, a, b, f"mixed step {steps} request {i} {a}:{b}")
                at += b - a
            steps += 1
    finally:
        tr.close()


def _uniform_attention(tensors):
    """Queries and keys scaled down: attention is close to uniform over what a token sees, so every key inside a window
    weighs 1 / size and one key more or less moves the logits far beyond the float32 tolerance."""
    for n in tensors:
        if n.endswith("mix.q") and n.replace("mix.q", "mix.v") not in tensors:
            tensors[n] = (tensors[n].float() * 0.05).to(torch.bfloat16)


def test_window_edges_show_and_agree(tmp_path):
    """With near-uniform attention the plain implementation itself moves by far more than the tolerance when a window is one
    token longer; the engine agrees with the right window at every position, in prompts (windows that straddle pages) and
    decoding token by token."""
    from stride_b200.engine.engine import StepEntry
    folder = write_model(tmp_path / "uniform", "P", _uniform_attention)
    cfg, w = load_plain(folder)
    toks = random_tokens(cfg["vocab"], 90, 77)
    want = plain.forward(cfg, w, toks)
    import copy
    longer = copy.deepcopy(cfg)
    for l in longer["layers"]:
        if l["type"] == "attention":
            l["mixer"]["mask"]["size"] += 1
    tol = logit_tolerance("float32", want)
    moved = (plain.forward(longer, w, toks) - want).abs().max(dim=1).values
    assert moved[30:].min() > 20 * tol, "the yardstick does not notice a window that is one token off"
    eng = _engine(folder, "float32", 16, 12)
    slot = eng.cache.acquire_slot()
    eng.cache.ensure(slot, 50)
    got = [eng.step([StepEntry(slot, 0, toks[:50], list(range(50)))]).cpu().clone()]
    for t in range(50, 90):
        eng.cache.ensure(slot, t + 1)
        got.append(eng.step([StepEntry(slot, t, [toks[t]], [0])]).cpu().clone())
        eng.cache.trim(slot)
    assert (torch.cat(got) - want).abs().max() <= tol


def test_long_decoding_and_slot_reuse(keralorn_dirs):
    """A short prompt, then 400 tokens one by one (the state is carried 400 times, every window passes over decoded tokens,
    pages behind the windows are given back), against the plain implementation; then the same slot again for another
    request, which must not see what the first left."""
    from stride_b200.engine.engine import StepEntry
    cfg, w = load_plain(keralorn_dirs["P"])
    eng = _engine(keralorn_dirs["P"], "float32", 16, 30)
    for seed in (1, 2):
        toks = random_tokens(cfg["vocab"], 410, seed)
        want = plain.forward(cfg, w, toks)
        slot = eng.cache.acquire_slot()
        assert slot == 0 or seed == 1
        eng.cache.ensure(slot, 10)
        got = [eng.step([StepEntry(slot, 0, toks[:10], list(range(10)))]).cpu().clone()]
        for t in range(10, 410):
            eng.cache.ensure(slot, t + 1)
            got.append(eng.step([StepEntry(slot, t, [toks[t]], [0])]).cpu().clone())
            eng.cache.trim(slot)
        assert (torch.cat(got) - want).abs().max() <= logit_tolerance("float32", want)
        eng.cache.release_slot(slot)
        eng.cache.check()


@pytest.mark.parametrize("native", [True, False])
def test_batches_of_unequal_requests_against_each_alone(keralorn_dirs, native):
    """Four requests of unequal length in one step, then single tokens of some beside portions of others: every logit has the
    bits of the request run alone; the native step program and the part-by-part driver agree."""
    from stride_b200.engine.engine import StepEntry
    cfg, _, page = KERALORN["Q"]
    reqs = [random_tokens(cfg["vocab"], n, 40 + n) for n in (150, 3, 64, 31)]
    for dtype in ("float32", "bfloat16"):
        eng = _engine(keralorn_dirs["Q"], dtype, page, 24, native_step=native)
        assert (eng._program is not None) == native
        alone = []
        for r in reqs:
            slot = eng.cache.acquire_slot()
            eng.cache.ensure(slot, len(r))
            alone.append(eng.step([StepEntry(slot, 0, r, list(range(len(r))))]).cpu().clone())
            eng.cache.release_slot(slot)
        slots = [eng.cache.acquire_slot() for _ in reqs]
        fed, got = [0] * 4, [[] for _ in reqs]
        plan = [[100, 2, 30, 1], [1, 1, 20, 30], [49, 0, 1, 0], [1, 1, 13, 0]]      # tokens of each request per step; then one by one
        step = 0
        while any(fed[i] < len(reqs[i]) for i in range(4)):
            entries, who = [], []
            for i, r in enumerate(reqs):
                n = plan[step][i] if step < len(plan) else 1
                n = min(n, len(r) - fed[i])
                if n > 0:
                    eng.cache.ensure(slots[i], fed[i] + n)
                    entries.append(StepEntry(slots[i], fed[i], r[fed[i]:fed[i] + n], list(range(n))))
                    who.append((i, n))
                    fed[i] += n
            out, at = eng.step(entries).cpu(), 0
            for i, n in who:
                got[i].append(out[at:at + n].clone())
                at += n
            step += 1
        for i in range(4):
            assert torch.equal(torch.cat(got[i]), alone[i]), f"{dtype}: request {i} in company differs from the request alone"


def test_greedy_generation_through_the_entry_point(keralorn_dirs):
    """LLM.generate with its scheduler (three requests on two slots, prompts cut into portions, a pool that forces
    requests to wait): the tokens of greedy decoding with the plain implementation."""
    from stride_b200 import LLM
    cfg, w = load_plain(keralorn_dirs["P"])
    prompts = [random_tokens(cfg["vocab"], n, 500 + n) for n in (5, 41, 23)]
    llm = LLM(keralorn_dirs["P"], dtype="float32", concurrency=2, max_rows=32, prefill_chunk=8, kv_pages=12, page_size=16,
              max_slots=2, max_context=128, device=DEV)
    outs = llm.generate(prompts, max_new_tokens=12)
    for p, o in zip(prompts, outs):
        seq = list(p)
        for tok in o.tokens:
            ref = plain.forward(cfg, w, seq)[-1]
            top = torch.topk(ref, 2).values
            if float(top[0] - top[1]) > 1e-3:       # (a near tie may go either way)
                assert tok == int(ref.argmax())
            seq.append(tok)
        assert len(o.tokens) == 12 and o.finish_reason == "length"
    bf = LLM(keralorn_dirs["Q"], dtype="bfloat16", concurrency=4, max_rows=64, prefill_chunk=16, kv_pages=16, page_size=32,
             max_slots=4, max_context=256, device=DEV)
    cfgq = KERALORN["Q"][0]
    outs = bf.generate([random_tokens(cfgq["vocab"], n, n) for n in (70, 9, 33, 120, 64)], max_new_tokens=8)
    assert all(len(o.tokens) == 8 for o in outs)


def test_command_line_generates_what_the_entry_point_generates(keralorn_dirs, tmp_path):
    """bin/stride_cli on a Keralorn folder (greedy, float32 and bfloat16): the tokens of LLM.generate."""
    import json
    import subprocess
    import sys
    from conftest import ROOT
    from stride_b200 import LLM
    cfg = KERALORN["R"][0]
    prompts = [random_tokens(cfg["vocab"], n, 900 + n) for n in (3, 50, 21)]
    (tmp_path / "in.jsonl").write_text("".join(json.dumps({"id": i, "tokens": p}) + "\n" for i, p in enumerate(prompts)))
    for path, dtype in (("exact", "float32"), ("tc", "bfloat16")):
        out = tmp_path / f"out_{path}.jsonl"
        subprocess.run([sys.executable, str(ROOT / "bin" / "stride_cli"), "--model", str(keralorn_dirs["R"]), "--input", str(tmp_path / "in.jsonl"),
                        "--output", str(out), "--max-new", "6", "--concurrency", "2", "--max-rows", "32", "--prefill-chunk", "16",
                        "--kv-blocks", "24", "--page-size", "8", "--max-slots", "4", "--max-context", "128", "--path", path], check=True, timeout=600)
        got = [json.loads(l) for l in out.read_text().splitlines()]
        llm = LLM(keralorn_dirs["R"], dtype=dtype, concurrency=2, max_rows=32, prefill_chunk=16, kv_pages=24, page_size=8, max_slots=4,
                  max_context=128, device=DEV)
        want = llm.generate(prompts, max_new_tokens=6)
        assert [g["tokens"] for g in got] == [w.tokens for w in want] and all(g["finish"] == "length" for g in got)
