"""Ganupel through the engine against the plain implementation (tests/plain_ganupel.py): every mechanism's kernels alone,
then whole models of three tiny configurations whole, decoded token by token, in portions down to two tokens and in mixed
batches with pages and slots used again, in 32-bit and in bfloat16; window edges and far tokens made to show; long
decoding; batches against each request alone; greedy generation through the entry point, its scheduler and the command line."""
from __future__ import annotations

import copy

import pytest
import torch

import plain_ganupel as plain
from conftest import TraceRun, logit_tolerance, random_tokens
from ganupel_cases import GANUPEL, load_plain, write_model
from test_replay_gpu import _Bits, _portions

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F = torch.float64


@pytest.fixture(scope="module")
def ganupel_dirs(tmp_path_factory):
    root = tmp_path_factory.mktemp("ganupel")
    return {name: write_model(root / name, name) for name in GANUPEL}


def _meta(entries):
    """[4, E] int32 on the device from (slot, first row, length, first position) records."""
    return torch.tensor([[e[k] for e in entries] for k in range(4)], dtype=torch.int32, device=DEV)


def _rows(entries):
    """positions and slots of every row of a step."""
    pos = [p for _, _, n, p0 in entries for p in range(p0, p0 + n)]
    slot = [s for s, _, n, _ in entries for _ in range(n)]
    return torch.tensor(pos, dtype=torch.int32, device=DEV), torch.tensor(slot, dtype=torch.int32, device=DEV)


# ---------------------------------------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("n,W,Sa,Sb", [(5, 96, 3, 0), (40, 100, 1, 9), (300, 64, 0, 2)])
def test_branch_fold_kernel(n, W, Sa, Sb):
    from stride_b200.kernels import ops
    g = torch.Generator().manual_seed(n + W)
    dst, a, b = (torch.randn(n, W, generator=g) for _ in range(3))
    pa = torch.randn(Sa, n, W, generator=g) if Sa else None
    pb = torch.randn(Sb, n, W, generator=g) if Sb else None
    gain = torch.randn(W, generator=g)
    dev = lambda t: None if t is None else t.to(DEV)
    d, ad, bd = dev(dst).clone(), dev(a).clone(), dev(b).clone()
    ops.branch_fold(d, a=ad, a_partials=dev(pa), ca=0.7, b=bd, b_partials=dev(pb), cb=1.3, gain=dev(gain.to(torch.bfloat16)))
    full = lambda h, p: h.double() + (p.double().sum(0) if p is not None else 0)
    want = dst.double() + gain.to(torch.bfloat16).double() * (0.7 * full(a, pa) + 1.3 * full(b, pb))
    assert (d.cpu().double() - want).abs().max() <= 1e-5 * float(want.abs().max())
    assert float(ad.abs().max()) == 0.0 and float(bd.abs().max()) == 0.0           # the branches are empty again
    # one branch, partial sums only, no gain
    d2 = dev(dst).clone()
    if pa is not None:
        ops.branch_fold(d2, a_partials=dev(pa))
        assert (d2.cpu().double() - (dst.double() + pa.double().sum(0))).abs().max() <= 1e-5 * float(want.abs().max())
    # the identity experts' share
    w = torch.rand(n, 7, generator=g)
    w[::2, 4:6] = 0.0
    x = torch.randn(n, W, generator=g).to(torch.bfloat16)
    d3 = dev(dst).clone()
    ops.row_scaled_add(d3, dev(x), dev(w), 4, 2)
    assert (d3.cpu().double() - (dst.double() + w[:, 4:6].double().sum(1, keepdim=True) * x.double())).abs().max() <= 1e-5 * float(want.abs().max())


@pytest.mark.parametrize("n,Fs,S", [(3, 136, 2), (17, 2048, 1), (2, 5000, 3)])
def test_polynorm_kernel(n, Fs, S):
    from stride_b200.kernels import ops
    g = torch.Generator().manual_seed(Fs)
    up = torch.randn(S, n, Fs, generator=g) * 1.5
    coef, eps = (0.9, -0.4, 0.3, 0.05), 1e-5
    z = up.double().sum(0)
    want = coef[0] * plain.rms(z, eps) + coef[1] * plain.rms(z ** 2, eps) + coef[2] * plain.rms(z ** 3, eps) + coef[3]
    for dt, tol in ((torch.float32, 2e-5), (torch.bfloat16, 8e-3)):
        out = torch.empty(n, Fs, dtype=dt, device=DEV)
        ops.polynorm(up.to(DEV), out, coef, eps)
        assert (out.cpu().double() - want).abs().max() <= tol * float(want.abs().max())


@pytest.mark.parametrize("E,I,top,Fs", [(5, 1, 2, 40), (3, 0, 1, 48), (4, 4, 4, 32), (40, 3, 6, 8)])
def test_routing_kernels_against_the_plain_feed_forward(E, I, top, Fs):
    """Router weights, the experts' hidden activations and the identity experts' share, put together with plain products,
    against the plain routed feed-forward; a correction that changes who is chosen but not the weights."""
    from stride_b200.kernels import ops
    g = torch.Generator().manual_seed(E * 10 + I)
    n, W, scale = 23, 24, 1.7
    t = {"p.router": torch.randn(E + I, W, generator=g), "p.correction": torch.randn(E + I, generator=g) * 0.3}
    for e in range(E):
        t[f"p.e{e}.up"], t[f"p.e{e}.down"] = torch.randn(Fs, W, generator=g) * 0.3, torch.randn(W, Fs, generator=g) * 0.3
    h = torch.randn(n, W, generator=g)
    want = plain.routed_feed_forward(h.double(), t, "p.", {"router": {"experts": E, "identity": I, "top": top, "scale": scale}})
    logits = (h.double() @ t["p.router"].double().T).float().to(DEV)
    weights = torch.empty(n, E + I, device=DEV)
    ops.moe_route(logits, t["p.correction"].to(DEV), weights, top, scale)
    assert int((weights != 0).sum(1).min()) == int((weights != 0).sum(1).max()) == top
    assert (weights.sum(1).cpu() - scale).abs().max() <= 1e-5
    up_all = torch.cat([t[f"p.e{e}.up"] for e in range(E)], 0)
    up = (h.double() @ up_all.double().T).float()
    parts = torch.stack([up * 0.25, up * 0.75]).to(DEV)                     # two K ranges
    z = torch.empty(n, E * Fs, device=DEV)
    ops.moe_activate(parts, weights, z, E, Fs)
    down_all = torch.cat([t[f"p.e{e}.down"] for e in range(E)], 1)
    out = (z.cpu().double() @ down_all.double().T).float().to(DEV)
    if I:
        ops.row_scaled_add(out, h.to(DEV), weights, E, I)
    assert (out.cpu().double() - want).abs().max() <= 2e-5 * float(want.abs().max())


def _attention_case(H, G, D, V, window, rot, page, lengths, seed, peak=None):
    """Requests of the given lengths appended in two steps each (so that the second step's queries read pages of the first),
    pages handed out in a shuffled order; returns the kernel's output and the plain result per request."""
    from stride_b200.kernels import ops
    g = torch.Generator().manual_seed(seed)
    row = max(D, V)
    scale, base = 0.3, 700.0
    width = H * D + G * D + G * V
    pages_per = [-(-n // page) for n in lengths]
    total = sum(pages_per)
    perm = torch.randperm(total + 3, generator=g).tolist()
    table = torch.full((len(lengths), max(pages_per)), -1, dtype=torch.int32)
    k = 0
    for r, c in enumerate(pages_per):
        for j in range(c):
            table[r, j] = perm[k]
            k += 1
    pages = torch.zeros(total + 3, 2, G, page, row, device=DEV)
    half = rot // 2
    freq = torch.tensor([base ** (-2.0 * i / rot) for i in range(half)], dtype=F) if rot else torch.zeros(0, dtype=F)
    angle = torch.arange(max(lengths), dtype=F)[:, None] * freq[None, :]
    cos_sin = torch.stack([torch.cos(angle), torch.sin(angle)], -1).float().to(DEV) if rot else torch.zeros(2, device=DEV)
    bias = torch.randn(H, generator=g)
    outs, wants = [], []
    for r, n in enumerate(lengths):
        qkv = torch.randn(n, width, generator=g)
        if peak is not None:      # one key whose value stands out, at a chosen distance from the last query
            far = n - 1 - peak
            qkv[far, H * D + G * D:] = 1e4
        cut = max(1, n // 3)
        got = []
        for a, b in ((0, cut), (cut, n)):
            if a == b:
                continue
            pos, slot = _rows([(r, 0, b - a, a)])
            q = torch.empty(b - a, H * D, device=DEV)
            parts = torch.stack([qkv[a:b] * 0.5, qkv[a:b] * 0.5]).to(DEV)
            ops.qkv_rotate_append(parts, pos, slot, cos_sin, rot, q, pages, table.to(DEV), H, G, D, V)
            out = torch.empty(b - a, H * V, device=DEV)
            ops.sigmoid_attention(q, out, pages, table.to(DEV), pos, slot, bias.to(DEV), H, G, D, V, window, scale)
            got.append(out.cpu())
        outs.append(torch.cat(got))
        t = {"p.q": torch.eye(H * D), "p.k": torch.eye(G * D), "p.v": torch.eye(G * V), "p.o": torch.eye(H * V), "p.pb": bias}
        m = {"heads": H, "kv_heads": G, "dim": D, "vdim": V, "scale": scale}
        if window:
            m["mask"] = {"size": window}
        if rot:
            m["rot"] = {"dims": rot, "base": base}
        # the plain function projects its input: feed q, k, v through identity matrices, one sequence at a time
        h = qkv.double()
        tt = {"p.q": torch.cat([torch.eye(H * D), torch.zeros(H * D, width - H * D)], 1),
              "p.k": torch.cat([torch.zeros(G * D, H * D), torch.eye(G * D), torch.zeros(G * D, G * V)], 1),
              "p.v": torch.cat([torch.zeros(G * V, H * D + G * D), torch.eye(G * V)], 1), "p.o": t["p.o"], "p.pb": bias}
        wants.append(plain.sigmoid_window_attention(h, tt, "p.", m))
    return outs, wants


@pytest.mark.parametrize("H,G,D,V,window,rot,page", [(4, 2, 32, 24, 24, 16, 16), (2, 2, 48, 64, 7, 48, 8), (8, 2, 64, 64, 100, 32, 32),
                                                      (2, 1, 128, 96, 0, 0, 16), (5, 5, 20, 12, 1, 10, 8), (3, 1, 12, 200, 33, 12, 16)])
def test_sigmoid_attention_kernels(H, G, D, V, window, rot, page):
    outs, wants = _attention_case(H, G, D, V, window, rot, page, [70, 3, 131], H * D + window)
    for got, want in zip(outs, wants):
        assert (got.double() - want).abs().max() <= 2e-5 * float(want.abs().max())


@pytest.mark.parametrize("H,G,D,V,window,page", [(8, 2, 64, 64, 100, 32), (4, 2, 32, 48, 24, 16), (2, 2, 96, 96, 72, 64), (16, 1, 16, 128, 0, 8),
                                                 (3, 3, 256, 16, 200, 16)])
def test_sigmoid_attention_on_the_tensor_cores(H, G, D, V, window, page):
    """The bfloat16 tile kernel against the kernel with a block per token and head on the same pages (the weights' two bfloat16
    parts keep them to 2^-17, so what differs is the order of the sums), against the sum in 64-bit, and a request cut into a
    prompt, portions and single tokens in the same bits."""
    from stride_b200.kernels import ops
    assert ops.sigmoid_attention_tiles_supported(H, G, D, V, max(D, V))
    g = torch.Generator().manual_seed(H * D + V)
    n, row, scale = 300, max(D, V), 0.11
    per = -(-n // page)
    perm = torch.randperm(per + 2, generator=g)[:per].to(torch.int32)
    table = perm.view(1, per).to(DEV)
    k = (torch.randn(n, G, D, generator=g)).to(torch.bfloat16)
    v = (torch.randn(n, G, V, generator=g)).to(torch.bfloat16)
    q = (torch.randn(n, H, D, generator=g)).to(torch.bfloat16)
    bias = torch.randn(H, generator=g)
    pages = torch.zeros(per + 2, 2, G, page, row, dtype=torch.bfloat16)
    for j in range(n):
        pages[perm[j // page], 0, :, j % page, :D] = k[j]
        pages[perm[j // page], 1, :, j % page, :V] = v[j]
    pages = pages.to(DEV)
    want = torch.zeros(n, H, V, dtype=F)
    i, j = torch.arange(n)[:, None], torch.arange(n)[None, :]
    seen = (j <= i) & ((i - j < window) if window else (j <= i))
    for h in range(H):
        w = torch.sigmoid(q[:, h].double() @ k[:, h // (H // G)].double().T * scale + bias[h].double()) * seen
        want[:, h] = w @ v[:, h // (H // G)].double()

    def run(a, b, tiles):
        pos = torch.arange(a, b, dtype=torch.int32, device=DEV)
        slot = torch.zeros(b - a, dtype=torch.int32, device=DEV)
        out = torch.empty(b - a, H * V, dtype=torch.bfloat16, device=DEV)
        qd = q[a:b].reshape(b - a, H * D).to(DEV)
        if tiles:
            ops.sigmoid_attention_tiles(qd, out, pages, table, _meta([(0, 0, b - a, a)]), 1, bias.to(DEV), H, G, D, V, window, scale)
        else:
            ops.sigmoid_attention(qd, out, pages, table, pos, slot, bias.to(DEV), H, G, D, V, window, scale)
        return out.cpu()

    whole, simple = run(0, n, True), run(0, n, False)
    tol = 2.0 ** -7 * float(want.abs().max())
    assert (whole.double().view(n, H, V) - want).abs().max() <= tol
    assert (whole.double() - simple.double()).abs().max() <= tol
    cuts = [0, 70, 71, 73, 130, 131, 290, 291, 300]
    parts = torch.cat([run(a, b, True) for a, b in zip(cuts, cuts[1:])])
    assert torch.equal(parts, whole)


@pytest.mark.parametrize("window", [9, 64, 65])
def test_a_key_at_the_window_edge_shows(window):
    """A value of 10,000 among values of order one: just inside the window it dominates the last token's output, just outside it
    is gone; with a sum that is not normalised one key more or less can not hide."""
    for peak, inside in ((window - 1, True), (window, False)):
        outs, wants = _attention_case(2, 1, 16, 8, window, 8, 16, [150], 5, peak=peak)
        last, want = outs[0][-1].double(), wants[0][-1]
        assert (last - want).abs().max() <= 2e-5 * float(want.abs().max())
        assert (float(want.abs().max()) > 50.0) == inside


def _scan_reference(q, g, k, v, state):
    """q, g, k [n, H, D], v [n, H, V]; returns (o [n, H, V], final state) in 64-bit."""
    o = torch.empty(v.shape, dtype=F)
    S = state.double().clone()
    for t in range(q.shape[0]):
        S = g[t].double()[:, :, None] * S + k[t].double()[:, :, None] * v[t].double()[:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t].double())
    return o, S


@pytest.mark.parametrize("H,D,V", [(3, 16, 40), (2, 40, 16), (1, 128, 128), (4, 64, 32), (2, 10, 30), (1, 200, 70)])
def test_gated_scan_kernel(H, D, V):
    """Entries of unequal length in one launch against the recurrence in 64-bit; a request cut into two launches and one
    walked token by token give the bits of one launch; position 0 starts from zero whatever the slot held."""
    from stride_b200.kernels import ops
    gen = torch.Generator().manual_seed(H * D + V)
    lengths, slots = [37, 1, 150, 2], [2, 0, 3, 1]
    n, HD, HV = sum(lengths), H * D, H * V
    width = 3 * HD + HV
    act = torch.randn(n, width, generator=gen) * 0.7
    act[:, HD:2 * HD] = torch.rand(n, HD, generator=gen)                     # gates in (0, 1)
    q, g, k = (act[:, i * HD:(i + 1) * HD].view(n, H, D) for i in range(3))
    v = act[:, 3 * HD:].view(n, H, V)
    rows = [sum(lengths[:i]) for i in range(4)]
    state = torch.randn(5, H, D, V, generator=gen).to(DEV)                   # garbage that a fresh request must not see

    def launch(entries, rows_of_act, st):
        out = torch.zeros(rows_of_act.shape[0], HV, device=DEV)
        ops.gated_scan(rows_of_act.to(DEV).contiguous(), 0, HD, 2 * HD, 3 * HD, _meta(entries), len(entries), st, out, H, D, V)
        return out.cpu()

    whole = launch([(slots[i], rows[i], lengths[i], 0) for i in range(4)], act, state)
    finals = state.cpu().clone()
    for i in range(4):
        a, b = rows[i], rows[i] + lengths[i]
        want, last = _scan_reference(q[a:b], g[a:b], k[a:b], v[a:b], torch.zeros(H, D, V))
        assert (whole[a:b].view(-1, H, V).double() - want).abs().max() <= 2e-5 * float(want.abs().max()), f"entry {i}"
        assert (finals[slots[i]].double() - last).abs().max() <= 2e-5 * float(last.abs().max())
    a, cut = rows[2], 53
    st2 = torch.full((5, H, D, V), 7.0, device=DEV)
    first = launch([(4, 0, cut, 0)], act[a:a + cut], st2)
    second = launch([(4, 0, lengths[2] - cut, cut)], act[a + cut:a + lengths[2]], st2)
    assert torch.equal(torch.cat([first, second]), whole[a:a + lengths[2]])
    assert torch.equal(st2[4].cpu(), finals[3])
    st3 = torch.zeros(5, H, D, V, device=DEV)
    single = torch.cat([launch([(1, 0, 1, t)], act[rows[0] + t:rows[0] + t + 1], st3) for t in range(lengths[0])])
    assert torch.equal(single, whole[rows[0]:rows[0] + lengths[0]])


def test_gated_scan_keeps_a_far_token():
    """One early token writes, gates of 0.995 for hundreds of tokens, then a query: the output is that token's value decayed
    exactly that often; a state that lost it, or decayed once more or less, shows."""
    from stride_b200.kernels import ops
    D, V, n, far = 32, 32, 600, 3
    act = torch.zeros(n, 3 * D + V)
    act[:, D:2 * D] = 0.995
    act[far, 2 * D:3 * D] = 1.0
    act[far, 3 * D:] = torch.arange(1, V + 1).float()
    act[n - 1, :D] = 0.5
    out, st = torch.zeros(n, V, device=DEV), torch.zeros(1, 1, D, V, device=DEV)
    ops.gated_scan(act.to(DEV), 0, D, 2 * D, 3 * D, _meta([(0, 0, n, 0)]), 1, st, out, 1, D, V)
    want = (0.995 ** (n - 1 - far)) * D * 0.5 * torch.arange(1, V + 1).double()
    assert (out[n - 1].cpu().double() - want).abs().max() <= 1e-4 * float(want.max())


def test_hgrn2_activation_and_group_norm_kernels():
    from stride_b200.kernels import ops
    g = torch.Generator().manual_seed(8)
    n, H, D, V = 11, 3, 16, 40
    HD, HV = H * D, H * V
    proj = torch.randn(2, n, 2 * HD + HV, generator=g)
    bias, lower = torch.randn(HD, generator=g), torch.rand(HD, generator=g)
    act = torch.empty(n, 3 * HD + HV, device=DEV)
    ops.hgrn2_activate(proj.to(DEV), bias.to(DEV), lower.to(DEV), act, HD, HV)
    z = proj.double().sum(0)
    f = lower.double() + (1 - lower.double()) * torch.sigmoid(z[:, HD:2 * HD] + bias.double())
    want = torch.cat([plain.silu(z[:, :HD]), f, 1 - f, z[:, 2 * HD:]], 1)
    assert (act.cpu().double() - want).abs().max() <= 1e-5
    o, gain = torch.randn(n, HV, generator=g) * 3, torch.randn(V, generator=g)
    for dt, tol in ((torch.float32, 1e-5), (torch.bfloat16, 8e-3)):
        y = torch.empty(n, HV, dtype=dt, device=DEV)
        ops.group_rmsnorm(o.to(DEV), gain.to(DEV), 1e-5, y, H, V)
        ref = (plain.rms(o.double().view(n, H, V), 1e-5) * gain.double()).view(n, HV)
        assert (y.cpu().double() - ref).abs().max() <= tol * float(ref.abs().max())


@pytest.mark.parametrize("C,B,K", [(80, 5, 3), (64, 1, 2), (256, 4, 4), (60, 3, 5), (48, 2, 1), (600, 2, 4)])
def test_rglru_kernels_across_steps(C, B, K):
    """The recurrent block between its projections, with requests cut into steps of 1, 2 and more tokens than taps, beside one
    another and in slots that hold another request's record: against the plain block (whose projections are identities here),
    and every cut in the bits of the whole."""
    from stride_b200.kernels import ops
    gen = torch.Generator().manual_seed(C + K)
    bw = C // B
    t = {"p.y": torch.cat([torch.eye(C), torch.zeros(C, C)], 1), "p.x": torch.cat([torch.zeros(C, C), torch.eye(C)], 1), "p.o": torch.eye(C),
         "p.y.b": torch.randn(C, generator=gen) * 0.3, "p.x.b": torch.randn(C, generator=gen) * 0.3, "p.conv": torch.randn(C, K, generator=gen) * 0.5,
         "p.conv.b": torch.randn(C, generator=gen) * 0.2, "p.ra": torch.randn(B, bw, bw, generator=gen) * 0.3, "p.ra.b": torch.randn(B, bw, generator=gen),
         "p.ri": torch.randn(B, bw, bw, generator=gen) * 0.3, "p.ri.b": torch.randn(B, bw, generator=gen), "p.lam": torch.randn(C, generator=gen) - 3.0}
    lengths = [23, 1, 9]
    inputs = [torch.randn(n, 2 * C, generator=gen) for n in lengths]
    wants = [plain.rglru(h.double(), t, "p.", {"width": C, "blocks": B}) for h in inputs]
    dev = lambda name: t[name].float().contiguous().to(DEV)
    gate_w = torch.cat([t["p.ra"], t["p.ri"]], 1).transpose(1, 2).contiguous().to(DEV)       # per block [input, outputs of r | i]

    def step(entries, rows, state):
        n = rows.shape[0]
        pos, slot = _rows(entries)
        proj = torch.stack([rows * 0.25, rows * 0.75]).to(DEV)
        u = torch.empty(n, C, device=DEV)
        ops.rglru_conv(proj, dev("p.x.b"), dev("p.conv"), dev("p.conv.b"), pos, slot, state, u)
        a, d, y = (torch.empty(n, C, device=DEV) for _ in range(3))
        ops.rglru_gates(gate_w, dev("p.ra.b").reshape(-1), dev("p.ri.b").reshape(-1), dev("p.lam"), dev("p.y.b"), u, proj, a, d, y)
        out = torch.empty(n, C, device=DEV)
        ops.rglru_scan(a, d, y, proj, dev("p.x.b"), _meta(entries), len(entries), state, out, K)
        return out.cpu()

    state = torch.randn(4, K, C, generator=gen).to(DEV)                       # what other requests left in the slots
    rows = [0, lengths[0], lengths[0] + lengths[1]]
    whole = step([(i, rows[i], lengths[i], 0) for i in range(3)], torch.cat(inputs), state)
    for i in range(3):
        got = whole[rows[i]:rows[i] + lengths[i]].double()
        assert (got - wants[i]).abs().max() <= 2e-5 * max(1.0, float(wants[i].abs().max())), f"request {i}"
    # requests 0 and 2 again in other slots, cut into steps of 1, 2, 1, 5, 1, 1, .. tokens side by side
    st2 = torch.full((4, K, C), 3.0, device=DEV)
    fed, got = {0: 0, 2: 0}, {0: [], 2: []}
    sizes = {0: [1, 2, 1, 5, 1, 1, 7, 3, 2], 2: [2, 1, 1, 1, 4]}
    k = 0
    while any(fed[i] < lengths[i] for i in fed):
        entries, chunks, at = [], [], 0
        for i in fed:
            m = min(sizes[i][k % len(sizes[i])], lengths[i] - fed[i])
            if m > 0:
                entries.append((3 - i, at, m, fed[i]))
                chunks.append((i, inputs[i][fed[i]:fed[i] + m]))
                at += m
                fed[i] += m
        out = step(entries, torch.cat([c for _, c in chunks]), st2)
        at = 0
        for i, c in chunks:
            got[i].append(out[at:at + c.shape[0]])
            at += c.shape[0]
        k += 1
    for i in fed:
        assert torch.equal(torch.cat(got[i]), whole[rows[i]:rows[i] + lengths[i]]), f"request {i} cut into steps"


# ---------------------------------------------------------------------------------------------- whole models
def _engine(model_dir, dtype, page, pages, rows=256, slots=4, **kw):
    from stride_b200.engine.engine import Engine, EngineOptions
    return Engine(model_dir, EngineOptions(dtype=dtype, max_rows=rows, max_full_rows=rows, max_slots=slots, kv_pages=pages,
                                           page_size=page, max_context=pages * page, device=DEV, **kw))


def _noise(cfg, w, tokens):
    """max and mean |plain with bfloat16 rounding - plain exact| over the sequence's logits."""
    d = (plain.forward(cfg, w, tokens, torch.bfloat16) - plain.forward(cfg, w, tokens)).abs()
    return float(d.max()), float(d.mean())


CLOSE_CALL = 3e-3      # a choice score's lead below this is within what bfloat16 rounding moves a score by


def _close_calls(cfg, w, tokens):
    """Per position: True where some routed layer chooses its experts by a lead that bfloat16 rounding can overturn. There two
    right implementations may choose different experts, and the position is held to the float32 engine alone."""
    margins = []
    plain.forward(cfg, w, tokens, margins=margins)
    if not margins:
        return torch.zeros(len(tokens), dtype=torch.bool)
    return torch.stack(margins).min(0).values < CLOSE_CALL


LENGTHS = {"X": [70, 130, 45, 33, 2], "Y": [300, 65, 140, 129, 40], "Z": [48, 90, 17, 64, 5]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["X", "Y", "Z"])
def test_replay_modes(name, dtype, ganupel_dirs, tmp_path):
    """Through bin/trace_run: whole; all but the last 32 tokens, then token by token; portions down to two tokens; mixed
    batches in a pool so small that pages are used again, four slots for five requests. Against the plain implementation,
    and all four in the same bits. float32: the framework's yardstick. bfloat16: the largest deviation from the plain
    implementation that rounds at the same places stays within the largest rounding noise of the same sequence, and the mean
    error against the exact logits within 1.25 times the mean rounding noise."""
    cfg, _, page = GANUPEL[name]
    vocab = cfg["vocab"]
    reqs = [random_tokens(vocab, n, 300 + i) for i, n in enumerate(LENGTHS[name])]
    pcfg, w = load_plain(ganupel_dirs[name])
    rnd = None if dtype == "float32" else torch.bfloat16
    exact = [plain.forward(pcfg, w, r).float() for r in reqs]
    want = exact if rnd is None else [plain.forward(pcfg, w, r, rnd).float() for r in reqs]
    noise = [None if rnd is None else _noise(pcfg, w, r) for r in reqs]
    close = [None if rnd is None else _close_calls(pcfg, w, r) for r in reqs]
    per = lambda n: -(-n // page) * page
    longest = sorted((per(len(r)) for r in reqs), reverse=True)
    pool = max(longest[0] + longest[1] + page, 4 * page)
    tr = TraceRun(ganupel_dirs[name], dtype, tmp_path, pool, page, extra=("--kv-shuffle", "5"))
    bits = _Bits()

    def compare(got, i, a, b, what):
        tol = logit_tolerance(dtype, want[i]) if noise[i] is None else noise[i][0]
        diff = (got - want[i][a:b]).abs()
        if close[i] is not None:
            diff = diff[~close[i][a:b]]
            if diff.numel() == 0:
                return bits.check(i, a, got, f"{name} {what}")
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


def test_window_edges_show_and_agree(ganupel_dirs):
    """The weights of this attention are not normalised, so a window that is one token longer adds a key's whole value: the
    plain implementation itself moves by far more than the tolerance. The engine agrees with the right windows at every
    position, in a prompt whose windows straddle pages and decoding token by token with pages trimmed behind the windows."""
    from stride_b200.engine.engine import StepEntry
    cfg, w = load_plain(ganupel_dirs["X"])
    toks = random_tokens(cfg["vocab"], 90, 77)
    want = plain.forward(cfg, w, toks).float()
    tol = logit_tolerance("float32", want)
    for delta in (1, -1):
        other = copy.deepcopy(cfg)
        for l in other["layers"]:
            if l["type"] == "parallel":
                l["mixer"]["left"]["mask"]["size"] += delta
        moved = (plain.forward(other, w, toks).float() - want).abs().max(dim=1).values
        assert moved[30:].min() > 20 * tol, "the yardstick does not notice a window that is one token off"
    eng = _engine(ganupel_dirs["X"], "float32", 16, 12)
    slot = eng.cache.acquire_slot()
    eng.cache.ensure(slot, 50)
    got = [eng.step([StepEntry(slot, 0, toks[:50], list(range(50)))]).cpu().clone()]
    for t in range(50, 90):
        eng.cache.ensure(slot, t + 1)
        got.append(eng.step([StepEntry(slot, t, [toks[t]], [0])]).cpu().clone())
        eng.cache.trim(slot)
    assert (torch.cat(got) - want).abs().max() <= tol


def test_the_first_tokens_of_a_sequence(ganupel_dirs):
    """Positions 0, 1, 2 one by one in a slot that another request used: zeros in front of the convolution, empty states, a
    window with fewer keys than its size."""
    from stride_b200.engine.engine import StepEntry
    cfg, w = load_plain(ganupel_dirs["Z"])
    eng = _engine(ganupel_dirs["Z"], "float32", 8, 16)
    for seed in (3, 4):
        toks = random_tokens(cfg["vocab"], 12, seed)
        want = plain.forward(cfg, w, toks).float()
        slot = eng.cache.acquire_slot()
        got = []
        for t in range(12):
            eng.cache.ensure(slot, t + 1)
            got.append(eng.step([StepEntry(slot, t, [toks[t]], [0])]).cpu().clone())
        assert (torch.cat(got) - want).abs().max() <= logit_tolerance("float32", want)
        eng.cache.release_slot(slot)


def test_long_decoding_and_slot_reuse(ganupel_dirs):
    """A short prompt, then 400 tokens one by one (the states are carried 400 times, every window passes over decoded tokens,
    pages behind the windows are given back), against the plain implementation; then the same slot again for another request,
    which must not see what the first left."""
    from stride_b200.engine.engine import StepEntry
    cfg, w = load_plain(ganupel_dirs["X"])
    eng = _engine(ganupel_dirs["X"], "float32", 16, 30)
    for seed in (1, 2):
        toks = random_tokens(cfg["vocab"], 410, seed)
        want = plain.forward(cfg, w, toks).float()
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


def test_a_forgotten_state_would_show(ganupel_dirs):
    """With the recurrences made to remember (ganupel_cases.remember_longer), a request whose states are dropped in the middle
    moves its later logits far beyond the tolerance: the replay tests can see a lost or a foreign state."""
    cfg, w = load_plain(ganupel_dirs["X"])
    toks = random_tokens(cfg["vocab"], 80, 9)
    want = plain.forward(cfg, w, toks).float()
    fresh = plain.forward(cfg, w, toks[60:]).float()          # the same tokens without what came before
    assert (fresh[-1] - want[-1]).abs().max() > 50 * logit_tolerance("float32", want)


@pytest.mark.parametrize("native", [True, False])
def test_batches_of_unequal_requests_against_each_alone(ganupel_dirs, native):
    """Four requests of unequal length in one step, then single tokens of some beside portions of others: every logit has the
    bits of the request run alone; the native step program and the part-by-part driver agree."""
    from stride_b200.engine.engine import StepEntry
    cfg, _, page = GANUPEL["Y"]
    reqs = [random_tokens(cfg["vocab"], n, 40 + n) for n in (150, 3, 64, 31)]
    for dtype in ("float32", "bfloat16"):
        eng = _engine(ganupel_dirs["Y"], dtype, page, 24, native_step=native)
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


def test_greedy_generation_through_the_entry_point(ganupel_dirs):
    """LLM.generate with its scheduler (three requests on two slots, prompts cut into portions, decode steps replayed from
    CUDA graphs): the tokens of greedy decoding with the plain implementation."""
    from stride_b200 import LLM
    cfg, w = load_plain(ganupel_dirs["X"])
    prompts = [random_tokens(cfg["vocab"], n, 500 + n) for n in (5, 41, 23)]
    llm = LLM(ganupel_dirs["X"], dtype="float32", concurrency=2, max_rows=32, prefill_chunk=8, kv_pages=12, page_size=16,
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
    bf = LLM(ganupel_dirs["Y"], dtype="bfloat16", concurrency=4, max_rows=64, prefill_chunk=16, kv_pages=16, page_size=32,
             max_slots=4, max_context=256, device=DEV)
    cfgy = GANUPEL["Y"][0]
    outs = bf.generate([random_tokens(cfgy["vocab"], n, n) for n in (70, 9, 33, 120, 64)], max_new_tokens=8)
    assert all(len(o.tokens) == 8 for o in outs)


def test_command_line_generates_what_the_entry_point_generates(ganupel_dirs, tmp_path):
    """bin/stride_cli on a Ganupel folder (greedy, float32 and bfloat16): the tokens of LLM.generate."""
    import json
    import subprocess
    import sys
    from conftest import ROOT
    from stride_b200 import LLM
    cfg = GANUPEL["Z"][0]
    prompts = [random_tokens(cfg["vocab"], n, 900 + n) for n in (3, 50, 21)]
    (tmp_path / "in.jsonl").write_text("".join(json.dumps({"id": i, "tokens": p}) + "\n" for i, p in enumerate(prompts)))
    for path, dtype in (("exact", "float32"), ("tc", "bfloat16")):
        out = tmp_path / f"out_{path}.jsonl"
        subprocess.run([sys.executable, str(ROOT / "bin" / "stride_cli"), "--model", str(ganupel_dirs["Z"]), "--input", str(tmp_path / "in.jsonl"),
                        "--output", str(out), "--max-new", "6", "--concurrency", "2", "--max-rows", "32", "--prefill-chunk", "16",
                        "--kv-blocks", "24", "--page-size", "8", "--max-slots", "4", "--max-context", "128", "--path", path], check=True, timeout=600)
        got = [json.loads(l) for l in out.read_text().splitlines()]
        llm = LLM(ganupel_dirs["Z"], dtype=dtype, concurrency=2, max_rows=32, prefill_chunk=16, kv_pages=24, page_size=8, max_slots=4,
                  max_context=128, device=DEV)
        want = llm.generate(prompts, max_new_tokens=6)
        assert [g["tokens"] for g in got] == [w.tokens for w in want] and all(g["finish"] == "length" for g in got)
