"""Ganupel on the CPU: configuration errors, the tensor plan, the cache manager's books for layers that ask for pages and a
state at once, and the plain implementation against hand-made cases of every mechanism."""
from __future__ import annotations

import copy
import math

import pytest
import torch

import plain_ganupel as plain
from ganupel_cases import GANUPEL, GANUPEL_X, GANUPEL_Z

F = torch.float64


def test_the_architecture_is_registered_and_chosen_by_config():
    from stride_b200.config import resolve_architecture
    assert resolve_architecture(GANUPEL_X).name == "Ganupel"
    assert resolve_architecture({"model_type": "ganupel"}).name == "Ganupel"


@pytest.mark.parametrize("name", list(GANUPEL))
def test_tensor_plan(name):
    from stride_b200.weights.random_init import model_plan
    cfg = GANUPEL[name][0]
    plan = model_plan(cfg)
    W = cfg["width"]
    assert plan["embed"].shape == (cfg["vocab"], W) and plan["head"].shape == (cfg["vocab"], W) and plan["final.norm"].shape == (W,)
    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}."
        assert plan[p + "norm1"].shape == plan[p + "ls1"].shape == (W,)
        assert (p + "ls2" in plan) == (p + "norm2" in plan) == (l["mlp"] is not None)
        m = l["mixer"]
        if l["type"] == "parallel":
            a, g = m["left"], m["right"]
            assert plan[p + "mix.left.q"].shape == (a["heads"] * a["dim"], W) and plan[p + "mix.left.v"].shape == (a["kv_heads"] * a["vdim"], W)
            assert plan[p + "mix.left.o"].shape == (W, a["heads"] * a["vdim"]) and plan[p + "mix.left.pb"].shape == (a["heads"],)
            assert plan[p + "mix.right.f"].shape == (g["heads"] * g["dim"], W) and plan[p + "mix.right.norm"].shape == (g["vdim"],)
            assert plan[p + "mix.right.lower"].shape == plan[p + "mix.right.f.b"].shape == (g["heads"] * g["dim"],)
        else:
            bw = m["width"] // m["blocks"]
            assert plan[p + "mix.ra"].shape == plan[p + "mix.ri"].shape == (m["blocks"], bw, bw)
            assert plan[p + "mix.conv"].shape == (m["width"], m["conv"]) and plan[p + "mix.o"].shape == (W, m["width"])
        if l["mlp"] and l["mlp"]["kind"] == "moe":
            r = l["mlp"]["router"]
            assert plan[p + "mlp.router"].shape == (r["experts"] + r["identity"], W)
            assert sum(n.startswith(p + "mlp.e") for n in plan) == 2 * r["experts"]
        elif l["mlp"]:
            assert plan[p + "mlp.act"].shape == (4,)


@pytest.mark.parametrize("edit,word", [
    (lambda c: c["layers"][0].__setitem__("type", "conv"), "type"),
    (lambda c: c["layers"][0]["mixer"]["left"].__setitem__("kv_heads", 3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].__setitem__("dims", 15), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"].pop("left_scale"), "left_scale"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("blocks", 7), "blocks"),
    (lambda c: c["layers"][1]["mlp"].__setitem__("kind", "gated"), "mlp.kind"),
    (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 9), "router"),
    (lambda c: c.pop("norm"), "norm.eps"),
])
def test_config_errors_name_the_key(edit, word):
    from stride_b200.config import ConfigError, resolve_architecture
    cfg = copy.deepcopy(GANUPEL_X)
    edit(cfg)
    with pytest.raises(ConfigError, match=word.replace(".", r"\.").replace("[", r"\[")):
        resolve_architecture(cfg).parse_config(cfg)


def test_model_spec_follows_the_layer_list():
    from stride_b200.config import resolve_architecture
    arch = resolve_architecture(GANUPEL_Z)
    spec = arch.model_spec(arch.parse_config(GANUPEL_Z))
    assert [l.block for l in spec.layers] == ["prenorm_scaled_mixer", "prenorm_scaled", "prenorm_scaled"]
    assert [l.mixer.kind for l in spec.layers] == ["rglru", "parallel", "parallel"]
    assert [m.kind for m in spec.layers[1].mixer.params["members"]] == ["sigmoid_attention", "hgrn2"]
    assert spec.layers[1].mixer.params["members"][0].params["window"] == 1
    assert spec.layers[2].feed_forward.kind == "routed" and spec.layers[1].feed_forward.kind == "polynorm"
    assert spec.layers[0].mixer_norm.params["offset"] == 1.0


def test_a_layer_may_ask_for_pages_and_a_state():
    """The cache manager takes a list of needs for one schedule entry: pages with a window and a state record side by side;
    slots and pages are given back and used again, and the books stay whole."""
    from stride_b200.cache.manager import CacheManager
    from stride_b200.parts.base import CacheNeed
    pages = CacheNeed("pages", kv_heads=2, head_dim=8, window=5, dtype=torch.float32)
    state = CacheNeed("state", state_shape=(3, 4))
    other = CacheNeed("state", state_shape=(2, 6))
    cm = CacheManager([[pages, state], other, [pages, state], None], device="cpu", max_slots=2, max_context=64, page_size=4, num_pages=10)
    first, second, third = cm.layer_cache(0), cm.layer_cache(1), cm.layer_cache(2)
    assert first.parts is not None and len(first.parts) == 2 and second.parts is None
    assert first.parts[0].pages.shape[1:] == (2, 2, 4, 8) and first.parts[1].state.shape == (3, 3, 4) and second.state.shape == (3, 2, 6)
    assert first.parts[0].pages.data_ptr() != third.parts[0].pages.data_ptr() and len(cm.groups) == 1
    a = cm.acquire_slot()
    first.parts[1].state[a].fill_(7.0)
    assert cm.ensure(a, 30)
    assert cm.trim(a) > 0            # pages behind the window come back
    cm.release_slot(a)
    b = cm.acquire_slot()
    assert b == a and float(first.parts[1].state[b].abs().sum()) == 0.0
    cm.check()


# ------------------------------------------------------------------------------------------------ the plain implementation itself
def test_plain_norm_and_rotation():
    x = torch.tensor([[3.0, 4.0]], dtype=F)
    assert torch.allclose(plain.offset_rms_norm(x, torch.tensor([0.0, 1.0], dtype=F), 0.0), torch.tensor([[3.0, 8.0]], dtype=F) / math.sqrt(12.5))
    v = torch.zeros(3, 1, 6, dtype=F)
    v[:, 0, 0] = 1.0
    v[:, 0, 5] = 9.0
    r = plain.rotate(v, 4, 100.0)
    assert torch.allclose(r[2, 0, :4], torch.tensor([math.cos(2.0), 0.0, math.sin(2.0), 0.0], dtype=F)) and float(r[2, 0, 5]) == 9.0
    assert torch.equal(r[0], v[0])


def test_plain_window_and_sigmoid_weights():
    """Values that name their position: with zero queries every visible key weighs sigmoid(bias), so the output counts the window."""
    T, W = 9, 4
    t = {"q": torch.zeros(2, W), "k": torch.zeros(2, W), "v": torch.zeros(1, W), "o": torch.eye(1), "pb": torch.tensor([0.0])}
    t["v"][0, 0] = 1.0
    h = torch.zeros(T, W, dtype=F)
    h[:, 0] = torch.arange(1, T + 1, dtype=F)
    out = plain.sigmoid_window_attention(h, {"p." + k: v for k, v in t.items()}, "p.", {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 1, "scale": 1.0,
                                                                                      "mask": {"size": 3}})
    want = [0.5 * sum(range(max(1, i - 1), i + 2)) for i in range(T)]      # positions i-2..i, values 1-based
    assert torch.allclose(out[:, 0], torch.tensor(want, dtype=F))


def test_plain_routing():
    """Three experts and one identity expert; the correction decides who is chosen, not what the chosen weigh."""
    W = 2
    t = {"p.router": torch.tensor([[1.0, 0.0], [0.0, 1.0], [0.0, 0.0], [-1.0, 0.0]]), "p.correction": torch.tensor([0.0, 0.0, 10.0, 0.0])}
    for e in range(3):
        t[f"p.e{e}.up"], t[f"p.e{e}.down"] = torch.eye(W) * (e + 1), torch.eye(W)
    mlp = {"router": {"experts": 3, "identity": 1, "top": 2, "scale": 3.0}}
    h = torch.tensor([[2.0, 0.0]], dtype=F)
    s = torch.softmax(torch.tensor([2.0, 0.0, 0.0, -2.0], dtype=F), 0)
    g0, g2 = 3.0 * s[0] / (s[0] + s[2]), 3.0 * s[2] / (s[0] + s[2])        # experts 2 (by its correction) and 0
    want = g0 * torch.tensor([4.0, 0.0], dtype=F) + g2 * torch.tensor([36.0, 0.0], dtype=F)
    assert torch.allclose(plain.routed_feed_forward(h, t, "p.", mlp), want[None])
    t["p.correction"] = torch.tensor([0.0, 0.0, 0.0, 10.0])                  # now the identity expert and expert 0
    g0, g3 = 3.0 * s[0] / (s[0] + s[3]), 3.0 * s[3] / (s[0] + s[3])
    assert torch.allclose(plain.routed_feed_forward(h, t, "p.", mlp), (g0 * torch.tensor([4.0, 0.0], dtype=F) + g3 * h[0])[None])


def test_plain_recurrences_by_hand():
    # the gated linear attention with one head, one key channel, one value: S = f S + (1 - f) v, o = S q
    t = {"p.q": torch.tensor([[1.0]]), "p.f": torch.tensor([[0.0]]), "p.f.b": torch.tensor([0.0]), "p.lower": torch.tensor([0.5]),
         "p.v": torch.tensor([[2.0]]), "p.norm": torch.tensor([1.0]), "p.o": torch.eye(1)}
    h = torch.ones(3, 1, dtype=F)
    f, S, outs = 0.75, 0.0, []
    for _ in range(3):
        S = f * S + (1 - f) * 2.0
        outs.append(S * (1.0 / (1.0 + math.exp(-1.0))))
    got = plain.hgrn2(h, t, "p.", {"heads": 1, "dim": 1, "vdim": 1}, 0.0)
    assert torch.allclose(got[:, 0], torch.tensor([1.0, 1.0, 1.0], dtype=F))          # a norm over one value leaves its sign
    got = plain.hgrn2(h, dict(t, **{"p.norm": torch.tensor([1.0, 1.0]), "p.v": torch.tensor([[2.0], [0.0]]), "p.o": torch.eye(2)}), "p.",
                      {"heads": 1, "dim": 1, "vdim": 2}, 0.0)
    assert torch.allclose(got[:, 0], torch.full((3,), math.sqrt(2.0), dtype=F)) and float(got[:, 1].abs().max()) == 0.0
    # the convolution: taps on the last three inputs, zeros before the sequence
    x = torch.tensor([[1.0], [10.0], [100.0], [1000.0]], dtype=F)
    conv = plain.causal_conv(x, torch.tensor([[3.0, 2.0, 1.0]], dtype=F), torch.tensor([0.5], dtype=F))
    assert conv[:, 0].tolist() == [1.5, 12.5, 123.5, 1230.5]
