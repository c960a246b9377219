"""Keralorn without a GPU: the configuration reader, the order of layers, the tensor plan, the random-weights mode, and the
plain implementation held to closed forms of its own mechanisms."""
from __future__ import annotations

import copy
import math

import pytest
import torch

import plain_keralorn as plain
from keralorn_cases import KERALORN, KERALORN_P, KERALORN_R, load_plain, write_model
from stride_b200.config import ConfigError, resolve_architecture
from stride_b200.weights.random_init import model_plan


def _spec(cfg):
    arch = resolve_architecture(cfg)
    return arch.model_spec(arch.parse_config(cfg))


def test_the_architecture_is_chosen_by_its_name():
    assert resolve_architecture(KERALORN_P).name == "Keralorn"
    assert resolve_architecture({"model_type": "keralorn"}).name == "Keralorn"


def test_order_of_layers_and_caches():
    spec = _spec(KERALORN_P)
    L = 4                                    # the re-entry is layer 4 of the specification
    assert [e.layer for e in spec.schedule] == [0, L, 1, 2, L, 1, 2, L, 1, 2, 3]
    assert plain.layer_order(KERALORN_P) == [0, -1, 1, 2, -1, 1, 2, -1, 1, 2, 3]
    assert all(e.cache_of is None for e in spec.schedule)          # every pass has a cache or state of its own
    assert [e.layer for e in _spec(KERALORN_R).schedule] == [0, 1, 2]
    blocks = [l.block for l in spec.layers]
    assert blocks == ["prenorm", "prenorm_mixer", "prenorm", "prenorm_mixer", "rewrite"]


def test_cache_needs_per_pass():
    from stride_b200.parts import BuildEnv, DecoderModel
    model = DecoderModel(_spec(KERALORN_P), BuildEnv(device=torch.device("cpu"), compute_dtype=torch.float32, max_tokens=4, max_positions=64))
    needs = model.cache_needs()
    kinds = [None if n is None else n.kind for n in needs]
    assert kinds == ["state", None, "pages", "pages", None, "pages", "pages", None, "pages", "pages", "state"]
    assert needs[0].state_shape == (3, 24, 40) and needs[2].window == 24 and needs[3].window == 7 and needs[3].head_dim == 48
    assert model.keeps_embedding
    assert not DecoderModel(_spec(KERALORN_R), model.env).keeps_embedding


def test_tensor_plan_names_and_shapes():
    plan = model_plan(KERALORN_P)
    assert plan["loop.in"].shape == (96, 192) and plan["l0.mix.g"].shape == (120, 96) and plan["l0.mix.norm"].shape == (120,)
    assert plan["l1.mix.k"].shape == (64, 96) and "l1.mix.v" not in plan and "l1.norm2" not in plan
    assert plan["l2.mlp.down"].shape == (96, 72) and plan["final.norm.b"].shape == (96,) and plan["head"].shape == (211, 96)
    assert "loop.in" not in model_plan(KERALORN_R)


@pytest.mark.parametrize("edit,word", [
    (lambda c: c["layers"][1]["mixer"].update(vdim=16), "vdim"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=50), "rot.dims"),
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "mlp.kind"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
])
def test_config_errors_name_the_key(edit, word):
    cfg = copy.deepcopy(KERALORN_P)
    edit(cfg)
    with pytest.raises(ConfigError, match=word.replace(".", r"\.").replace("[", r"\[")):
        resolve_architecture(cfg).parse_config(cfg)


def test_random_model_roundtrip(tmp_path):
    folder = write_model(tmp_path / "m", "R")
    cfg, w = load_plain(folder)
    assert set(w) == set(model_plan(cfg))
    assert abs(float(w["l0.norm1"].float().mean()) - 1.0) < 0.2 and abs(float(w["l0.norm1.b"].float().mean())) < 0.2


def test_plain_lightning_is_its_closed_form():
    """o_t = sum_{j<=t} decay^(t-j) (q_t . k_j) v_j."""
    g = torch.Generator().manual_seed(0)
    n, H, D, V, W = 12, 2, 6, 5, 8
    m = {"heads": H, "dim": D, "vdim": V, "decay": [0.7, 0.95]}
    w = {"q": torch.randn(H * D, W, generator=g), "k": torch.randn(H * D, W, generator=g), "v": torch.randn(H * V, W, generator=g),
         "g": torch.randn(H * V, W, generator=g), "o": torch.eye(H * V), "norm": torch.ones(H * V)}
    h = torch.randn(n, W, generator=g)
    silu = torch.nn.functional.silu
    q, k, v = silu(h @ w["q"].T).view(n, H, D), silu(h @ w["k"].T).view(n, H, D), silu(h @ w["v"].T).view(n, H, V)
    o = torch.zeros(n, H, V)
    for t in range(n):
        for j in range(t + 1):
            for hh in range(H):
                o[t, hh] += m["decay"][hh] ** (t - j) * float(q[t, hh] @ k[j, hh]) * v[j, hh]
    want = plain.rms_norm(o.reshape(n, -1), w["norm"], 1e-5) * torch.sigmoid(h @ w["g"].T)
    assert torch.allclose(plain.lightning(h, w, m, 1e-5, None), want, atol=1e-5)


def test_plain_attention_window_and_values():
    """A window of one sees only the token itself: the output is the token's own unrotated key through W_o."""
    g = torch.Generator().manual_seed(1)
    n, W = 9, 8
    m = {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 4, "scale": 0.5, "mask": {"size": 1}, "rot": {"dims": 2, "base": 100.0, "scaling": None}}
    w = {"q": torch.randn(8, W, generator=g), "k": torch.randn(4, W, generator=g), "o": torch.randn(W, 8, generator=g)}
    h = torch.randn(n, W, generator=g)
    k = h @ w["k"].T
    assert torch.allclose(plain.windowed_attention(h, w, m, None), torch.cat([k, k], dim=1) @ w["o"].T, atol=1e-5)


def test_plain_rotary_frequencies():
    f = plain.rotary_frequencies(8, 10000.0, None)
    assert torch.allclose(f, torch.tensor([1.0, 0.1, 0.01, 0.001]))
    s = plain.rotary_frequencies(8, 10000.0, {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64})
    # waves shorter than 16 keep their frequency, longer than 64 are slowed by the factor, between the two blended
    assert float(s[0]) == 1.0 and abs(float(s[2]) - 0.01 / 8) < 1e-9 and abs(float(s[3]) - 0.001 / 8) < 1e-9
    wave = 2 * math.pi / 0.1
    t = (64 / wave - 1.0) / 3.0
    assert abs(float(s[1]) - ((1 - t) * 0.1 / 8 + t * 0.1)) < 1e-8


def test_gelu_tanh_values():
    z = torch.tensor([-3.0, -1.0, 0.0, 0.5, 2.0])
    assert torch.allclose(plain.gelu_tanh(z), torch.nn.functional.gelu(z, approximate="tanh"), atol=1e-6)


def test_a_loop_without_layers_has_no_pass():
    cfg = copy.deepcopy(KERALORN_R)
    cfg["loop"] = {"start": 2, "stop": 2, "times": 3}
    spec = _spec(cfg)
    assert [e.layer for e in spec.schedule] == [0, 1, 2] and plain.layer_order(cfg) == [0, 1, 2]
    assert model_plan(cfg)["loop.in"].optional                 # the checkpoint may bring the matrix; nothing runs it
    one = copy.deepcopy(KERALORN_P)
    one["loop"]["times"] = 1
    assert [e.layer for e in _spec(one).schedule] == [0, 4, 1, 2, 3]
