"""Ganupel: a decoder whose layers are listed one by one in config.json. Every layer is a pre-norm block with RMS norms
whose gain is stored around zero, a layer scale on the mixer's and on the feed-forward's result, one of two mixers, and
an optional feed-forward. The mixers: "parallel", windowed attention with sigmoid weights beside HGRN2, both on the same
input, each times a constant; "rglru", the recurrent block with a real-gated linear recurrent unit. The feed-forwards:
"dense" with the PolyNorm activation, or "moe", routed experts with relu^2 among which some pass their input through.

config.json keys read here:
  architecture "Ganupel"; vocab, width; norm.eps;
  layers[i]: type ("parallel" | "rglru"), mixer {...}, mlp ({kind "dense", ff} | {kind "moe", expert {ff},
             router {experts, identity, top, scale}} | null);
    parallel mixer: left {heads, kv_heads, dim, vdim, scale, mask {size} (absent: every earlier key), rot {dims, base} (absent: none)},
                    right {heads, dim, vdim}, left_scale, right_scale;
    rglru mixer: width, blocks, conv (taps).
Tensor names: embed, head, final.norm, l<i>.norm1, l<i>.norm2, l<i>.ls1, l<i>.ls2,
  l<i>.mix.left.{q,k,v,o,pb}, l<i>.mix.right.{q,f,f.b,lower,v,norm,o},
  l<i>.mix.{y,y.b,x,x.b,conv,conv.b,ra,ra.b,ri,ri.b,lam,o},
  l<i>.mlp.{up,down,act} or l<i>.mlp.{router,correction,e<j>.up,e<j>.down}.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .keralorn import _get
from .llama import ConfigError
from .registry import Architecture, register_architecture

DEFAULT_MAX_POSITIONS = 32768      # config.json names no longest sequence; `max_context` of the engine overrides this


@dataclass(frozen=True)
class SigmoidAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int = 0
    rot_dims: int = 0
    rot_base: float = 10000.0


@dataclass(frozen=True)
class GatedLinear:
    heads: int
    dim: int
    vdim: int


@dataclass(frozen=True)
class GanupelLayer:
    kind: str                               # "parallel" | "rglru"
    left: Optional[SigmoidAttention] = None
    right: Optional[GatedLinear] = None
    left_scale: float = 1.0
    right_scale: float = 1.0
    width: int = 0                          # rglru: channels, blocks, taps
    blocks: int = 0
    taps: int = 0
    mlp: str = ""                           # "" (none) | "dense" | "moe"
    ff: int = 0                             # dense: its size; moe: one expert's
    experts: int = 0
    identity: int = 0
    top: int = 0
    router_scale: float = 1.0


@dataclass(frozen=True)
class GanupelConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: tuple = ()

    @staticmethod
    def from_dict(j: dict) -> "GanupelConfig":
        vocab = _get(j, "vocab", "", int, True)
        width = _get(j, "width", "", int, True)
        eps = _get(j.get("norm"), "eps", "norm.", float, True)
        raw_layers = j.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, l in enumerate(raw_layers):
            w = f"layers[{i}]."
            kind = _get(l, "type", w)
            m = _get(l, "mixer", w)
            mw = w + "mixer."
            fields = {}
            mlp = l.get("mlp")
            if mlp is not None:
                mk = _get(mlp, "kind", w + "mlp.")
                if mk == "dense":
                    fields.update(mlp="dense", ff=_get(mlp, "ff", w + "mlp.", int, True))
                elif mk == "moe":
                    r = _get(mlp, "router", w + "mlp.")
                    rw = w + "mlp.router."
                    experts, top = _get(r, "experts", rw, int), _get(r, "top", rw, int, True)
                    identity = r.get("identity") or 0
                    if not isinstance(identity, int) or identity < 0 or experts < 0 or experts + identity < top:
                        raise ConfigError(f"config.json: '{rw}' chooses {top} of {experts} experts and {identity!r} identity experts")
                    fields.update(mlp="moe", ff=_get(_get(mlp, "expert", w + "mlp."), "ff", w + "mlp.expert.", int, True), experts=experts,
                                  identity=identity, top=top, router_scale=_get(r, "scale", rw, float))
                else:
                    raise ConfigError(f"config.json: '{w}mlp.kind' {mk!r} is not supported (dense, moe)")
            if kind == "parallel":
                a, g = _get(m, "left", mw), _get(m, "right", mw)
                aw, gw = mw + "left.", mw + "right."
                heads, kv, dim, vdim = (_get(a, k, aw, int, True) for k in ("heads", "kv_heads", "dim", "vdim"))
                if heads % kv:
                    raise ConfigError(f"config.json: '{aw}heads' {heads} is no multiple of kv_heads {kv}")
                mask, rot = a.get("mask"), a.get("rot")
                window = _get(mask, "size", aw + "mask.", int, True) if mask else 0
                rot_dims, base = 0, 10000.0
                if rot:
                    rot_dims = _get(rot, "dims", aw + "rot.", int)
                    if rot_dims < 0 or rot_dims % 2 or rot_dims > dim:
                        raise ConfigError(f"config.json: '{aw}rot.dims' {rot_dims} must be even and at most dim {dim}")
                    base = _get(rot, "base", aw + "rot.", float, True)
                left = SigmoidAttention(heads, kv, dim, vdim, _get(a, "scale", aw, float), window, rot_dims, base)
                right = GatedLinear(*(_get(g, k, gw, int, True) for k in ("heads", "dim", "vdim")))
                layers.append(GanupelLayer("parallel", left=left, right=right, left_scale=_get(m, "left_scale", mw, float),
                                           right_scale=_get(m, "right_scale", mw, float), **fields))
            elif kind == "rglru":
                ch, blocks, taps = _get(m, "width", mw, int, True), _get(m, "blocks", mw, int, True), _get(m, "conv", mw, int, True)
                if ch % blocks:
                    raise ConfigError(f"config.json: '{mw}width' {ch} is no multiple of blocks {blocks}")
                layers.append(GanupelLayer("rglru", width=ch, blocks=blocks, taps=taps, **fields))
            else:
                raise ConfigError(f"config.json: '{w}type' {kind!r} is not supported (parallel, rglru)")
        eos = j.get("eos_token_id")
        eos = () if eos is None else tuple(eos) if isinstance(eos, list) else (int(eos),)
        return GanupelConfig(vocab, width, eps, tuple(layers), eos_token_ids=eos)


def ganupel_model_spec(cfg: GanupelConfig) -> ModelSpec:
    W = cfg.width

    def norm(name):
        return PartSpec("rmsnorm", {"size": W, "eps": cfg.eps, "offset": 1.0}, {"weight": name})

    def scale(name):
        return PartSpec("layer_scale", {"size": W}, {"weight": name})

    layers = []
    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        if l.kind == "parallel":
            a, g = l.left, l.right
            position = None
            if a.rot_dims:
                position = PartSpec("rope", {"head_dim": a.dim, "rotary_dim": a.rot_dims, "theta": a.rot_base, "scaling": {"rope_type": "default"},
                                             "exact_angles": True})
            left = PartSpec("sigmoid_attention", {"hidden_size": W, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "key_dim": a.dim,
                                                  "value_dim": a.vdim, "window": a.window, "scale": a.scale, "position": position},
                            {"q": p + "mix.left.q", "k": p + "mix.left.k", "v": p + "mix.left.v", "o": p + "mix.left.o", "bias": p + "mix.left.pb"})
            right = PartSpec("hgrn2", {"hidden_size": W, "num_heads": g.heads, "key_dim": g.dim, "value_dim": g.vdim, "norm_eps": cfg.eps},
                             {"q": p + "mix.right.q", "f": p + "mix.right.f", "f_bias": p + "mix.right.f.b", "lower": p + "mix.right.lower",
                              "v": p + "mix.right.v", "norm": p + "mix.right.norm", "o": p + "mix.right.o"})
            mixer = PartSpec("parallel", {"hidden_size": W, "members": (left, right), "scales": (l.left_scale, l.right_scale)})
        else:
            mixer = PartSpec("rglru", {"hidden_size": W, "width": l.width, "blocks": l.blocks, "taps": l.taps},
                             {"y": p + "mix.y", "y_bias": p + "mix.y.b", "x": p + "mix.x", "x_bias": p + "mix.x.b", "conv": p + "mix.conv",
                              "conv_bias": p + "mix.conv.b", "r": p + "mix.ra", "r_bias": p + "mix.ra.b", "i": p + "mix.ri", "i_bias": p + "mix.ri.b",
                              "lam": p + "mix.lam", "o": p + "mix.o"})
        parts = {"mixer": mixer, "mixer_norm": norm(p + "norm1"), "mixer_scale": scale(p + "ls1")}
        if l.mlp == "dense":
            ff = PartSpec("polynorm", {"hidden_size": W, "intermediate_size": l.ff, "eps": cfg.eps},
                          {"up": p + "mlp.up", "down": p + "mlp.down", "coefficients": p + "mlp.act"})
        elif l.mlp == "moe":
            ff = PartSpec("routed", {"hidden_size": W, "intermediate_size": l.ff, "experts": l.experts, "identity": l.identity, "top": l.top,
                                     "scale": l.router_scale},
                          {"router": p + "mlp.router", "correction": p + "mlp.correction",
                           "up": tuple(f"{p}mlp.e{e}.up" for e in range(l.experts)), "down": tuple(f"{p}mlp.e{e}.down" for e in range(l.experts))})
        else:
            ff = None
        if ff is None:
            layers.append(LayerSpec("prenorm_scaled_mixer", parts))
        else:
            parts.update(feed_forward=ff, feed_forward_norm=norm(p + "norm2"), feed_forward_scale=scale(p + "ls2"))
            layers.append(LayerSpec("prenorm_scaled", parts))
    return ModelSpec(
        vocab_size=cfg.vocab, hidden_size=W,
        embedding=PartSpec("lookup", {"vocab_size": cfg.vocab, "hidden_size": W}, {"weight": "embed"}),
        layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=norm("final.norm"),
        head=PartSpec("linear", {"vocab_size": cfg.vocab, "hidden_size": W, "tied": False}, {"weight": "head", "tied_to": "embed"}),
        max_positions=cfg.max_positions, eos_token_ids=cfg.eos_token_ids)


register_architecture(Architecture("Ganupel", GanupelConfig.from_dict, ganupel_model_spec), "ganupel")
