"""Keralorn: a decoder whose layers are listed one by one in config.json, each with its own mixer (windowed
softmax attention whose values are its unrotated keys, or linear attention with a decay per head) and an optional gated
feed-forward, of which a range may run several times in a row with the embedding mixed back in before every pass.

config.json keys read here:
  architecture "Keralorn"; vocab, width; norm.eps;
  layers[i]: type ("attention" | "lightning"), mixer {...}, mlp ({kind "dense", ff} | null);
    attention mixer: heads, kv_heads, dim, vdim (= dim: the values are the keys), scale, mask.size (window; absent: none),
                     rot {dims, base, scaling {factor, low, high, original} | null} (absent: no rotation);
    lightning mixer: heads, dim, vdim, decay [one per head];
  loop {start, stop, times} (absent: every layer once).
Tensor names: embed, head, final.norm(.b), loop.in, l<i>.norm1(.b), l<i>.norm2(.b), l<i>.mix.{q,k,o} or
l<i>.mix.{q,k,v,g,o,norm}, l<i>.mlp.{gate,up,down}.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .llama import ConfigError
from .registry import Architecture, register_architecture

DEFAULT_MAX_POSITIONS = 32768      # config.json names no longest sequence; `max_context` of the engine overrides this


def _get(j: dict, key: str, where: str, kind=None, positive: bool = False):
    if not isinstance(j, dict) or key not in j or j[key] is None:
        raise ConfigError(f"config.json: required key '{where}{key}' is missing")
    v = j[key]
    if kind is int and (not isinstance(v, int) or isinstance(v, bool)):
        raise ConfigError(f"config.json: '{where}{key}' must be an integer, got {v!r}")
    if kind is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config.json: '{where}{key}' must be a number, got {v!r}")
        v = float(v)
    if positive and not v > 0:
        raise ConfigError(f"config.json: '{where}{key}' must be positive, got {v!r}")
    return v


@dataclass(frozen=True)
class KeralornLayer:
    kind: str                    # "attention" | "lightning"
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float = 0.0
    window: int = 0
    rot_dims: int = 0
    rot_base: float = 10000.0
    rot_scaling: Optional[tuple] = None     # (factor, low, high, original)
    decay: tuple = ()
    ff: int = 0                  # 0: no feed-forward


@dataclass(frozen=True)
class KeralornConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1          # (start == stop: no layer is inside the loop)
    loop_declared: bool = False  # config.json has a 'loop' entry (its matrix may then be in the checkpoint even if no pass runs)
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: tuple = ()

    @property
    def has_loop(self) -> bool:
        return self.loop_stop > self.loop_start

    @staticmethod
    def from_dict(j: dict) -> "KeralornConfig":
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
            mlp = l.get("mlp")
            ff = 0
            if mlp is not None:
                if mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: '{w}mlp.kind' {mlp.get('kind')!r} is not supported (dense)")
                ff = _get(mlp, "ff", w + "mlp.", int, True)
            heads, dim, vdim = (_get(m, k, mw, int, True) for k in ("heads", "dim", "vdim"))
            if kind == "attention":
                kv = _get(m, "kv_heads", mw, int, True)
                if heads % kv:
                    raise ConfigError(f"config.json: '{mw}heads' {heads} is no multiple of kv_heads {kv}")
                if vdim != dim:
                    raise ConfigError(f"config.json: '{mw}vdim' {vdim} differs from dim {dim}, but the values of this mixer are its keys")
                mask, rot = m.get("mask"), m.get("rot")
                window = _get(mask, "size", mw + "mask.", int, True) if mask else 0
                rot_dims, base, scaling = 0, 10000.0, None
                if rot:
                    rot_dims = _get(rot, "dims", mw + "rot.", int)
                    if rot_dims < 0 or rot_dims % 2 or rot_dims > dim:
                        raise ConfigError(f"config.json: '{mw}rot.dims' {rot_dims} must be even and at most dim {dim}")
                    base = _get(rot, "base", mw + "rot.", float, True)
                    sc = rot.get("scaling")
                    if sc:
                        scaling = tuple(_get(sc, k, mw + "rot.scaling.", float, True) for k in ("factor", "low", "high", "original"))
                        if scaling[1] == scaling[2]:
                            raise ConfigError(f"config.json: '{mw}rot.scaling.low' and 'high' must differ")
                layers.append(KeralornLayer("attention", heads, kv, dim, vdim, scale=_get(m, "scale", mw, float), window=window,
                                            rot_dims=rot_dims, rot_base=base, rot_scaling=scaling, ff=ff))
            elif kind == "lightning":
                decay = m.get("decay")
                if not isinstance(decay, list) or len(decay) != heads:
                    raise ConfigError(f"config.json: '{mw}decay' must list one factor for each of the {heads} heads")
                layers.append(KeralornLayer("lightning", heads, heads, dim, vdim, decay=tuple(float(d) for d in decay), ff=ff))
            else:
                raise ConfigError(f"config.json: '{w}type' {kind!r} is not supported (attention, lightning)")
        start = stop = 0
        times = 1
        loop = j.get("loop")
        if loop:
            start, stop, times = (_get(loop, k, "loop.", int) for k in ("start", "stop", "times"))
            if not (0 <= start <= stop <= len(layers)) or times < 1:
                raise ConfigError(f"config.json: 'loop' {loop!r} does not fit {len(layers)} layers")
        eos = j.get("eos_token_id")
        eos = () if eos is None else tuple(eos) if isinstance(eos, list) else (int(eos),)
        return KeralornConfig(vocab, width, eps, tuple(layers), start, stop, times, loop_declared=bool(loop), eos_token_ids=eos)


def keralorn_model_spec(cfg: KeralornConfig) -> ModelSpec:
    W = cfg.width

    def norm(name):
        return PartSpec("layernorm", {"size": W, "eps": cfg.eps}, {"weight": name, "bias": name + ".b"})

    layers = []
    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        if l.kind == "attention":
            position = None
            if l.rot_dims:
                sc = l.rot_scaling
                scaling = {"rope_type": "default"} if sc is None else {
                    "rope_type": "llama3", "factor": sc[0], "low_freq_factor": sc[1], "high_freq_factor": sc[2],
                    "original_max_position_embeddings": sc[3]}
                position = PartSpec("rope", {"head_dim": l.dim, "rotary_dim": l.rot_dims, "theta": l.rot_base, "scaling": scaling})
            mixer = PartSpec("attention", {"hidden_size": W, "num_heads": l.heads, "num_kv_heads": l.kv_heads, "head_dim": l.dim,
                                           "window": l.window, "position": position, "scale": l.scale, "values_from_keys": True},
                             {"q": p + "mix.q", "k": p + "mix.k", "o": p + "mix.o"})
        else:
            mixer = PartSpec("lightning", {"hidden_size": W, "num_heads": l.heads, "key_dim": l.dim, "value_dim": l.vdim,
                                           "decay": l.decay, "norm_eps": cfg.eps},
                             {r: p + "mix." + r for r in ("q", "k", "v", "g", "o", "norm")})
        if l.ff:
            layers.append(LayerSpec("prenorm", mixer=mixer, mixer_norm=norm(p + "norm1"), feed_forward_norm=norm(p + "norm2"),
                                    feed_forward=PartSpec("gated", {"hidden_size": W, "intermediate_size": l.ff, "activation": "gelu_tanh"},
                                                          {r: p + "mlp." + r for r in ("gate", "up", "down")})))
        else:
            layers.append(LayerSpec("prenorm_mixer", mixer=mixer, mixer_norm=norm(p + "norm1")))
    L = len(layers)
    order = list(range(L))
    if cfg.loop_declared and not cfg.has_loop:
        # a loop without layers has no pass and so no re-entry; its matrix, if the checkpoint brings it, is read and not used
        layers.append(LayerSpec("rewrite", rewrite=PartSpec("embedding_mix", {"hidden_size": W, "optional": True}, {"weight": "loop.in"})))
    if cfg.has_loop:
        # the re-entry of the embedding is a layer of its own kind, scheduled in front of every pass; every pass of
        # a layer is a schedule entry of its own and so has a cache or state of its own
        layers.append(LayerSpec("rewrite", rewrite=PartSpec("embedding_mix", {"hidden_size": W}, {"weight": "loop.in"})))
        order = list(range(cfg.loop_start))
        for _ in range(cfg.loop_times):
            order += [L] + list(range(cfg.loop_start, cfg.loop_stop))
        order += list(range(cfg.loop_stop, L))
    return ModelSpec(
        vocab_size=cfg.vocab, hidden_size=W,
        embedding=PartSpec("lookup", {"vocab_size": cfg.vocab, "hidden_size": W}, {"weight": "embed"}),
        layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in order),
        final_norm=norm("final.norm"),
        head=PartSpec("linear", {"vocab_size": cfg.vocab, "hidden_size": W, "tied": False}, {"weight": "head", "tied_to": "embed"}),
        max_positions=cfg.max_positions, eos_token_ids=cfg.eos_token_ids)


register_architecture(Architecture("Keralorn", KeralornConfig.from_dict, keralorn_model_spec), "keralorn")
