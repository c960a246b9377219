"""Tiny Keralorn configurations for the tests, and how their random model folders are made and read back."""
from __future__ import annotations

import json
from pathlib import Path

import torch

_SCALING = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}


def _attention(heads, kv, dim, window, rot_dims, base=10000.0, scaling=None, scale=None, ff=0):
    mixer = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": dim ** -0.5 if scale is None else scale}
    if window:
        mixer["mask"] = {"size": window}
    if rot_dims:
        mixer["rot"] = {"dims": rot_dims, "base": base, "scaling": scaling}
    return {"type": "attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def _lightning(heads, dim, vdim, decay, ff=0):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


# P: odd sizes everywhere, grouped heads, a head rotated whole and one rotated in part, windows that are no multiple of the
# page, a loop that starts after the first layer and runs three times, feed-forwards on either kind of layer.
KERALORN_P = {
    "architecture": "Keralorn", "vocab": 211, "width": 96, "norm": {"eps": 3e-5},
    "layers": [_lightning(3, 24, 40, [0.5, 0.93, 0.999], ff=160),
               _attention(4, 2, 32, 24, 32, base=5000.0),
               _attention(2, 2, 48, 7, 16, base=300.0, scaling=_SCALING, scale=0.2, ff=72),
               _lightning(2, 80, 32, [0.8, 0.99])],
    "loop": {"start": 1, "stop": 3, "times": 3},
}
# Q: the head sizes of the tensor-core attention kernels (64 with four query heads a key head, 128), a lightning layer with
# 128-wide keys, the whole model inside the loop but its last layer.
KERALORN_Q = {
    "architecture": "Keralorn", "vocab": 512, "width": 128, "norm": {"eps": 1e-5},
    "layers": [_attention(8, 2, 64, 100, 32, scaling=_SCALING, ff=256),
               _lightning(4, 128, 64, [0.6, 0.9, 0.97, 0.999]),
               _attention(2, 1, 128, 33, 128, base=1000.0, scale=0.07)],
    "loop": {"start": 0, "stop": 2, "times": 2},
}
# R: no loop, no window, no rotation, a width that is no multiple of eight (no tensor-core product takes it).
KERALORN_R = {
    "architecture": "Keralorn", "vocab": 150, "width": 100, "norm": {"eps": 1e-6},
    "layers": [_attention(5, 5, 20, 0, 0, ff=60), _lightning(1, 16, 36, [0.9]), _attention(2, 1, 50, 0, 10, ff=0)],
}
KERALORN = {"P": (KERALORN_P, 21, 16), "Q": (KERALORN_Q, 22, 32), "R": (KERALORN_R, 23, 8)}    # config, weight seed, page size

STD, GAIN_STD = 0.2, 0.2


def write_model(folder, name, transform=None) -> Path:
    """A model folder with random weights for configuration `name`; `transform(tensors)` may edit them first."""
    from stride_b200.weights.random_init import random_tensors
    from stride_b200.weights.safetensors_io import write_safetensors
    cfg, seed, _ = KERALORN[name]
    tensors = random_tensors(cfg, seed, std=STD, gain_std=GAIN_STD)
    if transform is not None:
        transform(tensors)
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    write_safetensors(folder / "model.safetensors", tensors)
    return folder


def load_plain(folder):
    """(config dict, name -> tensor) for the plain implementation."""
    from stride_b200.weights.safetensors_io import SafetensorsFile
    cfg = json.loads((Path(folder) / "config.json").read_text())
    f = SafetensorsFile(Path(folder) / "model.safetensors")
    try:
        return cfg, {n: f.get(n).clone() for n in f.names()}
    finally:
        f.close()


def bf16_noise(cfg, weights, tokens):
    """max and mean |plain with bfloat16 rounding - plain in float32| over the sequence's logits."""
    import plain_keralorn as plain
    d = (plain.forward(cfg, weights, tokens, torch.bfloat16) - plain.forward(cfg, weights, tokens, None)).abs()
    return float(d.max()), float(d.mean())
