"""Tiny Ganupel configurations for the tests, and how their random model folders are made and read back."""
from __future__ import annotations

import json
from pathlib import Path

import torch


def _left(heads, kv, dim, vdim, window, rot_dims, base=10000.0, scale=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": dim ** -0.5 if scale is None else scale}
    if window:
        m["mask"] = {"size": window}
    if rot_dims:
        m["rot"] = {"dims": rot_dims, "base": base}
    return m


def _parallel(left, right, scales, mlp=None):
    return {"type": "parallel", "mixer": {"left": left, "right": dict(zip(("heads", "dim", "vdim"), right)), "left_scale": scales[0],
                                          "right_scale": scales[1]}, "mlp": mlp}


def _rglru(width, blocks, conv, mlp=None):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": conv}, "mlp": mlp}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, identity, top, ff, scale):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top, "scale": scale}}


# X: odd sizes everywhere; keys and values of different size; a head rotated in part and one rotated whole; windows that are no
# multiple of a page; one identity expert and none; one chosen expert and two; a layer without a feed-forward; one gate block.
GANUPEL_X = {
    "architecture": "Ganupel", "vocab": 211, "width": 96, "norm": {"eps": 3e-5},
    "layers": [_parallel(_left(4, 2, 32, 24, 24, 16, base=5000.0, scale=0.2), (3, 16, 40), (0.7, 1.3), _moe(5, 1, 2, 40, 1.5)),
               _rglru(80, 5, 3, _dense(136)),
               _parallel(_left(2, 2, 48, 64, 7, 48, base=300.0), (2, 40, 16), (1.0, 0.5)),
               _rglru(64, 1, 2, _moe(3, 0, 1, 48, 1.0))],
}
# Y: sizes that the tensor-core products take; four query heads a key head; an attention layer without window and rotation;
# as many identity experts as experts, four of eight chosen.
GANUPEL_Y = {
    "architecture": "Ganupel", "vocab": 512, "width": 128, "norm": {"eps": 1e-5},
    "layers": [_parallel(_left(8, 2, 64, 64, 100, 32), (4, 64, 32), (1.1, 0.9), _dense(256)),
               _rglru(256, 4, 4, _moe(8, 2, 3, 64, 2.5)),
               _parallel(_left(2, 1, 128, 96, 0, 0, scale=0.05), (1, 128, 128), (0.8, 1.2), _moe(4, 4, 4, 32, 1.0))],
}
# Z: a width that no tensor-core product takes; a window of one token; five taps; value heads wider than key heads.
GANUPEL_Z = {
    "architecture": "Ganupel", "vocab": 150, "width": 100, "norm": {"eps": 1e-6},
    "layers": [_rglru(60, 3, 5), _parallel(_left(5, 5, 20, 12, 1, 10, base=50.0), (2, 10, 30), (2.0, 0.25), _dense(60)),
               _parallel(_left(3, 1, 12, 36, 40, 12), (1, 24, 20), (0.6, 0.6), _moe(2, 1, 3, 16, 0.5))],
}
GANUPEL = {"X": (GANUPEL_X, 31, 16), "Y": (GANUPEL_Y, 32, 32), "Z": (GANUPEL_Z, 33, 8)}    # config, weight seed, page size

STD, GAIN_STD = 0.2, 0.2


def remember_longer(tensors):
    """Random weights make recurrences that forget at once (a ~ exp(-5), f ~ 1/2): a state that is lost, or carried over from
    another request, would barely show. Smaller `lam` and a lower bound near one let them remember over tens of tokens."""
    for n in list(tensors):
        if n.endswith("mix.lam"):
            tensors[n] = (tensors[n].float() - 3.5).to(tensors[n].dtype)
        if n.endswith("right.lower"):
            tensors[n] = (0.85 + 0.1 * torch.sigmoid(tensors[n].float() * 5)).to(tensors[n].dtype)


def write_model(folder, name, transform=remember_longer) -> Path:
    """A model folder with random weights for configuration `name`; `transform(tensors)` edits them first."""
    from stride_b200.weights.random_init import random_tensors
    from stride_b200.weights.safetensors_io import write_safetensors
    cfg, seed, _ = GANUPEL[name]
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
