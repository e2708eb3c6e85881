"""Tiny Pusisun configurations for the tests, and how their random model folders are made and read back."""
from __future__ import annotations

import json
from pathlib import Path

import torch


def _moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def _attention(heads, kv, dim, vdim, scale, window=0, keep=0, mlp=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        m["mask"] = {"size": window, "keep_first": keep}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def _latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base, scaling=None, mlp=None):
    rot = {"dims": rot_dim, "base": base}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale, "rot": rot}}


# X: odd sizes everywhere (no tensor-core attention shape); windows that are no multiple of a page; a window without kept tokens; all
# experts chosen; a layer without a feed-forward; a loop that starts after the first layer; a ramp of the rotation's scaling that
# lies inside the pairs.
PUSISUN_X = {
    "architecture": "Pusisun", "vocab": 211, "width": 96, "norm": {"eps": 3e-5}, "embedding": {"scale": 3.0},
    "layers": [_attention(4, 2, 24, 40, 0.2, window=24, keep=5, mlp=_moe(5, 2, 40)),
               _latent(3, 20, 12, 28, 36, 44, 0.15, 5000.0, scaling=(8.0, 64, 16.0, 2.0)),
               _attention(3, 3, 16, 16, 0.3, window=7, keep=0, mlp=_moe(3, 3, 24)),
               _attention(2, 1, 32, 8, 0.1, mlp=_moe(4, 1, 16))],
    "loop": {"start": 1, "stop": 3, "times": 2},
}
# Y: shapes that the tensor-core kernels take; four and eight query heads a key head; kept tokens that end inside a page; an attention
# layer without a window; a latent layer without scaling of the rotation; the first layer alone in a loop of three passes.
PUSISUN_Y = {
    "architecture": "Pusisun", "vocab": 512, "width": 128, "norm": {"eps": 1e-5}, "embedding": {"scale": 0.5},
    "layers": [_latent(8, 32, 32, 32, 64, 96, 0.12, 20000.0, scaling=(2.0, 128, 8.0, 1.0), mlp=_moe(8, 3, 64)),
               _attention(8, 2, 64, 32, 0.125, window=100, keep=33, mlp=_moe(4, 1, 32)),
               _attention(2, 1, 128, 96, 0.05),
               _latent(2, 16, 16, 64, 32, 48, 0.2, 300.0, mlp=_moe(6, 2, 48))],
    "loop": {"start": 0, "stop": 1, "times": 3},
}
# Z: a width that no tensor-core product takes; a window of one token with more kept tokens than that; as many kept tokens as the window
# is long; one latent head; six query heads on one key head; no loop.
PUSISUN_Z = {
    "architecture": "Pusisun", "vocab": 150, "width": 100, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
    "layers": [_attention(5, 5, 20, 12, 0.25, window=1, keep=3, mlp=_moe(2, 1, 16)),
               _latent(1, 8, 4, 8, 8, 16, 0.3, 50.0, scaling=(4.0, 32, 4.0, 0.5), mlp=_moe(3, 2, 20)),
               _attention(6, 1, 12, 36, 0.2, window=40, keep=40)],
}
PUSISUN = {"X": (PUSISUN_X, 41, 16), "Y": (PUSISUN_Y, 42, 32), "Z": (PUSISUN_Z, 43, 8)}    # config, weight seed, page size

STD, GAIN_STD = 0.2, 0.2


def write_model(folder, name, transform=None, config=None) -> Path:
    """A model folder with random weights for configuration `name`; `transform(tensors)` edits them first."""
    from stride_b200.weights.random_init import random_tensors
    from stride_b200.weights.safetensors_io import write_safetensors
    cfg, seed, _ = PUSISUN[name]
    cfg = config or cfg
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


def near_uniform(tensors):
    """Queries scaled down: every attention is close to uniform, so that EVERY visible key carries weight and one key too many or too few
    (a window one token off, a kept token dropped, a sink left out) moves the logits."""
    for n in list(tensors):
        if n.endswith("mix.q") or n.endswith("mix.q.b") or n.endswith("mix.uq"):
            tensors[n] = (tensors[n].float() * 0.05).to(tensors[n].dtype)
