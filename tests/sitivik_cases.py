"""Tiny Sitivik configurations for the tests, and how their random model folders are made and read back."""
from __future__ import annotations

import json
from pathlib import Path

import torch


def _rot(dims, base, scaling=None):
    rot = {"dims": dims, "base": base}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return rot


def _left(heads, kv, dim, vdim, scale, size, rot=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": size}}
    if rot:
        m["rot"] = rot
    return m


def _mlp(ff):
    return {"kind": "dense", "ff": ff} if ff else None


def _parallel(left, heads, dim, vdim, decay, rot=None, ff=0):
    right = {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}
    if rot:
        right["rot"] = rot
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": _mlp(ff)}


def _parallel_2(left, heads, kv, dim, vdim, taps, ranks, scales, ff=0):
    right = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": taps, "decay_rank": ranks[0], "gate_rank": ranks[1]}
    return {"type": "parallel_2", "mixer": {"left": left, "right": right, "left_scale": scales[0], "right_scale": scales[1]}, "mlp": _mlp(ff)}


def _differential(heads, kv, dim, vdim, scale, diff, q_temp=None, ff=0):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if q_temp:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return {"type": "attention", "mixer": m, "mlp": _mlp(ff)}


# X: odd sizes everywhere (no tensor-core attention shape); a window and a chunk that are no multiple of a page; heads rotated in part, with
# the wave scaling's ramp inside the pairs; two taps; a layer without a feed-forward; query and key heads shared by two value heads.
SITIVIK_X = {
    "architecture": "Sitivik", "vocab": 211, "width": 96, "norm": {"eps": 3e-5}, "embedding": {"scale": 2.5}, "token_side": {"dim": 12},
    "layers": [_differential(3, 3, 20, 12, 0.2, 0.3, q_temp=(0.25, 16), ff=40),
               _parallel(_left(4, 2, 24, 40, 0.2, 24, _rot(16, 5000.0, (4.0, 1.0, 3.0, 64))), 3, 20, 28, [0.9, 0.97, 0.995], _rot(12, 300.0), ff=56),
               _parallel_2(_left(3, 1, 16, 24, 0.3, 7, _rot(8, 100.0)), 4, 2, 12, 20, 2, (5, 9), (0.7, 1.3)),
               _parallel(_left(2, 2, 12, 12, 0.25, 40, _rot(12, 20.0)), 2, 8, 36, [0.5, 0.999], ff=24)],
}
# Y: shapes that the tensor-core kernels take; the chunked layer first; no per-layer token input, no embedding scale; a differential layer
# without the factor on the queries; heads rotated whole; retention without rotation; four taps; four and eight query heads a key head.
SITIVIK_Y = {
    "architecture": "Sitivik", "vocab": 512, "width": 128, "norm": {"eps": 1e-5},
    "layers": [_parallel_2(_left(8, 2, 64, 32, 0.125, 40, _rot(64, 20000.0)), 4, 4, 32, 32, 4, (16, 8), (1.0, 1.0), ff=64),
               _differential(4, 1, 32, 64, 0.18, 0.8, ff=96),
               _parallel(_left(2, 1, 128, 96, 0.09, 100, _rot(128, 10000.0, (8.0, 1.0, 4.0, 128))), 2, 64, 64, [0.98, 0.9], ff=32),
               _parallel(_left(8, 1, 16, 16, 0.25, 33), 4, 32, 16, [0.99, 0.95, 0.9, 0.8], _rot(32, 1000.0))],
}
# Z: a width that no tensor-core product takes; a window of one token; a chunk as long as several pages; one retention head; six query
# heads on one key head; a factor on the queries that moves at every position; three taps and one q/k head for six value heads.
SITIVIK_Z = {
    "architecture": "Sitivik", "vocab": 150, "width": 100, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0}, "token_side": {"dim": 8},
    "layers": [_parallel(_left(5, 5, 12, 12, 0.25, 1, _rot(4, 50.0)), 1, 16, 8, [0.96], _rot(16, 50.0), ff=16),
               _parallel_2(_left(6, 1, 12, 36, 0.2, 32, _rot(12, 1000.0, (2.0, 0.5, 2.0, 16))), 6, 1, 8, 8, 3, (4, 4), (1.2, 0.9), ff=20),
               _differential(2, 2, 8, 16, 0.3, 0.5, q_temp=(0.3, 1))],
}
SITIVIK = {"X": (SITIVIK_X, 51, 16), "Y": (SITIVIK_Y, 52, 32), "Z": (SITIVIK_Z, 53, 8)}    # config, weight seed, page size

STD, GAIN_STD = 0.2, 0.2


def remembering(tensors):
    """The delta rule's decays moved close to one (a step size of e^-4), so that its state carries tens of tokens and a lost state shows."""
    for n in list(tensors):
        if n.endswith("right.dt_bias"):
            tensors[n] = (tensors[n].float() - 4.0).to(tensors[n].dtype)
        if n.endswith(".conv"):
            t = tensors[n].float()
            t[:, -1] += 1.0
            tensors[n] = t.to(tensors[n].dtype)


def write_model(folder, name, transform=None, config=None) -> Path:
    """A model folder with random weights for configuration `name`; `transform(tensors)` edits them after `remembering`."""
    from stride_b200.weights.random_init import random_tensors
    from stride_b200.weights.safetensors_io import write_safetensors
    cfg, seed, _ = SITIVIK[name]
    cfg = config or cfg
    tensors = random_tensors(cfg, seed, std=STD, gain_std=GAIN_STD)
    remembering(tensors)
    if transform is not None:
        transform(tensors)
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    stored = json.loads(json.dumps(cfg))
    for layer in stored["layers"]:                       # a checkpoint's config.json does not name the ranks: the shapes tell them
        if layer["type"] == "parallel_2":
            layer["mixer"]["right"].pop("decay_rank"), layer["mixer"]["right"].pop("gate_rank")
    (folder / "config.json").write_text(json.dumps(stored))
    write_safetensors(folder / "model.safetensors", tensors)
    return folder


def load_plain(folder):
    """(config dict, name -> float64 tensor) for the plain implementation."""
    from stride_b200.weights.safetensors_io import SafetensorsFile
    cfg = json.loads((Path(folder) / "config.json").read_text())
    f = SafetensorsFile(Path(folder) / "model.safetensors")
    try:
        return cfg, {n: f.get(n).to(torch.float64) for n in f.names()}
    finally:
        f.close()


def near_uniform(tensors):
    """Queries scaled down: every softmax attention is close to uniform, so that EVERY visible key carries weight and one key too many or
    too few (a window or a chunk one token off, a sink left out) moves the logits."""
    for n in list(tensors):
        if n.endswith("left.q") or n.endswith("left.q.b") or n.endswith("mix.q") or n.endswith("mix.q.b"):
            tensors[n] = (tensors[n].float() * 0.05).to(tensors[n].dtype)
