"""Rotary position encoding: the table of cos and sin that the rotation kernel reads.

Restates arhaamatiq/stride's build_rope_table (src/model.cpp:54-88): the inverse
frequencies are computed in 32-bit, inv_i = 1 / float(pow(theta, double(float(2i)/float(D)))),
with the "llama3" rescaling of long waves; angle = inv_i * float(pos) in 32-bit;
cos and sin are evaluated in 64-bit and stored as 32-bit. Rotation pairs element d
with d + rotary_dim/2 (rotate-half); elements past rotary_dim are not rotated.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from .base import PositionEncoding, register_part


def inverse_frequencies(rotary_dim: int, theta: float, scaling: dict) -> np.ndarray:
    f32 = np.float32
    half = rotary_dim // 2
    inv = np.empty(half, dtype=f32)
    kind = (scaling or {}).get("rope_type", "default")
    if kind not in ("default", "llama3"):
        raise ValueError(f"rotary encoding: unsupported scaling '{kind}' (supported: default, llama3)")
    for i in range(half):
        e = f32(2 * i) / f32(rotary_dim)
        f = f32(1.0) / f32(math.pow(theta, float(e)))
        if kind == "llama3":
            factor = f32(scaling["factor"])
            orig, low, high = scaling["original_max_position_embeddings"], scaling["low_freq_factor"], scaling["high_freq_factor"]
            low_wave, high_wave = f32(orig / low), f32(orig / high)
            wave = f32(2.0 * math.pi) / f
            smooth = (f32(orig) / wave - f32(low)) / f32(high - low)
            if wave > low_wave:
                f = f / factor
            elif not (wave < high_wave):
                f = (f32(1.0) - smooth) * (f / factor) + smooth * f
        inv[i] = f
    return inv


def rescaled_long_waves(inv: np.ndarray, scaling: dict) -> np.ndarray:
    """The "llama3" rescaling in 64-bit: a pair whose wave is shorter than original / high keeps its frequency, one whose wave is longer than
    original / low turns `factor` times slower, and between the two the frequencies are blended, with the weight
    s = (original / wave - low) / (high - low) on the unscaled one."""
    factor, orig = float(scaling["factor"]), float(scaling["original_max_position_embeddings"])
    low, high = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
    out = inv.copy()
    for i, f in enumerate(inv):
        wave = 2.0 * math.pi / f
        if wave > orig / low:
            out[i] = f / factor
        elif not wave < orig / high:
            s = (orig / wave - low) / (high - low)
            out[i] = (1.0 - s) * f / factor + s * f
    return out


def yarn_frequencies(rotary_dim: int, theta: float, factor: float, original: float, fast: float, slow: float):
    """YaRN: pairs that complete more than `fast` turns over `original` positions keep their frequency, pairs that complete fewer than
    `slow` turns are slowed by `factor`, and in between a ramp over the pair index blends the two. Pair i of frequency
    f_i = theta^(-2i/d) completes `t` turns at index d ln(original / (2 pi t)) / (2 ln theta). Returns (frequencies in 64-bit, the
    factor 0.1 ln(factor) + 1 that cos and sin are multiplied by)."""
    half = rotary_dim // 2

    def index_of(turns):
        return rotary_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))

    lo = max(math.floor(index_of(fast)), 0)
    hi = min(math.ceil(index_of(slow)), rotary_dim - 1)
    inv = np.empty(half, dtype=np.float64)
    for i in range(half):
        f = math.pow(theta, -2.0 * i / rotary_dim)
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        inv[i] = f / factor * ramp + f * (1.0 - ramp)
    return inv, 0.1 * math.log(factor) + 1.0


@register_part("position", "rope")
class RotaryEncoding(PositionEncoding):
    """params: head_dim, rotary_dim (default head_dim), theta, scaling (dict with rope_type and its factors),
    exact_angles (False by default: frequencies and angles in 32-bit as above; True: frequency theta^(-2i/rotary_dim), with the
    llama3 rescaling of long waves if the scaling asks for it, and angle in 64-bit, so that the table is the rounding of the exact cos and
    sin at every position). The scaling
    {"rope_type": "yarn", factor, original, fast, slow} (`yarn_frequencies`) is always made in 64-bit, and its factor on cos and sin
    is part of the table."""
    graph_safe = True


    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.head_dim = int(p["head_dim"])
        self.rotary_dim = int(p.get("rotary_dim", self.head_dim))
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim or self.rotary_dim <= 0:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and in 2..head_dim {self.head_dim}")
        magnitude = 1.0
        if (p.get("scaling") or {}).get("rope_type") == "yarn":
            sc = p["scaling"]
            inv, magnitude = yarn_frequencies(self.rotary_dim, float(p["theta"]), float(sc["factor"]), float(sc["original"]), float(sc["fast"]),
                                              float(sc["slow"]))
            angle = inv[None, :] * np.arange(env.max_positions, dtype=np.float64)[:, None]
        elif p.get("exact_angles"):
            inv = np.array([math.pow(float(p["theta"]), -2.0 * i / self.rotary_dim) for i in range(self.rotary_dim // 2)], dtype=np.float64)
            kind = (p.get("scaling") or {}).get("rope_type", "default")
            if kind == "llama3":
                inv = rescaled_long_waves(inv, p["scaling"])
            elif kind != "default":
                raise ValueError(f"rotary encoding: exact_angles goes with the default and the llama3 scaling, not '{kind}'")
            angle = inv[None, :] * np.arange(env.max_positions, dtype=np.float64)[:, None]
        else:
            inv = inverse_frequencies(self.rotary_dim, float(p["theta"]), p.get("scaling") or {})
            pos = np.arange(env.max_positions, dtype=np.float32)
            angle = (inv[None, :] * pos[:, None]).astype(np.float32).astype(np.float64)
        table = (np.stack([np.cos(angle), np.sin(angle)], axis=-1) * magnitude).astype(np.float32)
        self.cos_sin = torch.from_numpy(table).to(env.device)   # [max_positions, rotary_dim / 2, 2]
