"""Sitivik on the CPU: the configuration reader and the model specification, the sizes that only a checkpoint's shapes tell, and the
plain implementation (tests/plain_sitivik.py) against cases small enough to be written out by hand."""
from __future__ import annotations

import copy
import math

import pytest
import torch

import plain_sitivik as plain
from sitivik_cases import SITIVIK, load_plain, near_uniform, write_model

F = torch.float64


def test_configurations_parse_and_plan_their_tensors():
    from stride_b200.config import ConfigError, resolve_architecture
    from stride_b200.weights.random_init import model_plan
    for name, (cfg, _, _) in SITIVIK.items():
        arch = resolve_architecture(cfg)
        assert arch.name == "Sitivik"
        spec = arch.model_spec(arch.parse_config(cfg))
        L = len(cfg["layers"])
        side = "token_side" in cfg
        assert len(spec.schedule) == (2 * L if side else L) and len(spec.layers) == (2 * L if side else L)
        plan = model_plan(cfg)
        assert "embed" in plan and "final.norm" in plan and ("side.embed" in plan) == side and "head" not in plan
        for i, layer in enumerate(cfg["layers"]):
            assert (f"l{i}.mlp.gate" in plan) == (layer["mlp"] is not None) and f"l{i}.ls1" in plan
            if layer["type"] == "parallel_2":
                r = layer["mixer"]["right"]
                assert plan[f"l{i}.mix.right.a1"].shape == (r["decay_rank"], cfg["width"])
                assert plan[f"l{i}.mix.right.g2"].shape == (r["heads"] * r["vdim"], r["gate_rank"])
                assert plan[f"l{i}.mix.right.q.conv"].shape == (r["kv_heads"] * r["dim"], r["conv"])
                assert plan[f"l{i}.mix.left.q.norm"].shape == (layer["mixer"]["left"]["dim"],)
            elif layer["type"] == "parallel":
                m = layer["mixer"]["left"]
                assert plan[f"l{i}.mix.left.q.norm"].shape == (m["heads"] * m["dim"],) and f"l{i}.mix.left.o.b" in plan
                assert f"l{i}.mix.right.out" in plan
            else:
                m = layer["mixer"]
                assert plan[f"l{i}.mix.q"].shape == (2 * m["heads"] * m["dim"], cfg["width"]) and plan[f"l{i}.mix.g"].shape == (m["heads"], cfg["width"])
    bad = copy.deepcopy(SITIVIK["X"][0])
    bad["layers"][1]["mixer"]["right"]["decay"] = [0.9]
    with pytest.raises(ConfigError, match="decay"):
        resolve_architecture(bad).parse_config(bad)
    bad = copy.deepcopy(SITIVIK["X"][0])
    bad["layers"][2]["type"] = "parallel_3"
    with pytest.raises(ConfigError, match="parallel_3"):
        resolve_architecture(bad).parse_config(bad)
    bad = copy.deepcopy(SITIVIK["X"][0])
    del bad["layers"][0]["mixer"]["diff"]
    with pytest.raises(ConfigError, match="diff"):
        resolve_architecture(bad).parse_config(bad)


def test_ranks_come_from_the_checkpoints_shapes(tmp_path):
    """config.json does not name the ranks of the delta rule's low-rank projections; the shapes of a1 and g1 do."""
    import json
    from stride_b200.config import resolve_architecture
    from stride_b200.weights.loader import tensor_shapes
    folder = write_model(tmp_path / "x", "X")
    stored = json.loads((folder / "config.json").read_text())
    assert "decay_rank" not in stored["layers"][2]["mixer"]["right"]
    arch = resolve_architecture(stored)
    full = arch.complete_config(stored, tensor_shapes(folder))
    assert full["layers"][2]["mixer"]["right"]["decay_rank"] == 5 and full["layers"][2]["mixer"]["right"]["gate_rank"] == 9
    assert "decay_rank" not in stored["layers"][2]["mixer"]["right"]            # the caller's dict is left alone
    right = arch.parse_config(full).layers[2].right
    assert (right.decay_rank, right.gate_rank) == (5, 9)


def test_plain_rotation_pairs_and_scaled_frequencies():
    x = torch.arange(1.0, 9.0, dtype=F).view(1, 1, 8)
    pos = torch.tensor([3])
    rot = {"dims": 4, "base": 100.0}
    f = [1.0, 100.0 ** -0.5]
    inter = plain.rotate(x, pos, rot, True)[0, 0]
    half = plain.rotate(x, pos, rot, False)[0, 0]
    for i in range(2):
        c, s = math.cos(3 * f[i]), math.sin(3 * f[i])
        u, v = float(x[0, 0, 2 * i]), float(x[0, 0, 2 * i + 1])
        assert abs(float(inter[2 * i]) - (u * c - v * s)) < 1e-12 and abs(float(inter[2 * i + 1]) - (v * c + u * s)) < 1e-12
        u, v = float(x[0, 0, i]), float(x[0, 0, i + 2])
        assert abs(float(half[i]) - (u * c - v * s)) < 1e-12 and abs(float(half[i + 2]) - (v * c + u * s)) < 1e-12
    assert torch.equal(inter[4:], x[0, 0, 4:]) and torch.equal(half[4:], x[0, 0, 4:])
    # waves shorter than original / high stay, longer than original / low slow down by the factor, the ramp in between
    got = plain.frequencies({"dims": 8, "base": 10000.0, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}})
    plainf = [10000.0 ** (-2.0 * i / 8) for i in range(4)]
    assert float(got[0]) == plainf[0]                                           # wave 6.3 < 16
    assert abs(float(got[3]) - plainf[3] / 4.0) < 1e-15                          # wave 6283 > 64
    wave = 2 * math.pi / plainf[1]                                                # 62.8: between 16 and 64
    s = (64 / wave - 1.0) / 3.0
    assert 16 < wave < 64 and abs(float(got[1]) - ((1 - s) * plainf[1] / 4.0 + s * plainf[1])) < 1e-15
    # the engine's table is the same angles
    from stride_b200.parts import BuildEnv, PartSpec, part_class
    env = BuildEnv(device=torch.device("cpu"), compute_dtype=torch.float32, max_tokens=1, max_positions=50)
    spec = PartSpec("rope", {"head_dim": 8, "rotary_dim": 8, "theta": 10000.0, "exact_angles": True,
                             "scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                         "original_max_position_embeddings": 64}})
    table = part_class("position", "rope")(spec, env).cos_sin
    want = torch.stack([torch.cos(torch.arange(50, dtype=F)[:, None] * got), torch.sin(torch.arange(50, dtype=F)[:, None] * got)], -1)
    assert (table.double() - want).abs().max() < 1e-7


def test_plain_masks_sink_and_maps_by_hand():
    assert plain.window_mask(5, 2).tolist() == [[j in (i - 1, i) for j in range(5)] for i in range(5)]
    assert plain.chunk_mask(7, 3).tolist() == [[j <= i and j // 3 == i // 3 for j in range(7)] for i in range(7)]
    # values that name their position: uniform scores make the result the mean of the visible positions
    T = 6
    q, k = torch.zeros(T, 1, 2, dtype=F), torch.zeros(T, 1, 2, dtype=F)
    v = torch.arange(T, dtype=F).view(T, 1, 1)
    got = plain.softmax_attention(q, k, v, 1.0, plain.chunk_mask(T, 4), False)[:, 0, 0]
    assert torch.allclose(got, torch.tensor([0.0, 0.5, 1.0, 1.5, 4.0, 4.5], dtype=F))
    sunk = plain.softmax_attention(q, k, v, 1.0, plain.chunk_mask(T, 4), True)[:, 0, 0]        # one more term of weight 1, no value
    assert torch.allclose(sunk, torch.tensor([0.0, 1 / 3, 3 / 4, 6 / 5, 4 / 2, 9 / 3], dtype=F))
    win = plain.softmax_attention(q, k, v, 1.0, plain.window_mask(T, 3), False)[:, 0, 0]
    assert torch.allclose(win, torch.tensor([0.0, 0.5, 1.0, 2.0, 3.0, 4.0], dtype=F))


def test_plain_convolution_and_delta_rule_by_hand():
    x = torch.tensor([[1.0], [2.0], [4.0]], dtype=F)
    y = plain.short_convolution(x, torch.tensor([[100.0, 10.0, 1.0]], dtype=F))                 # the last tap is the current token's
    assert y.view(-1).tolist() == [1.0, 12.0, 124.0]
    # beta 1, no decay, q along k: the state returns the value written for that key direction, and writing the same pair again changes
    # nothing (the correction v - S^T k is zero), while another value for the same key replaces the old one
    g = torch.Generator().manual_seed(1)
    W, D, V = 6, 4, 3
    wk = torch.randn(D, W, generator=g, dtype=F)
    w = {"p.q": wk, "p.k": wk, "p.v": torch.randn(V, W, generator=g, dtype=F), "p.b": torch.full((1, W), 0.0, dtype=F),
         "p.q.conv": torch.ones(D, 1, dtype=F), "p.k.conv": torch.ones(D, 1, dtype=F), "p.v.conv": torch.ones(V, 1, dtype=F),
         "p.A_log": torch.tensor([-40.0], dtype=F), "p.dt_bias": torch.zeros(D, dtype=F), "p.a1": torch.zeros(2, W, dtype=F),
         "p.a2": torch.zeros(D, 2, dtype=F), "p.g1": torch.zeros(2, W, dtype=F), "p.g2": torch.zeros(V, 2, dtype=F),
         "p.norm": torch.ones(V, dtype=F), "p.o": torch.eye(V, dtype=F)}
    m = {"heads": 1, "kv_heads": 1, "dim": D, "vdim": V, "conv": 1}
    h0 = torch.randn(W, generator=g, dtype=F)
    for beta_logit, same in ((40.0, True), (40.0, False)):
        w["p.b"] = torch.zeros(1, W, dtype=F)
        w["p.b"][0] = beta_logit * h0 / (h0 @ h0)                               # sigmoid(40) = 1 for both tokens below
        h1 = h0 if same else h0 * 1.0
        out = plain.delta_right(w, "p.", m, torch.stack([h0, h1]), 1e-6, False)
        v0 = plain.silu(w["p.v"] @ h0)
        want = 0.5 * v0 / torch.sqrt((v0 * v0).mean() + 1e-6 * D)               # o = D^-1/2 v; the norm divides D^-1/2 out again (eps scaled with it)
        assert (out[0] - want).abs().max() < 1e-5 and (out[1] - out[0]).abs().max() < 1e-9


def test_the_yardsticks_notice_a_mask_one_off_and_a_missing_sink(tmp_path):
    """With attention close to uniform the plain logits move far beyond the float32 tolerance when a window or a chunk is one token longer
    or shorter, and when the sink is left out of the denominator: what the engine tests then hold the engine to."""
    from conftest import logit_tolerance, random_tokens
    folder = write_model(tmp_path / "xu", "X", transform=near_uniform)
    cfg, w = load_plain(folder)
    toks = random_tokens(cfg["vocab"], 70, 5)
    want = plain.forward(cfg, w, toks).float()
    tol = logit_tolerance("float32", want)
    for layer, delta in ((1, 1), (1, -1), (2, 1), (2, -1)):
        other = copy.deepcopy(cfg)
        other["layers"][layer]["mixer"]["left"]["mask"]["size"] += delta
        moved = (plain.forward(other, w, toks).float() - want).abs().max(dim=1).values
        assert moved[45:].min() > 20 * tol, f"the yardstick does not notice layer {layer}'s mask {delta:+d}"
    keep = plain.softmax_attention
    try:
        plain.softmax_attention = lambda q, k, v, scale, mask, sink: keep(q, k, v, scale, mask, False)
        moved = (plain.forward(cfg, w, toks).float() - want).abs().max(dim=1).values
    finally:
        plain.softmax_attention = keep
    assert moved.min() > 20 * tol
