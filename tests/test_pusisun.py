"""Pusisun on the CPU: the architecture's registration, configuration errors, the tensor plan, the schedule of a looped range of
layers, the cache manager's books for a window that keeps first tokens, and the plain implementation against cases made by hand
for every mechanism."""
from __future__ import annotations

import copy
import math

import pytest
import torch

import plain_pusisun as plain
from pusisun_cases import PUSISUN, PUSISUN_X, PUSISUN_Y, PUSISUN_Z, load_plain, near_uniform, write_model

F = torch.float64


def test_the_architecture_is_registered_and_chosen_by_config():
    from stride_b200.config import resolve_architecture
    assert resolve_architecture(PUSISUN_X).name == "Pusisun"
    assert resolve_architecture({"model_type": "pusisun"}).name == "Pusisun"


@pytest.mark.parametrize("name", list(PUSISUN))
def test_tensor_plan(name):
    from stride_b200.weights.random_init import model_plan
    cfg = PUSISUN[name][0]
    plan = model_plan(cfg)
    W = cfg["width"]
    assert plan["embed"].shape == plan["head"].shape == (cfg["vocab"], W) and plan["final.norm"].shape == (W,)
    assert ("loop.step" in plan) == ("loop" in cfg)
    if "loop" in cfg:
        assert plan["loop.step"].shape == (cfg["loop"]["times"], W)
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        assert plan[p + "norm1"].shape == plan[p + "norm1b"].shape == (W,)
        assert (p + "norm2" in plan) == (p + "norm2b" in plan) == (p + "mlp.router" in plan) == (l["mlp"] is not None)
        H, D, V = m["heads"], m["dim"], m["vdim"]
        assert plan[p + "mix.o"].shape == (W, H * V)
        if l["type"] == "attention":
            G = m["kv_heads"]
            assert plan[p + "mix.q"].shape == (H * D, W) and plan[p + "mix.k"].shape == (G * D, W) and plan[p + "mix.v"].shape == (G * V, W)
            assert plan[p + "mix.q.b"].shape == plan[p + "mix.q.norm"].shape == (H * D,)
            assert plan[p + "mix.k.b"].shape == plan[p + "mix.k.norm"].shape == (G * D,)
            assert plan[p + "mix.v.b"].shape == (G * V,) and plan[p + "mix.sink"].shape == (H,)
        else:
            R, C, Q = m["rot_dim"], m["kv_rank"], m["q_rank"]
            assert plan[p + "mix.dq"].shape == (Q, W) and plan[p + "mix.dq.norm"].shape == (Q,) and plan[p + "mix.uq"].shape == (H * (D + R), Q)
            assert plan[p + "mix.dkv"].shape == (C + R, W) and plan[p + "mix.dkv.norm"].shape == (C,)
            assert plan[p + "mix.uk"].shape == (H * D, C) and plan[p + "mix.uv"].shape == (H * V, C)
        if l["mlp"]:
            r, ff = l["mlp"]["router"], l["mlp"]["expert"]["ff"]
            assert plan[p + "mlp.router"].shape == (r["experts"], W) and plan[p + "mlp.router.b"].shape == (r["experts"],)
            assert plan[p + f"mlp.e{r['experts'] - 1}.gate"].shape == plan[p + "mlp.e0.up"].shape == (ff, W)
            assert plan[p + "mlp.e0.down"].shape == (W, ff) and p + f"mlp.e{r['experts']}.up" not in plan


@pytest.mark.parametrize("edit,word", [
    (lambda c: c["layers"][0].__setitem__("type", "conv"), "type"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("kv_heads", 3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("keep_first", -1), "keep_first"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 8), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("rot_dim", 7), "rot_dim"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "dense"), "mlp.kind"),
    (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 9), "router"),
    (lambda c: c["loop"].__setitem__("stop", 9), "loop"),
    (lambda c: c.pop("norm"), "norm.eps"),
    (lambda c: c.__setitem__("layers", []), "layers"),
])
def test_config_errors_name_the_key(edit, word):
    from stride_b200.config import ConfigError, resolve_architecture
    cfg = copy.deepcopy(PUSISUN_X)
    edit(cfg)
    with pytest.raises(ConfigError, match=word.replace(".", r"\.")):
        resolve_architecture(cfg).parse_config(cfg)


def test_model_spec_follows_the_layer_list_and_the_loop():
    """Every pass over the looped layers is a run of schedule entries of its own (so each has a cache of its own), with the part that
    rewrites the stream in front: the first adds its row of the table only, the later ones the embedding output too."""
    from stride_b200.config import resolve_architecture
    arch = resolve_architecture(PUSISUN_X)
    spec = arch.model_spec(arch.parse_config(PUSISUN_X))
    assert [l.block for l in spec.layers[:4]] == ["prenorm_scaled", "prenorm_scaled_mixer", "prenorm_scaled", "prenorm_scaled"]
    assert [l.mixer.kind for l in spec.layers[:4]] == ["masked_attention", "latent_attention", "masked_attention", "masked_attention"]
    assert [e.layer for e in spec.schedule] == [0, 4, 1, 2, 5, 1, 2, 3]
    first, second = spec.layers[4].rewrite.params, spec.layers[5].rewrite.params
    assert (first["row"], first["add_embedding"], second["row"], second["add_embedding"]) == (0, False, 1, True)
    a = spec.layers[0].mixer.params
    assert (a["window"], a["keep_first"], a["num_kv_heads"], a["key_dim"], a["value_dim"]) == (24, 5, 2, 24, 40)
    assert spec.layers[3].mixer.params["window"] == 0
    r = spec.layers[1].mixer.params["position"].params
    assert r["scaling"]["rope_type"] == "yarn" and r["scaling"]["factor"] == 8.0 and r["rotary_dim"] == 12
    ff = spec.layers[2].feed_forward.params
    assert (ff["experts"], ff["top"], ff["weights_from"]) == (3, 3, "logits")
    # no loop: the layers in their order, nothing in front of them
    arch = resolve_architecture(PUSISUN_Z)
    spec = arch.model_spec(arch.parse_config(PUSISUN_Z))
    assert [e.layer for e in spec.schedule] == [0, 1, 2] and len(spec.layers) == 3
    # a loop of one layer at the front, three passes
    arch = resolve_architecture(PUSISUN_Y)
    spec = arch.model_spec(arch.parse_config(PUSISUN_Y))
    assert [e.layer for e in spec.schedule] == [4, 0, 5, 0, 6, 0, 1, 2, 3]
    assert spec.layers[3].mixer.params["position"].params["scaling"]["rope_type"] == "default"


def test_trimming_a_window_leaves_the_pages_of_the_kept_first_tokens():
    """A group whose window keeps the first 5 tokens (pages of 4: two pages) gives back the pages between those and the window, never
    the first two; a group with the same window and no kept tokens gives back everything behind the window. Slots and pages come back
    and are used again; the books stay whole."""
    from stride_b200.cache.manager import CacheManager
    from stride_b200.parts.base import CacheNeed
    kept = CacheNeed("pages", kv_heads=2, head_dim=8, window=6, dtype=torch.float32, keep_first=5)
    bare = CacheNeed("pages", kv_heads=2, head_dim=8, window=6, dtype=torch.float32)
    cm = CacheManager([kept, bare, kept], device="cpu", max_slots=2, max_context=64, page_size=4, num_pages=12)
    assert len(cm.groups) == 2
    gk = next(g for g in cm.groups if g.keep_first == 5)
    gb = next(g for g in cm.groups if g.keep_first == 0)
    s = cm.acquire_slot()
    assert cm.ensure(s, 30)                          # 8 pages each
    cm.trim(s)
    tk, tb = gk.table_host[s], gb.table_host[s]
    # the next token stands at 30 and sees 25..30: page 6 (24..27) on; pages 0 and 1 hold tokens 0..4
    assert [int(i) for i in range(8) if tk[i] >= 0] == [0, 1, 6, 7]
    assert [int(i) for i in range(8) if tb[i] >= 0] == [6, 7]
    held = {int(tk[0]), int(tk[1])}
    assert cm.ensure(s, 45)
    cm.trim(s)
    assert {int(tk[0]), int(tk[1])} == held and [int(i) for i in range(12) if tk[i] >= 0] == [0, 1, 10, 11]
    cm.check()
    cm.release_slot(s)
    cm.check()
    t = cm.acquire_slot()
    assert cm.ensure(t, 48)                          # every page of the pool is there again
    cm.check()


# ------------------------------------------------------------------------------------------------ the plain implementation itself
def test_plain_norm():
    x = torch.tensor([[3.0, 4.0]], dtype=F)
    got = plain.rms_norm(x, torch.tensor([1.0, 2.0], dtype=F), 0.5)
    assert torch.allclose(got, torch.tensor([[3.0, 8.0]], dtype=F) / math.sqrt(13.0))


def test_plain_scaled_frequencies_by_hand():
    """8 dims, base 16: f = 1, 1/2, 1/4, 1/8. original 2 pi * 16: a pair that turns t times within the original length has index
    8 ln(16 / t) / (2 ln 16); fast 16 -> 0, slow 1 -> 4, so ramp_i = i / 4."""
    freq, mag = plain.yarn_frequencies(8, 16.0, {"factor": 4.0, "original": 2 * math.pi * 16, "fast": 16.0, "slow": 1.0})
    want = [f / 4.0 * r + f * (1 - r) for f, r in zip((1.0, 0.5, 0.25, 0.125), (0.0, 0.25, 0.5, 0.75))]
    assert freq == pytest.approx(want, rel=1e-12) and mag == pytest.approx(0.1 * math.log(4.0) + 1.0)
    # lo = hi: the ramp is a step (the difference is held at 0.001)
    freq, _ = plain.yarn_frequencies(8, 16.0, {"factor": 2.0, "original": 2 * math.pi * 4, "fast": 1.0, "slow": 1.0})
    assert freq == pytest.approx([1.0, 0.5, 0.25, 0.125 / 2], rel=1e-12)              # lo = hi = 8 ln 4 / (2 ln 16) = 2: pair 2 stays, 3 is slowed
    freq, mag = plain.yarn_frequencies(8, 16.0, None)
    assert freq == pytest.approx([1.0, 0.5, 0.25, 0.125]) and mag == 1.0


def test_plain_rotation_pairs_halves():
    v = torch.zeros(3, 1, 4, dtype=F)
    v[:, 0, 0], v[:, 0, 3] = 1.0, 2.0
    r = plain.rotate(v, torch.arange(3), [0.5, 0.25], 3.0)
    # (u, v) = (x0, x2) turns by 0.5 p, (x1, x3) by 0.25 p; both times 3
    p = 2
    want = torch.tensor([math.cos(1.0), -2.0 * math.sin(0.5), math.sin(1.0), 2.0 * math.cos(0.5)], dtype=F) * 3.0
    assert torch.allclose(r[p, 0], want)
    assert torch.allclose(r[0, 0], v[0, 0] * 3.0)


def _identity_attention(H, G, D, V, extra=None):
    """Tensors that make the plain attention read q, k, v straight from its input [q | k | v] (q and k still normed as wholes)."""
    width = H * D + G * D + G * V
    eye = torch.eye(width)
    t = {"p.q": eye[:H * D], "p.k": eye[H * D:H * D + G * D], "p.v": eye[H * D + G * D:], "p.o": torch.eye(H * V),
         "p.q.b": torch.zeros(H * D), "p.k.b": torch.zeros(G * D), "p.v.b": torch.zeros(G * V), "p.q.norm": torch.ones(H * D),
         "p.k.norm": torch.ones(G * D), "p.sink": torch.full((H,), -1e9)}
    t.update(extra or {})
    return t, width


def test_plain_window_kept_tokens_sink_and_slopes_by_hand():
    """One head, zero queries: the scores are the distance terms alone. Values name their position, so the output says which keys
    were seen and how they were weighed."""
    T = 12
    t, width = _identity_attention(1, 1, 2, 1)
    h = torch.zeros(T, width, dtype=F)
    h[:, 2:4] = 1.0                                         # keys (any), queries zero
    h[:, 4] = torch.arange(T, dtype=F)                      # value = position
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 1, "scale": 1.0, "mask": {"size": 3, "keep_first": 2}}
    out = plain.sink_attention(h, t, "p.", m, 1e-6)[:, 0]
    slope = 2.0 ** -8.0                                     # one head: 2^(-8 * 1 / 1)
    for i in (0, 1, 2, 4, 5, 11):
        seen = [j for j in range(i + 1) if i - j < 3 or j < 2]
        wts = [math.exp(-slope * (i - j)) for j in seen]
        assert float(out[i]) == pytest.approx(sum(w * j for w, j in zip(wts, seen)) / sum(wts), rel=1e-12), f"position {i}"
    # a sink of 0 counts as one more key of score 0 without a value
    t["p.sink"] = torch.zeros(1)
    out = plain.sink_attention(h, t, "p.", m, 1e-6)[:, 0]
    seen = [0, 1, 9, 10, 11]
    wts = [math.exp(-slope * (11 - j)) for j in seen]
    assert float(out[11]) == pytest.approx(sum(w * j for w, j in zip(wts, seen)) / (sum(wts) + 1.0), rel=1e-12)
    # no mask: every earlier key
    m.pop("mask")
    out = plain.sink_attention(h, t, "p.", m, 1e-6)[:, 0]
    wts = [math.exp(-slope * (11 - j)) for j in range(12)]
    assert float(out[11]) == pytest.approx(sum(w * j for j, w in enumerate(wts)) / (sum(wts) + 1.0), rel=1e-12)


def test_plain_slopes_groups_and_whole_projection_norm():
    """Four heads on two key heads: head h reads key head h // 2 and has slope 2^(-2 (h + 1)); q is normed over all its H D elements
    at once, so scaling one head's query rows changes the other heads' scores."""
    H, G, D, V, T = 4, 2, 2, 1, 6
    t, width = _identity_attention(H, G, D, V)
    g = torch.Generator().manual_seed(5)
    h = torch.randn(T, width, generator=g).to(F)
    m = {"heads": H, "kv_heads": G, "dim": D, "vdim": V, "scale": 0.7}
    out = plain.sink_attention(h, t, "p.", m, 1e-6)
    q = h[:, :H * D] / torch.sqrt((h[:, :H * D] ** 2).mean(-1, keepdim=True) + 1e-6)
    k = h[:, H * D:H * D + G * D] / torch.sqrt((h[:, H * D:H * D + G * D] ** 2).mean(-1, keepdim=True) + 1e-6)
    v = h[:, H * D + G * D:]
    i = T - 1
    for head in range(H):
        kv = head // 2
        sc = [0.7 * float(q[i, head * D:(head + 1) * D] @ k[j, kv * D:(kv + 1) * D]) - 2.0 ** (-2.0 * (head + 1)) * (i - j) for j in range(T)]
        e = [math.exp(s) for s in sc]
        assert float(out[i, head]) == pytest.approx(sum(a * float(v[j, kv]) for j, a in enumerate(e)) / sum(e), rel=1e-10)
    h2 = h.clone()
    h2[:, :D] *= 10.0                                       # head 0's query
    assert not torch.allclose(plain.sink_attention(h2, t, "p.", m, 1e-6)[:, 1:], out[:, 1:])


def test_plain_routing_by_hand():
    """Three experts, two chosen: the bias decides who is chosen AND enters the weights (the softmax is over the chosen logits)."""
    W = 2
    t = {"p.router": torch.tensor([[1.0, 0.0], [0.0, 1.0], [0.0, 0.0]]), "p.router.b": torch.tensor([0.0, 0.0, 1.5])}
    for e in range(3):
        t[f"p.e{e}.gate"], t[f"p.e{e}.up"], t[f"p.e{e}.down"] = torch.eye(W), torch.eye(W) * (e + 1), torch.eye(W)
    mlp = {"router": {"experts": 3, "top": 2}}
    h = torch.tensor([[2.0, 1.0]], dtype=F)                 # logits 2, 1, 1.5: experts 0 and 2
    s = torch.softmax(torch.tensor([2.0, 1.5], dtype=F), 0)
    act = plain.silu(h) * h
    want = s[0] * act * 1.0 + s[1] * act * 3.0
    assert torch.allclose(plain.routed_experts(h, t, "p.", mlp), want)
    leads = []
    plain.routed_experts(h, t, "p.", mlp, leads=leads)
    assert float(leads[0][0]) == pytest.approx(0.5)
    mlp["router"]["top"] = 3                                # all chosen: the softmax over all logits
    s = torch.softmax(torch.tensor([2.0, 1.0, 1.5], dtype=F), 0)
    assert torch.allclose(plain.routed_experts(h, t, "p.", mlp), s[0] * act + s[1] * act * 2.0 + s[2] * act * 3.0)


def test_plain_latent_attention_against_explicit_heads():
    """The latent mixer written out the long way for one position: keys and values of every head built from the latent, the shared
    rotated part appended to every head's key."""
    g = torch.Generator().manual_seed(11)
    W, H, D, R, V, Q, C, T = 10, 2, 3, 4, 5, 6, 7, 5
    t = {"p.dq": torch.randn(Q, W, generator=g), "p.dq.norm": torch.rand(Q, generator=g) + 0.5, "p.uq": torch.randn(H * (D + R), Q, generator=g),
         "p.dkv": torch.randn(C + R, W, generator=g), "p.dkv.norm": torch.rand(C, generator=g) + 0.5, "p.uk": torch.randn(H * D, C, generator=g),
         "p.uv": torch.randn(H * V, C, generator=g), "p.o": torch.eye(H * V)}
    m = {"heads": H, "dim": D, "rot_dim": R, "vdim": V, "q_rank": Q, "kv_rank": C, "scale": 0.4, "rot": {"dims": R, "base": 9.0}}
    h = torch.randn(T, W, generator=g).to(F)
    out = plain.latent_attention(h, t, "p.", m, 1e-5)
    freq = [1.0, 9.0 ** -0.5]

    def turn(x, p):
        u, v = x[:2], x[2:]
        c, s = torch.tensor([math.cos(p * f) for f in freq], dtype=F), torch.tensor([math.sin(p * f) for f in freq], dtype=F)
        return torch.cat([u * c - v * s, v * c + u * s])

    norm = lambda x, gain: x / torch.sqrt((x * x).mean() + 1e-5) * gain.to(F)
    i = T - 1
    q = t["p.uq"].to(F) @ norm(t["p.dq"].to(F) @ h[i], t["p.dq.norm"])
    for head in range(H):
        qh = q[head * (D + R):(head + 1) * (D + R)]
        sc, vals = [], []
        for j in range(T):
            down = t["p.dkv"].to(F) @ h[j]
            c = norm(down[:C], t["p.dkv.norm"])
            kh = t["p.uk"].to(F)[head * D:(head + 1) * D] @ c
            sc.append(0.4 * float(qh[:D] @ kh + turn(qh[D:], i) @ turn(down[C:], j)))
            vals.append(t["p.uv"].to(F)[head * V:(head + 1) * V] @ c)
        wts = torch.softmax(torch.tensor(sc, dtype=F), 0)
        assert torch.allclose(out[i, head * V:(head + 1) * V], sum(a * v for a, v in zip(wts, vals)), rtol=1e-10, atol=1e-12)


def test_plain_loop_adds_the_embedding_and_a_row_before_each_pass(tmp_path):
    """The order of runs, and what stands in front of a pass: with the looped layers' sublayers silenced (their closing norms'
    gains set to zero) the stream is the embedding output times the number of passes plus the rows of the table."""
    assert [(i, t) for i, t, _ in plain.layer_order(PUSISUN_X)] == [(0, None), (1, 0), (2, 0), (1, 1), (2, 1), (3, None)]
    assert [o for _, _, o in plain.layer_order(PUSISUN_X)] == [False, True, False, True, False, False]
    assert [(i, t) for i, t, _ in plain.layer_order(PUSISUN_Y)][:4] == [(0, 0), (0, 1), (0, 2), (1, None)]

    def silence(tensors):
        for n in tensors:
            if n.endswith("norm1b") or n.endswith("norm2b"):
                tensors[n] = torch.zeros_like(tensors[n])

    cfg, w = load_plain(write_model(tmp_path / "m", "Y", transform=silence))
    toks = [3, 1, 4]
    streams = []
    plain.forward(cfg, w, toks, streams=streams)
    e = w["embed"].to(F)[toks] * cfg["embedding"]["scale"]
    step = w["loop.step"].to(F)
    assert torch.allclose(streams[0], e + step[0]) and torch.allclose(streams[1], 2 * e + step[0] + step[1])
    assert torch.allclose(streams[2], 3 * e + step.sum(0)) and torch.allclose(streams[-1], streams[2]) and len(streams) == 6


def test_the_yardstick_notices_each_mechanism(tmp_path):
    """With attention made close to uniform every visible key carries weight, and the plain implementation itself moves by far more
    than the 32-bit tolerance when a window is one token off, a kept token is dropped, the sink is left out, the distance term is
    dropped, the pass's row is not added, or the router's bias is left out of the weights."""
    from conftest import logit_tolerance, random_tokens
    cfg, w = load_plain(write_model(tmp_path / "u", "X", transform=near_uniform))
    toks = random_tokens(cfg["vocab"], 60, 3)
    want = plain.forward(cfg, w, toks).float()
    tol = logit_tolerance("float32", want)

    def moved(edit_cfg=None, edit_w=None):
        c, ww = copy.deepcopy(cfg), dict(w)
        if edit_cfg:
            edit_cfg(c)
        if edit_w:
            edit_w(ww)
        return float((plain.forward(c, ww, toks).float() - want)[40:].abs().max(dim=1).values.min())

    for delta in (1, -1):
        assert moved(lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("size", 24 + delta)) > 20 * tol
        assert moved(lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("keep_first", 5 + delta)) > 20 * tol
        assert moved(lambda c: c["layers"][2]["mixer"]["mask"].__setitem__("size", 7 + delta)) > 20 * tol
    assert moved(edit_w=lambda t: t.__setitem__("l0.mix.sink", torch.full_like(t["l0.mix.sink"], -1e9))) > 20 * tol
    assert moved(edit_w=lambda t: t.__setitem__("loop.step", torch.zeros_like(t["loop.step"]))) > 20 * tol
    assert moved(edit_w=lambda t: t.__setitem__("l0.mlp.router.b", torch.zeros_like(t["l0.mlp.router.b"]))) > 20 * tol
    assert moved(lambda c: c["embedding"].__setitem__("scale", 3.01)) > 20 * tol
