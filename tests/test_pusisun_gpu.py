"""Pusisun through the engine against the plain implementation (tests/plain_pusisun.py): every mechanism's kernels alone, then whole
models of three tiny configurations whole, decoded token by token, in portions down to two tokens and in mixed batches with pages and
slots used again, in 32-bit and in bfloat16; window edges, kept first tokens, sinks and far keys made to show; long decoding; batches
against each request alone; greedy generation through the entry point, its scheduler and the command line."""
from __future__ import annotations

import copy
import math

import pytest
import torch

import plain_pusisun as plain
from conftest import TraceRun, logit_tolerance, random_tokens
from pusisun_cases import PUSISUN, load_plain, near_uniform, write_model
from test_replay_gpu import _Bits, _portions

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F = torch.float64


@pytest.fixture(scope="module")
def pusisun_dirs(tmp_path_factory):
    root = tmp_path_factory.mktemp("pusisun")
    out = {name: write_model(root / name, name) for name in PUSISUN}
    out["XU"] = write_model(root / "XU", "X", transform=near_uniform)
    return out


def _meta(entries):
    """[4, E] int32 on the device from (slot, first row, length, first position) records."""
    return torch.tensor([[e[k] for e in entries] for k in range(4)], dtype=torch.int32, device=DEV)


def _rows(entries):
    """positions and slots of every row of a step."""
    pos = [p for _, _, n, p0 in entries for p in range(p0, p0 + n)]
    slot = [s for s, _, n, _ in entries for _ in range(n)]
    return torch.tensor(pos, dtype=torch.int32, device=DEV), torch.tensor(slot, dtype=torch.int32, device=DEV)


def _table(lengths, page, spare, g):
    """A block table that hands the pages out in a shuffled order: [requests, most pages], and the number of pages."""
    per = [-(-n // page) for n in lengths]
    perm = torch.randperm(sum(per) + spare, generator=g).tolist()
    table = torch.full((len(lengths), max(per)), -1, dtype=torch.int32)
    k = 0
    for r, c in enumerate(per):
        for j in range(c):
            table[r, j] = perm[k]
            k += 1
    return table.to(DEV), sum(per) + spare


# ---------------------------------------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("n,W,Sa", [(5, 96, 3), (40, 100, 1), (300, 64, 0), (2, 1000, 2)])
def test_result_norm_and_stream_add_kernels(n, W, Sa):
    """h += gain * r / sqrt(mean(r^2) + eps) with r a buffer plus partial sums; and h <- (h + partial sums + e) + vector."""
    from stride_b200.kernels import ops
    g = torch.Generator().manual_seed(n + W)
    dst, a, e = (torch.randn(n, W, generator=g) for _ in range(3))
    pa = torch.randn(Sa, n, W, generator=g) if Sa else None
    gain = (torch.randn(W, generator=g)).to(torch.bfloat16)
    eps = 1e-3
    dev = lambda t: None if t is None else t.to(DEV)
    r = a.double() * 0.7 + (pa.double().sum(0) * 0.7 if pa is not None else 0)
    want = dst.double() + plain.rms_norm(r, gain.double(), eps)
    d, ad = dev(dst).clone(), dev(a).clone()
    ops.branch_norm_fold(d, dev(gain), eps, a=ad, a_partials=dev(pa), ca=0.7)
    assert (d.cpu().double() - want).abs().max() <= 1e-5 * float(want.abs().max())
    assert float(ad.abs().max()) == 0.0                                           # the branch is empty again
    if pa is not None:                                                             # partial sums alone, float32 gain
        d2 = dev(dst).clone()
        ops.branch_norm_fold(d2, dev(gain.float()), eps, a_partials=dev(pa))
        want2 = dst.double() + plain.rms_norm(pa.double().sum(0), gain.double(), eps)
        assert (d2.cpu().double() - want2).abs().max() <= 1e-5 * float(want2.abs().max())
    vec = torch.randn(W, generator=g).to(torch.bfloat16)
    d3 = dev(dst).clone()
    ops.stream_add(d3, dev(e), dev(vec), partials=dev(pa))
    want3 = dst.double() + (pa.double().sum(0) if pa is not None else 0) + e.double() + vec.double()
    assert (d3.cpu().double() - want3).abs().max() <= 1e-6 * float(want3.abs().max())
    d4 = dev(dst).clone()
    ops.stream_add(d4, None, dev(vec))
    assert (d4.cpu().double() - (dst.double() + vec.double())).abs().max() <= 1e-6 * float(want3.abs().max())


@pytest.mark.parametrize("E,top,Fs", [(5, 2, 40), (3, 3, 24), (4, 1, 16), (40, 6, 8), (2, 1, 48)])
def test_routing_by_logits_and_gated_experts_against_the_plain_feed_forward(E, top, Fs):
    """Router weights from the logits plus bias (the softmax over the chosen alone) and the gated experts' hidden activations, put
    together with plain products, against the plain routed feed-forward."""
    from stride_b200.kernels import ops
    g = torch.Generator().manual_seed(E * 10 + top)
    n, W = 23, 24
    t = {"p.router": torch.randn(E, W, generator=g), "p.router.b": torch.randn(E, generator=g)}
    for e in range(E):
        t[f"p.e{e}.gate"], t[f"p.e{e}.up"] = torch.randn(Fs, W, generator=g) * 0.4, torch.randn(Fs, W, generator=g) * 0.4
        t[f"p.e{e}.down"] = torch.randn(W, Fs, generator=g) * 0.3
    h = torch.randn(n, W, generator=g)
    want = plain.routed_experts(h.double(), t, "p.", {"router": {"experts": E, "top": top}})
    logits = (h.double() @ t["p.router"].double().T).float().to(DEV)
    weights = torch.empty(n, E, device=DEV)
    ops.moe_route(logits, t["p.router.b"].to(DEV), weights, top, 1.0, biased=True)
    assert int((weights != 0).sum(1).min()) == int((weights != 0).sum(1).max()) == top
    assert (weights.sum(1).cpu() - 1.0).abs().max() <= 1e-5
    z = h.double() @ t["p.router"].double().T + t["p.router.b"].double()
    chosen = torch.zeros(n, E, dtype=torch.bool).scatter_(1, torch.topk(z, top, dim=1).indices, True)
    assert torch.equal(weights.cpu() != 0, chosen)
    rows = torch.cat([torch.cat([t[f"p.e{e}.gate"], t[f"p.e{e}.up"]]) for e in range(E)], 0)       # an expert's gate rows above its up rows
    up = (h.double() @ rows.double().T).float()
    parts = torch.stack([up * 0.25, up * 0.75]).to(DEV)
    mid = torch.empty(n, E * Fs, device=DEV)
    ops.moe_activate(parts, weights, mid, E, Fs, gated=True)
    down_all = torch.cat([t[f"p.e{e}.down"] for e in range(E)], 1)
    out = mid.cpu().double() @ down_all.double().T
    assert (out - want).abs().max() <= 2e-5 * float(want.abs().max())


def _identity_attention(H, G, D, V, g):
    """Tensors that let the plain attention read [q | k | v] straight from its input, with random biases, gains and sinks."""
    width = H * D + G * D + G * V
    eye = torch.eye(width)
    return {"p.q": eye[:H * D], "p.k": eye[H * D:H * D + G * D], "p.v": eye[H * D + G * D:], "p.o": torch.eye(H * V),
            "p.q.b": torch.randn(H * D, generator=g) * 0.3, "p.k.b": torch.randn(G * D, generator=g) * 0.3,
            "p.v.b": torch.randn(G * V, generator=g) * 0.3, "p.q.norm": 1.0 + 0.3 * torch.randn(H * D, generator=g),
            "p.k.norm": 1.0 + 0.3 * torch.randn(G * D, generator=g), "p.sink": torch.randn(H, generator=g)}, width


def _masked_case(H, G, D, V, window, keep, page, lengths, seed, dtype=torch.float32, tiles=False, peak=None, scale=0.3, quiet=False):
    """Requests of the given lengths appended in two steps each (the second step's queries read pages of the first), pages handed
    out in a shuffled order; returns the kernels' output and the plain result per request. `peak`: the key at that distance from the
    last query is made to fit the last query and its value made large, so that it alone decides the last row if it is seen. `quiet`:
    the queries' gains scaled down and their biases dropped, so that every visible key weighs about the same."""
    from stride_b200.kernels import ops
    g = torch.Generator().manual_seed(seed)
    row = max(D, V)
    t, width = _identity_attention(H, G, D, V, g)
    eps = 1e-5
    table, total = _table(lengths, page, 3, g)
    pages = torch.full((total, 2, G, page, row), 1e4, dtype=dtype, device=DEV)       # a row that nobody wrote would show if it were read
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=torch.float32, device=DEV)
    if quiet:
        t["p.q.b"], t["p.q.norm"] = torch.zeros(H * D), torch.full((H * D,), 0.02)
    bias = torch.cat([t["p.q.b"], t["p.k.b"], t["p.v.b"]]).to(DEV)
    rnd = None if dtype == torch.float32 else dtype
    outs, wants = [], []
    for r, n in enumerate(lengths):
        qkv = torch.randn(n, width, generator=g)
        if peak is not None and n - 1 - peak >= 0:          # (as many key heads as query heads)
            far = n - 1 - peak
            qkv[far, H * D:H * D + G * D] = qkv[n - 1, :H * D]
            qkv[far, H * D + G * D:] = 50.0
        cut = max(1, n // 3)
        got = []
        for a, b in ((0, cut), (cut, n)):
            if a == b:
                continue
            entries = [(r, 0, b - a, a)]
            pos, slot = _rows(entries)
            q = torch.empty(b - a, H * D, dtype=dtype, device=DEV)
            parts = torch.stack([qkv[a:b] * 0.5, qkv[a:b] * 0.5]).to(DEV)
            ops.qkv_norm_append(parts, bias, t["p.q.norm"].to(DEV), t["p.k.norm"].to(DEV), eps, pos, slot, q, pages, table, H, G, D, V)
            out = torch.empty(b - a, H * V, dtype=dtype, device=DEV)
            if tiles:
                ops.masked_attention_tiles(q, out, pages, table, _meta(entries), 1, slopes, t["p.sink"].to(DEV), H, G, D, V, window, keep, scale)
            else:
                ops.masked_attention(q, out, pages, table, pos, slot, slopes, t["p.sink"].to(DEV), H, G, D, V, window, keep, scale)
            got.append(out.cpu())
        outs.append(torch.cat(got))
        m = {"heads": H, "kv_heads": G, "dim": D, "vdim": V, "scale": scale}
        if window:
            m["mask"] = {"size": window, "keep_first": keep}
        wants.append(plain.sink_attention(qkv.double(), t, "p.", m, eps, rnd))
    return outs, wants


MASKED_SHAPES = [(4, 2, 32, 24, 24, 5, 16), (2, 2, 48, 64, 7, 0, 8), (8, 2, 64, 64, 100, 33, 32), (2, 1, 128, 96, 0, 0, 16), (5, 5, 20, 12, 1, 3, 8),
                 (3, 1, 12, 200, 33, 33, 16), (6, 1, 12, 36, 40, 64, 16)]


@pytest.mark.parametrize("H,G,D,V,window,keep,page", MASKED_SHAPES)
def test_masked_attention_kernels(H, G, D, V, window, keep, page):
    outs, wants = _masked_case(H, G, D, V, window, keep, page, [70, 3, 131], H * D + window)
    for got, want in zip(outs, wants):
        assert (got.double() - want).abs().max() <= 2e-5 * float(want.abs().max())


@pytest.mark.parametrize("tiles", [False, True])
@pytest.mark.parametrize("distance,seen", [(23, True), (24, False), (135, True), (134, False), (139, True), (130, False), (25, False), (0, True)])
def test_a_key_at_a_window_or_kept_edge_decides_the_row(distance, seen, tiles):
    """Window 24, the first 5 tokens kept, 140 tokens in pages of 16: the key 23 back is the window's last, the key 24 back its first
    outside; the key 135 back is token 4, the last kept one, the key 134 back token 5, the first that is not kept. The marked key's
    value is 50 and its key fits the last query, so the last row is about 50 (in the heads whose slope leaves a key that far back
    any weight) when it is seen and stays small when it is not."""
    dtype = torch.bfloat16 if tiles else torch.float32
    outs, wants = _masked_case(4, 4, 32, 16, 24, 5, 16, [140], 7, dtype=dtype, tiles=tiles, peak=distance, scale=1.0)
    got, want = outs[0].double(), wants[0]
    assert (float(want[-1].abs().max()) > 25.0) == seen
    tol = 2e-5 if not tiles else 2.0 ** -7
    assert (got - want).abs().max() <= tol * float(want.abs().max())


@pytest.mark.parametrize("H,G,D,V,window,keep,page", [(8, 2, 64, 64, 100, 33, 32), (4, 2, 32, 48, 24, 5, 16), (2, 2, 96, 96, 72, 0, 64),
                                                      (16, 1, 16, 128, 0, 0, 8), (8, 4, 32, 80, 90, 21, 16), (4, 4, 256, 16, 200, 1, 16),
                                                      (32, 1, 16, 32, 50, 3, 16), (64, 2, 32, 16, 0, 0, 32)])
def test_masked_attention_on_the_tensor_cores(H, G, D, V, window, keep, page):
    """The bfloat16 tile kernel against the plain attention that rounds q, k and v to bfloat16 (its weights stay 32-bit), and against
    the kernel with a block per token and head on the same inputs; with queries scaled down, so that every visible key weighs alike
    and one key too many or too few would move the result."""
    from stride_b200.kernels import ops
    assert ops.masked_attention_tiles_supported(H, G, D, V, max(D, V), G * page * max(D, V))
    for quiet in (False, True):
        tiled, wants = _masked_case(H, G, D, V, window, keep, page, [300, 70, 2], H + D + V, dtype=torch.bfloat16, tiles=True, quiet=quiet)
        simple, _ = _masked_case(H, G, D, V, window, keep, page, [300, 70, 2], H + D + V, dtype=torch.bfloat16, tiles=False, quiet=quiet)
        for a, b, want in zip(tiled, simple, wants):
            top = float(want.abs().max())
            assert (a.double() - want).abs().max() <= 2.0 ** -7 * top                    # one bfloat16 step of the output
            assert (a.double() - b.double()).abs().max() <= 2.0 ** -7 * top


@pytest.mark.parametrize("H,D,R,V,Q,C,page,scaling", [(3, 20, 12, 28, 36, 44, 16, (8.0, 64, 16.0, 2.0)), (8, 32, 32, 32, 64, 96, 32, (2.0, 128, 8.0, 1.0)),
                                                      (2, 16, 16, 64, 32, 48, 8, None), (1, 8, 4, 8, 8, 16, 8, (4.0, 32, 4.0, 0.5)),
                                                      (4, 48, 16, 40, 72, 112, 16, (3.0, 256, 24.0, 1.5))])
def test_latent_attention_kernels(H, D, R, V, Q, C, page, scaling):
    """The latents normed and the shared rotated key part appended as one row per token, the queries' rotated slices, the key
    projection taken into the queries, attention over the latent rows, the value projection behind it: against the plain latent
    attention, which builds every head's keys and values. 32-bit, and bfloat16 (with the tensor-core form where the shape has one)
    against the plain form that rounds at the same places."""
    from stride_b200.kernels import ops
    from stride_b200.parts.rope import yarn_frequencies
    g = torch.Generator().manual_seed(H * D + C)
    W, eps, base = 40, 1e-5, 900.0
    scale = 1.5 / (0.09 * math.sqrt(Q * C * (D + R)))                 # scores of a spread of about 1.5: a softmax that is neither flat nor one key
    t = {"p.dq": torch.randn(Q, W, generator=g) * 0.3, "p.dq.norm": 1.0 + 0.3 * torch.randn(Q, generator=g), "p.uq": torch.randn(H * (D + R), Q, generator=g) * 0.3,
         "p.dkv": torch.randn(C + R, W, generator=g) * 0.3, "p.dkv.norm": 1.0 + 0.3 * torch.randn(C, generator=g),
         "p.uk": torch.randn(H * D, C, generator=g) * 0.3, "p.uv": torch.randn(H * V, C, generator=g) * 0.3, "p.o": torch.eye(H * V)}
    m = {"heads": H, "dim": D, "rot_dim": R, "vdim": V, "q_rank": Q, "kv_rank": C, "scale": scale, "rot": {"dims": R, "base": base}}
    if scaling:
        m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
        inv, mag = yarn_frequencies(R, base, *scaling)
        inv = torch.tensor(inv, dtype=F)
    else:
        inv, mag = torch.tensor([base ** (-2.0 * i / R) for i in range(R // 2)], dtype=F), 1.0
    lengths = [70, 3, 131]
    angle = torch.arange(max(lengths), dtype=F)[:, None] * inv[None, :]
    cos_sin = (torch.stack([torch.cos(angle), torch.sin(angle)], -1) * mag).float().to(DEV)
    for dtype in (torch.float32, torch.bfloat16):
        t16 = {k: (v if dtype == torch.float32 else v.to(dtype).float()) for k, v in t.items()}       # weights the engine would hold
        row = C + R
        table, total = _table(lengths, page, 2, g)
        pages = torch.full((total, 1, 1, page, row), 1e4, dtype=dtype, device=DEV)
        uk = t16["p.uk"].to(dtype).view(H, D, C).contiguous().to(DEV)
        uv = t16["p.uv"].to(dtype).view(H, V, C).transpose(1, 2).contiguous().to(DEV)
        tiles = dtype == torch.bfloat16 and ops.masked_attention_tiles_supported(H, 1, row, C, row, 0)
        for r, n in enumerate(lengths):
            h = torch.randn(n, W, generator=g)
            hh = h if dtype == torch.float32 else h.to(dtype).float()
            want = plain.latent_attention(hh.double(), t16, "p.", m, eps, None if dtype == torch.float32 else dtype)
            down = torch.cat([t16["p.dq"], t16["p.dkv"]]).double()
            proj_all = (hh.double() @ down.T).float()
            cut = max(1, n // 3)
            got = []
            for a, b in ((0, cut), (cut, n)):
                if a == b:
                    continue
                k = b - a
                entries = [(r, 0, k, a)]
                pos, slot = _rows(entries)
                proj = torch.stack([proj_all[a:b] * 0.5, proj_all[a:b] * 0.5]).to(DEV)
                cq = torch.empty(k, Q, dtype=dtype, device=DEV)
                ops.latent_prepare(proj, t["p.dq.norm"].to(DEV), t["p.dkv.norm"].to(DEV), eps, pos, slot, cos_sin, cq, pages, table, Q, C, R)
                qp = (cq.cpu().double() @ t16["p.uq"].double().T).float().to(DEV).unsqueeze(0)
                q = torch.empty(k, H, D + R, dtype=dtype, device=DEV)
                ops.rotate_heads(qp, pos, cos_sin, q.view(k, H * (D + R)), H, D + R, D, R)
                ql = torch.empty(k, H, row, dtype=dtype, device=DEV)
                ops.head_linear(q, uk, ql, tail=R)
                ol = torch.empty(k, H, C, dtype=dtype, device=DEV)
                if tiles:
                    ops.masked_attention_tiles(ql.view(k, H * row), ol.view(k, H * C), pages, table, _meta(entries), 1, None, None, H, 1, row, C, 0, 0, scale)
                else:
                    ops.masked_attention(ql.view(k, H * row), ol.view(k, H * C), pages, table, pos, slot, None, None, H, 1, row, C, 0, 0, scale)
                out = torch.empty(k, H, V, dtype=dtype, device=DEV)
                ops.head_linear(ol, uv, out)
                got.append(out.view(k, H * V).cpu())
            got = torch.cat(got).double()
            # bfloat16: the kernels round the query in the latent's coordinates and the result there, the plain form the heads' own: the
            # two deviate from the exact result independently, each by about the plain form's own rounding noise on the same input
            top = float(want.abs().max())
            tol = 2e-5 * top if dtype == torch.float32 else max(2.0 * float((want - plain.latent_attention(hh.double(), t16, "p.", m, eps)).abs().max()),
                                                                2.0 ** -6 * top)
            assert (got - want).abs().max() <= tol, f"{dtype} request {r}"
            if dtype == torch.bfloat16:
                assert (got - want).abs().mean() <= 2.0 ** -8 * top


def test_head_linear_strides_and_tail():
    """A matrix per head on views with any row and head strides; the tail is copied behind the product."""
    from stride_b200.kernels import ops
    g = torch.Generator().manual_seed(3)
    n, H, K, N, tail = 7, 3, 10, 6, 4
    big = torch.randn(n, H, K + tail + 5, generator=g).to(DEV)
    w = torch.randn(H, K, N, generator=g).to(DEV)
    out = torch.zeros(n, H, N + tail + 2, device=DEV)
    ops.head_linear(big[:, :, :K + tail], w, out[:, :, :N + tail], tail=tail)
    want = torch.einsum("rhk,hkn->rhn", big[:, :, :K].double().cpu(), w.double().cpu())
    assert (out[:, :, :N].cpu().double() - want).abs().max() <= 1e-5 * float(want.abs().max())
    assert torch.equal(out[:, :, N:N + tail], big[:, :, K:K + tail]) and float(out[:, :, N + tail:].abs().max()) == 0.0


# ---------------------------------------------------------------------------------------------- whole models
def _engine(model_dir, dtype, page, pages, rows=256, slots=4, **kw):
    from stride_b200.engine.engine import Engine, EngineOptions
    return Engine(model_dir, EngineOptions(dtype=dtype, max_rows=rows, max_full_rows=rows, max_slots=slots, kv_pages=pages,
                                           page_size=page, max_context=pages * page, device=DEV, **kw))


def _noise(cfg, w, tokens):
    """max and mean |plain with bfloat16 rounding - plain exact| over the sequence's logits."""
    d = (plain.forward(cfg, w, tokens, torch.bfloat16) - plain.forward(cfg, w, tokens)).abs()
    return float(d.max()), float(d.mean())


CLOSE_CALL = 0.1       # a router logit's lead below this is within what bfloat16 rounding on the way to the router moves a logit by


def _close_calls(cfg, w, tokens):
    """Per position: True where some routed layer chooses its experts by a lead that bfloat16 rounding can overturn. There two
    right implementations that round at different places may choose different experts."""
    leads = []
    plain.forward(cfg, w, tokens, leads=leads)
    if not leads:
        return torch.zeros(len(tokens), dtype=torch.bool)
    return torch.stack(leads).min(0).values < CLOSE_CALL


def _after_close_calls(close):
    """Attention carries a changed choice forward, thinly (one key among many): True from the first close call on."""
    out = close.clone()
    hit = torch.nonzero(close)
    if hit.numel():
        out[int(hit[0]):] = True
    return out


def test_every_layer_run_against_the_plain_streams(pusisun_dirs):
    """The residual stream after every run of a layer (a looped layer once per pass), in 32-bit, for a prompt in one step."""
    from stride_b200.engine.engine import StepEntry
    for name in ("X", "Y", "Z"):
        cfg, w = load_plain(pusisun_dirs[name])
        page = PUSISUN[name][2]
        toks = random_tokens(cfg["vocab"], 37, 12)
        streams = []
        plain.forward(cfg, w, toks, streams=streams)
        eng = _engine(pusisun_dirs[name], "float32", page, 8, native_step=False)
        slot = eng.cache.acquire_slot()
        eng.cache.ensure(slot, len(toks))
        seen = []
        for block, layer in zip(eng.model.blocks, eng.model.spec.layers):
            if layer.block == "rewrite":              # what stands in front of a pass is no layer run
                continue

            def run(ctx, stream, cache, inner=block.forward):
                inner(ctx, stream, cache)
                stream.fold()
                seen.append(stream.h[:len(toks)].detach().cpu().double().clone())
            block.forward = run
        eng.step([StepEntry(slot, 0, toks, list(range(len(toks))))])
        assert len(seen) == len(streams)
        for k, (got, want) in enumerate(zip(seen, streams)):
            assert (got - want).abs().max() <= 2e-4 * max(1.0, float(want.abs().max())), f"{name}: the stream after layer run {k} differs"


LENGTHS = {"X": [70, 130, 45, 33, 2], "Y": [300, 65, 140, 129, 40], "Z": [48, 90, 17, 64, 5]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["X", "Y", "Z"])
def test_replay_modes(name, dtype, pusisun_dirs, tmp_path):
    """Through bin/trace_run: whole; all but the last 32 tokens, then token by token; portions down to two tokens; mixed batches in
    a pool so small that pages are used again, four slots for five requests. Against the plain implementation, and all four in the
    same bits. float32: the framework's yardstick. bfloat16: the engine and the plain implementation with bfloat16 rounding do not
    round at the same places everywhere (the latent attention's queries and results are rounded in the latent's coordinates), so both
    deviate from the exact logits by about the rounding noise, independently. Up to a request's first close call of a router the
    largest deviation between the two stays within twice the largest rounding noise of the same sequence; over the whole request,
    where a choice of experts may have gone the other way at some positions, the median over the positions of the largest deviation
    does too, and the median of the mean error against the exact logits stays within twice the mean rounding noise. The other three
    ways of feeding a request are held to the bits of the first."""
    cfg, _, page = PUSISUN[name]
    vocab = cfg["vocab"]
    reqs = [random_tokens(vocab, n, 300 + i) for i, n in enumerate(LENGTHS[name])]
    pcfg, w = load_plain(pusisun_dirs[name])
    rnd = None if dtype == "float32" else torch.bfloat16
    exact = [plain.forward(pcfg, w, r).float() for r in reqs]
    want = exact if rnd is None else [plain.forward(pcfg, w, r, rnd).float() for r in reqs]
    noise = [None if rnd is None else _noise(pcfg, w, r) for r in reqs]
    close = [None if rnd is None else _after_close_calls(_close_calls(pcfg, w, r)) for r in reqs]
    per = lambda n: -(-n // page) * page
    longest = sorted((per(len(r)) for r in reqs), reverse=True)
    pool = max(longest[0] + longest[1] + page, 4 * page)
    tr = TraceRun(pusisun_dirs[name], dtype, tmp_path, pool, page, extra=("--kv-shuffle", "5"))
    bits = _Bits()

    def compare(got, i, a, b, what):
        tol = logit_tolerance(dtype, want[i]) if noise[i] is None else 2.0 * noise[i][0]
        diff = (got - want[i][a:b]).abs()
        if close[i] is not None:
            if b - a == len(reqs[i]):
                worst = diff.max(dim=1).values.median()
                assert worst <= tol, f"{name} {what}: the median over positions of max |diff| {worst:.3e} > {tol:.3e}"
                mean = (got - exact[i]).abs().mean(dim=1).median()
                assert mean <= 2.0 * noise[i][1], f"{name} {what}: median of the mean error {mean:.3e} > twice the mean rounding noise {noise[i][1]:.3e}"
            diff = diff[~close[i][a:b]]
            if diff.numel() == 0:
                return bits.check(i, a, got, f"{name} {what}")
        assert diff.max() <= tol, f"{name} {dtype} {what}: max |diff| {diff.max():.3e} > {tol:.3e} at {a + int(diff.max(dim=1).values.argmax())}"
        bits.check(i, a, got, f"{name} {what}")

    try:
        for i, r in enumerate(reqs):
            s = tr.run([(f"w{i}", r, range(len(r)))], end=[f"w{i}"])
            compare(tr.logits(s, vocab), i, 0, len(r), f"whole request {i}")
        for i, r in enumerate(reqs):
            cut = max(1, len(r) - 32)
            s = tr.run([(f"d{i}", r[:cut], [cut - 1])], end=[f"d{i}"] if cut == len(r) else [])
            compare(tr.logits(s, vocab), i, cut - 1, cut, f"request {i} prefill end")
            for p in range(cut, len(r)):
                s = tr.run([(f"d{i}", r[p:p + 1], [0])], end=[f"d{i}"] if p == len(r) - 1 else [])
                compare(tr.logits(s, vocab), i, p, p + 1, f"request {i} decode at {p}")
        for i, r in enumerate(reqs):
            cuts = _portions(len(r), [7, 2, 19, 3, 2, 31, 5])
            for j, (a, b) in enumerate(cuts):
                s = tr.run([(f"p{i}", r[a:b], range(b - a))], end=[f"p{i}"] if j == len(cuts) - 1 else [])
                compare(tr.logits(s, vocab), i, a, b, f"request {i} portion {a}:{b}")
        fed, turn = [0] * len(reqs), [0] * len(reqs)
        sizes = [[9, 1, 1, 4, 1], [2, 13, 1, 1, 1, 6], [5, 1, 1, 1], [17, 1, 2, 1, 1], [3, 1, 8, 1]]
        live, waiting, steps = [], list(range(len(reqs))), 0
        while live or waiting:
            while waiting and len(live) < 4 and sum(per(len(reqs[i])) for i in live) + per(len(reqs[waiting[0]])) <= pool:
                live.append(waiting.pop(0))
            entries, ends, spans = [], [], []
            for k, i in enumerate(list(live)):
                if (steps + k) % 5 == 4 and len(live) > 1:
                    continue
                n = min(sizes[i][turn[i] % len(sizes[i])], len(reqs[i]) - fed[i])
                turn[i] += 1
                a, b = fed[i], fed[i] + n
                entries.append((f"m{i}", reqs[i][a:b], range(n)))
                spans.append((i, a, b))
                fed[i] = b
                if b == len(reqs[i]):
                    ends.append(f"m{i}")
                    live.remove(i)
            s = tr.run(entries, end=ends)
            got, at = tr.logits(s, vocab), 0
            for i, a, b in spans:
                compare(got[at:at + b - a], i, a, b, f"mixed step {steps} request {i} {a}:{b}")
                at += b - a
            steps += 1
    finally:
        tr.close()


def test_window_and_kept_edges_show_and_agree(pusisun_dirs):
    """With attention close to uniform every visible key carries weight: the plain implementation itself moves by far more than
    the tolerance when a window is one token longer or shorter or one first token more or fewer is kept. The engine agrees with the
    right masks at every position, in a prompt whose windows straddle pages and decoding token by token with pages trimmed behind
    the windows (the kept first tokens' pages stay)."""
    from stride_b200.engine.engine import StepEntry
    cfg, w = load_plain(pusisun_dirs["XU"])
    toks = random_tokens(cfg["vocab"], 90, 77)
    want = plain.forward(cfg, w, toks).float()
    tol = logit_tolerance("float32", want)
    for key, delta in (("size", 1), ("size", -1), ("keep_first", 1), ("keep_first", -1)):
        other = copy.deepcopy(cfg)
        other["layers"][0]["mixer"]["mask"][key] += delta
        moved = (plain.forward(other, w, toks).float() - want).abs().max(dim=1).values
        assert moved[40:].min() > 20 * tol, f"the yardstick does not notice {key} {delta:+d}"
    eng = _engine(pusisun_dirs["XU"], "float32", 16, 12)
    slot = eng.cache.acquire_slot()
    eng.cache.ensure(slot, 50)
    got = [eng.step([StepEntry(slot, 0, toks[:50], list(range(50)))]).cpu().clone()]
    for t in range(50, 90):
        eng.cache.ensure(slot, t + 1)
        got.append(eng.step([StepEntry(slot, t, [toks[t]], [0])]).cpu().clone())
        eng.cache.trim(slot)
    assert (torch.cat(got) - want).abs().max() <= tol
    eng.cache.check()


def test_the_first_tokens_of_a_sequence(pusisun_dirs):
    """Positions 0, 1, 2, .. one by one in a slot that another request used: a window with fewer keys than its size, kept tokens
    that are all there is, a sink beside a single key, position 0 of the rotation."""
    from stride_b200.engine.engine import StepEntry
    for name, page in (("Z", 8), ("X", 16)):
        cfg, w = load_plain(pusisun_dirs[name])
        eng = _engine(pusisun_dirs[name], "float32", page, 16)
        for seed in (3, 4):
            toks = random_tokens(cfg["vocab"], 12, seed)
            want = plain.forward(cfg, w, toks).float()
            slot = eng.cache.acquire_slot()
            got = []
            for t in range(12):
                eng.cache.ensure(slot, t + 1)
                got.append(eng.step([StepEntry(slot, t, [toks[t]], [0])]).cpu().clone())
            assert (torch.cat(got) - want).abs().max() <= logit_tolerance("float32", want)
            eng.cache.release_slot(slot)


def test_long_decoding_and_slot_reuse(pusisun_dirs):
    """A short prompt, then 400 tokens one by one (every window passes over decoded tokens, pages behind the windows are given back
    while the kept first tokens' pages stay, the latent layers see every token), against the plain implementation; then the same slot
    again for another request, which must not see what the first left."""
    from stride_b200.engine.engine import StepEntry
    cfg, w = load_plain(pusisun_dirs["XU"])
    eng = _engine(pusisun_dirs["XU"], "float32", 16, 30)
    for seed in (1, 2):
        toks = random_tokens(cfg["vocab"], 410, seed)
        want = plain.forward(cfg, w, toks).float()
        slot = eng.cache.acquire_slot()
        assert slot == 0 or seed == 1
        eng.cache.ensure(slot, 10)
        got = [eng.step([StepEntry(slot, 0, toks[:10], list(range(10)))]).cpu().clone()]
        for t in range(10, 410):
            eng.cache.ensure(slot, t + 1)
            got.append(eng.step([StepEntry(slot, t, [toks[t]], [0])]).cpu().clone())
            eng.cache.trim(slot)
        assert (torch.cat(got) - want).abs().max() <= logit_tolerance("float32", want)
        eng.cache.release_slot(slot)
        eng.cache.check()


def test_a_far_key_among_hundreds_shows(pusisun_dirs, tmp_path):
    """The latent layers see every earlier token. One early token's embedding is made large, so that it stands out among some 300
    keys: another token in its place moves the plain logits 300 tokens later far beyond the tolerance, and the engine, fed in
    portions that cut pages and then token by token, agrees with the whole sequence."""
    from stride_b200.engine.engine import StepEntry

    def loud(tensors):
        near_uniform(tensors)
        e = tensors["embed"].float()
        e[7] *= 6.0
        tensors["embed"] = e.to(tensors["embed"].dtype)

    folder = write_model(tmp_path / "far", "Y", transform=loud)
    cfg, w = load_plain(folder)
    toks = [t if t != 7 else 8 for t in random_tokens(cfg["vocab"], 330, 21)]
    toks[13] = 7
    want = plain.forward(cfg, w, toks).float()
    tol = logit_tolerance("float32", want)
    other = list(toks)
    other[13] = 8
    assert (plain.forward(cfg, w, other).float()[-20:] - want[-20:]).abs().max(dim=1).values.min() > 20 * tol
    eng = _engine(folder, "float32", 32, 14)
    slot = eng.cache.acquire_slot()
    got, at = [], 0
    for n in (45, 2, 150, 83, 3, 17):
        eng.cache.ensure(slot, at + n)
        got.append(eng.step([StepEntry(slot, at, toks[at:at + n], list(range(n)))]).cpu().clone())
        eng.cache.trim(slot)
        at += n
    for t in range(at, len(toks)):
        eng.cache.ensure(slot, t + 1)
        got.append(eng.step([StepEntry(slot, t, [toks[t]], [0])]).cpu().clone())
        eng.cache.trim(slot)
    assert (torch.cat(got) - want).abs().max() <= tol


@pytest.mark.parametrize("native", [True, False])
def test_batches_of_unequal_requests_against_each_alone(pusisun_dirs, native):
    """Four requests of unequal length in one step, then single tokens of some beside portions of others: every logit has the
    bits of the request run alone; the native step program and the part-by-part driver agree."""
    from stride_b200.engine.engine import StepEntry
    cfg, _, page = PUSISUN["Y"]
    reqs = [random_tokens(cfg["vocab"], n, 40 + n) for n in (150, 3, 64, 31)]
    for dtype in ("float32", "bfloat16"):
        eng = _engine(pusisun_dirs["Y"], dtype, page, 24, native_step=native)
        assert (eng._program is not None) == native
        alone = []
        for r in reqs:
            slot = eng.cache.acquire_slot()
            eng.cache.ensure(slot, len(r))
            alone.append(eng.step([StepEntry(slot, 0, r, list(range(len(r))))]).cpu().clone())
            eng.cache.release_slot(slot)
        slots = [eng.cache.acquire_slot() for _ in reqs]
        fed, got = [0] * 4, [[] for _ in reqs]
        plan = [[100, 2, 30, 1], [1, 1, 20, 30], [49, 0, 1, 0], [1, 1, 13, 0]]      # tokens of each request per step; then one by one
        step = 0
        while any(fed[i] < len(reqs[i]) for i in range(4)):
            entries, who = [], []
            for i, r in enumerate(reqs):
                n = plan[step][i] if step < len(plan) else 1
                n = min(n, len(r) - fed[i])
                if n > 0:
                    eng.cache.ensure(slots[i], fed[i] + n)
                    entries.append(StepEntry(slots[i], fed[i], r[fed[i]:fed[i] + n], list(range(n))))
                    who.append((i, n))
                    fed[i] += n
            out, at = eng.step(entries).cpu(), 0
            for i, n in who:
                got[i].append(out[at:at + n].clone())
                at += n
            step += 1
        for i in range(4):
            assert torch.equal(torch.cat(got[i]), alone[i]), f"{dtype}: request {i} in company differs from the request alone"


def test_greedy_generation_through_the_entry_point(pusisun_dirs):
    """LLM.generate with its scheduler (three requests on two slots, prompts cut into portions, decode steps replayed from CUDA
    graphs): the tokens of greedy decoding with the plain implementation."""
    from stride_b200 import LLM
    cfg, w = load_plain(pusisun_dirs["X"])
    prompts = [random_tokens(cfg["vocab"], n, 500 + n) for n in (5, 41, 23)]
    llm = LLM(pusisun_dirs["X"], dtype="float32", concurrency=2, max_rows=32, prefill_chunk=8, kv_pages=12, page_size=16,
              max_slots=2, max_context=128, device=DEV)
    outs = llm.generate(prompts, max_new_tokens=12)
    for p, o in zip(prompts, outs):
        seq = list(p)
        for tok in o.tokens:
            ref = plain.forward(cfg, w, seq)[-1]
            top = torch.topk(ref, 2).values
            if float(top[0] - top[1]) > 1e-3:       # (a near tie may go either way)
                assert tok == int(ref.argmax())
            seq.append(tok)
        assert len(o.tokens) == 12 and o.finish_reason == "length"
    bf = LLM(pusisun_dirs["Y"], dtype="bfloat16", concurrency=4, max_rows=64, prefill_chunk=16, kv_pages=16, page_size=32,
             max_slots=4, max_context=256, device=DEV)
    cfgy = PUSISUN["Y"][0]
    outs = bf.generate([random_tokens(cfgy["vocab"], n, n) for n in (70, 9, 33, 120, 64)], max_new_tokens=8)
    assert all(len(o.tokens) == 8 for o in outs)


def test_command_line_generates_what_the_entry_point_generates(pusisun_dirs, tmp_path):
    """bin/stride_cli on a Pusisun folder (greedy, float32 and bfloat16): the tokens of LLM.generate."""
    import json
    import subprocess
    import sys
    from conftest import ROOT
    from stride_b200 import LLM
    cfg = PUSISUN["Z"][0]
    prompts = [random_tokens(cfg["vocab"], n, 900 + n) for n in (3, 50, 21)]
    (tmp_path / "in.jsonl").write_text("".join(json.dumps({"id": i, "tokens": p}) + "\n" for i, p in enumerate(prompts)))
    for path, dtype in (("exact", "float32"), ("tc", "bfloat16")):
        out = tmp_path / f"out_{path}.jsonl"
        subprocess.run([sys.executable, str(ROOT / "bin" / "stride_cli"), "--model", str(pusisun_dirs["Z"]), "--input", str(tmp_path / "in.jsonl"),
                        "--output", str(out), "--max-new", "6", "--concurrency", "2", "--max-rows", "32", "--prefill-chunk", "16",
                        "--kv-blocks", "24", "--page-size", "8", "--max-slots", "4", "--max-context", "128", "--path", path], check=True, timeout=600)
        got = [json.loads(l) for l in out.read_text().splitlines()]
        llm = LLM(pusisun_dirs["Z"], dtype=dtype, concurrency=2, max_rows=32, prefill_chunk=16, kv_pages=24, page_size=8, max_slots=4,
                  max_context=128, device=DEV)
        want = llm.generate(prompts, max_new_tokens=6)
        assert [g["tokens"] for g in got] == [w.tokens for w in want] and all(g["finish"] == "length" for g in got)
