"""Sitivik through the engine against the plain implementation (tests/plain_sitivik.py): every mechanism's part alone, with caches made
by hand, cut into steps of one, two and more tokens beside one another; then whole models of three tiny configurations whole, decoded
token by token, in portions down to two tokens and in mixed batches with pages and slots used again, in 32-bit and in bfloat16; window
and chunk edges, the sink and far tokens made to show; long decoding; batches against each request alone; greedy generation through the
entry point, its scheduler and the command line."""
from __future__ import annotations

import copy

import pytest
import torch

import plain_sitivik as plain
from conftest import TraceRun, logit_tolerance, random_tokens
from sitivik_cases import SITIVIK, load_plain, near_uniform, write_model
from test_replay_gpu import _Bits, _portions

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F = torch.float64
ROWS = 256


@pytest.fixture(scope="module")
def sitivik_dirs(tmp_path_factory):
    root = tmp_path_factory.mktemp("sitivik")
    out = {name: write_model(root / name, name) for name in SITIVIK}
    out["XU"] = write_model(root / "XU", "X", transform=near_uniform)
    return out


# ---------------------------------------------------------------------------------------------- a step made by hand
class _Step:
    """A step's integer inputs in one device buffer, in the step program's layout, and the context over it."""

    def __init__(self, entries, dtype, workspace, tokens=None):
        from stride_b200.parts import StepContext
        R, n = ROWS, sum(e[2] for e in entries)
        ints = torch.zeros(9 * R + 64, dtype=torch.int32)
        at = 0
        for k, (slot, _, length, first) in enumerate(entries):
            ints[R + at:R + at + length] = torch.arange(first, first + length, dtype=torch.int32)
            ints[2 * R + at:2 * R + at + length] = slot
            for j, v in enumerate((slot, at, length, first)):
                ints[4 * R + j * R + k] = v
            at += length
        if tokens is not None:
            ints[:n] = torch.tensor(tokens, dtype=torch.int32)
        self.ints = d = ints.to(DEV)
        E = len(entries)
        self.ctx = StepContext(n=n, token_ids=d[0:n], positions=d[R:R + n], slots=d[2 * R:2 * R + n], workspace=workspace, compute_dtype=dtype,
                               entry_slots=[e[0] for e in entries], entry_first_row=[0] * E, entry_length=[e[2] for e in entries],
                               entry_first_pos=[e[3] for e in entries], entry_meta=d[4 * R:8 * R].view(4, R)[:, :E])


def _env(dtype):
    from stride_b200.parts import BuildEnv
    return BuildEnv(device=torch.device(DEV), compute_dtype=dtype, max_tokens=ROWS, max_positions=1024)


def _mixer_spec(name, layer, member=None):
    """The PartSpec of a layer's mixer (or of one member of its two), as the product's own reader makes it from the configuration."""
    from stride_b200.config import resolve_architecture
    cfg = SITIVIK[name][0]
    arch = resolve_architecture(cfg)
    spec = arch.model_spec(arch.parse_config(cfg)).layers[layer].parts["mixer"]
    return spec if member is None else spec.params["members"][member]


def _cache_for(need, slots, page, positions, g):
    """A LayerCache made by hand for one need: pages handed out in a shuffled order and full of large numbers, or state records full of
    large numbers (a request's first step must not read them)."""
    from stride_b200.cache.manager import LayerCache
    if need.kind == "state":
        return LayerCache(state=torch.full((slots + 1, *need.state_shape), 1e4, dtype=torch.float32, device=DEV))
    per = -(-positions // page)
    total = slots * per + 3
    perm = torch.randperm(total, generator=g)[:slots * per].view(slots, per).to(torch.int32)
    pages = torch.full((total, need.planes, need.kv_heads, page, need.head_dim), 1e4, dtype=need.dtype, device=DEV)
    return LayerCache(pages=pages, block_table=perm.to(DEV).contiguous(), page_size=page)


def _run_member(spec, tensors, dtype, h, schedule, page):
    """The mixer of `spec` over requests whose normed inputs are `h[r]`, fed as `schedule` says: a list of steps, each a list of
    (request, tokens). Returns one result [T_r, width] per request (what the mixer adds to the stream)."""
    from stride_b200.parts import ResidualStream, Workspace, part_class
    env = _env(dtype)
    part = part_class("mixer", spec.kind)(spec, env)
    part.bind({n: tensors[n].to(DEV) for n in part.tensor_plan()})
    g = torch.Generator().manual_seed(7)
    cache = _cache_for(part.cache_need(), len(h), page, max(len(x) for x in h), g)
    ws = Workspace(DEV, ROWS)
    fed, out = [0] * len(h), [[] for _ in h]
    W = h[0].shape[1]
    for step in schedule:
        entries, rows, at = [], [], 0
        for r, n in step:
            entries.append((r, at, n, fed[r]))
            rows.append(h[r][fed[r]:fed[r] + n])
            at += n
        st = _Step(entries, dtype, ws)
        x = ws.get("block.x", at, (W,), dtype)
        x.copy_(torch.cat(rows).to(DEV, dtype))
        buf = ws.get("test.out", at, (W,), torch.float32)
        buf.zero_()
        stream = ResidualStream(buf)
        part.forward(st.ctx, x, stream, cache)
        stream.fold()
        got, at = stream.h.cpu().double(), 0
        for r, n in step:
            out[r].append(got[at:at + n].clone())
            fed[r] += n
            at += n
    assert all(fed[r] == len(h[r]) for r in range(len(h)))
    return [torch.cat(o) for o in out]


def _schedules(lengths):
    """Whole requests side by side; and: portions of unequal size, two tokens, single tokens, a request that joins late."""
    whole = [[(r, n) for r, n in enumerate(lengths)]]
    left, cut, turn = list(lengths), [], 0
    sizes = [[9, 1, 2, 30, 1, 1], [2, 2, 1, 17, 1], [1, 1, 1, 40]]
    while any(left):
        step = []
        for r in range(len(lengths)):
            if left[r] and not (r == 2 and turn < 2):
                n = min(sizes[r % 3][turn % len(sizes[r % 3])], left[r])
                step.append((r, n))
                left[r] -= n
        cut.append(step)
        turn += 1
    return whole, cut


MEMBERS = [("X", 0, None, "differential_attention"), ("X", 1, 0, "windowed_left"), ("X", 1, 1, "retention_right"), ("X", 2, 0, "chunked_left"),
           ("X", 2, 1, "delta_right"), ("Y", 0, 0, "chunked_left"), ("Y", 0, 1, "delta_right"), ("Y", 1, None, "differential_attention"),
           ("Y", 2, 0, "windowed_left"), ("Y", 2, 1, "retention_right"), ("Y", 3, 0, "windowed_left"), ("Z", 0, 0, "windowed_left"),
           ("Z", 0, 1, "retention_right"), ("Z", 1, 0, "chunked_left"), ("Z", 1, 1, "delta_right"), ("Z", 2, None, "differential_attention")]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name,layer,member,fn", MEMBERS)
def test_every_mixer_alone(name, layer, member, fn, dtype, sitivik_dirs):
    """One mixer with caches made by hand against its plain function: three requests of unequal length in one step, and cut into steps of
    1, 2 and more tokens beside one another (with a request that joins late), in pages handed out in a shuffled order and slots that hold
    large numbers. The cut run has the bits of the whole one."""
    cfg, w = load_plain(sitivik_dirs[name])
    from stride_b200.weights.safetensors_io import SafetensorsFile
    f = SafetensorsFile(sitivik_dirs[name] / "model.safetensors")
    tensors = {n: f.get(n).clone() for n in f.names()}
    f.close()
    spec = _mixer_spec(name, layer, member)
    m = cfg["layers"][layer]["mixer"]
    p = f"l{layer}.mix."
    if member is not None:
        m, p = m[("left", "right")[member]], p + ("left.", "right.")[member]
    g = torch.Generator().manual_seed(layer * 10 + (member or 0))
    lengths = [83, 38, 5]
    h = [torch.randn(n, cfg["width"], generator=g).to(dtype).float() for n in lengths]
    want = [getattr(plain, fn)(w, p, m, x.double(), cfg["norm"]["eps"], dtype == torch.bfloat16) for x in h]
    whole, cut = _schedules(lengths)
    page = SITIVIK[name][2]
    a = _run_member(spec, tensors, dtype, h, whole, page)
    b = _run_member(spec, tensors, dtype, h, cut, page)
    for r in range(len(lengths)):
        scale = float(want[r].abs().max())
        tol = 2e-4 * scale if dtype == torch.float32 else 0.06 * scale
        assert (a[r] - want[r]).abs().max() <= tol, f"{fn} of {name}, request {r}: {(a[r] - want[r]).abs().max():.3e} > {tol:.3e}"
        assert torch.equal(a[r], b[r]), f"{fn} of {name}, request {r}: cut into steps it differs from the whole at {int((a[r] != b[r]).any(1).nonzero()[0])}"


@pytest.mark.parametrize("tiles", [False, True])
@pytest.mark.parametrize("window,chunk,distance,seen", [(24, 0, 23, True), (24, 0, 24, False), (0, 40, 29, True), (0, 40, 30, False), (0, 40, 0, True),
                                                        (0, 0, 149, True), (100, 0, 99, True), (100, 0, 100, False), (0, 64, 21, True), (0, 64, 22, False)])
def test_a_key_at_a_window_or_chunk_edge_decides_the_row(window, chunk, distance, seen, tiles):
    """One key fits the last query and carries a value of 50, `distance` positions back, among 150 keys across page borders: the row is
    about 50 exactly when the mask lets the key be seen, for the last token of a prompt and for the same token decoded alone, in both
    attention kernels. (The last position is 149: chunk 40 starts at 120, chunk 64 at 128.)"""
    from stride_b200.kernels.native import ImmediateProgram
    from stride_b200.parts import Workspace
    H, G, D, V, page, n = 4, 2, 32, 16, 16, 150
    dtype = torch.bfloat16 if tiles else torch.float32
    g = torch.Generator().manual_seed(distance)
    q = torch.randn(n, H * D, generator=g) * 0.1
    k = torch.randn(n, G, D, generator=g) * 0.1
    v = torch.randn(n, G, V, generator=g) * 0.1
    q[n - 1] = 3.0 * torch.sign(torch.randn(H * D, generator=g))
    far = n - 1 - distance
    k[far] = q[n - 1].view(G, H // G, D)[:, 0]
    q[n - 1] = k[far].repeat_interleave(H // G, 0).reshape(-1)
    v[far] = 50.0
    pages = torch.full((12, 2, G, page, max(D, V)), 1e4, dtype=dtype, device=DEV)
    table = torch.randperm(12, generator=g)[:10].view(1, 10).to(torch.int32).to(DEV)
    for t in range(n):
        pg, at = int(table[0, t // page]), t % page
        pages[pg, 0, :, at, :D] = k[t].to(DEV, dtype)
        pages[pg, 1, :, at, :V] = v[t].to(DEV, dtype)
    ws = Workspace(DEV, ROWS)
    where = [table.shape[1], page, pages.stride(0), pages.stride(1), pages.stride(2)]
    for entries, rows in (([(0, 0, n, 0)], slice(0, n)), ([(0, 0, 1, n - 1)], slice(n - 1, n))):
        st = _Step(entries, dtype, ws)
        qd = q[rows].to(DEV, dtype).contiguous()
        out = torch.zeros(qd.shape[0], H * V, dtype=torch.float32, device=DEV)
        with ImmediateProgram(st.ctx, None) as program:
            if tiles:
                program.add("masked_attention", "sb_op_masked_attention_tiles", [qd, out, pages, table, *where, None, None, H, G, D, V, pages.shape[4],
                                                                                window, 0, chunk, 1], [1.0])
            else:
                program.add("masked_attention", "sb_op_masked_attention", [qd, out, qd.dtype, pages, table, *where, None, None, H, G, D, V,
                                                                          pages.shape[4], window, 0, chunk, 1], [1.0])
        last = out[-1].cpu()
        if seen:
            assert last.min() > 45.0, f"the key {distance} back is not seen: {last.min():.2f}"
        else:
            assert last.abs().max() < 5.0, f"the key {distance} back is seen: {last.abs().max():.2f}"


def test_token_side_and_normed_pair_against_the_plain_functions(sitivik_dirs):
    """The per-layer token input (a slice of the second table per layer, a token of -1 read from the sampled tokens) and the fold of two
    branches normed one by one, each with buffers and partial sums."""
    from stride_b200.kernels.native import ImmediateProgram
    from stride_b200.parts import PartSpec, ResidualStream, Workspace, part_class
    cfg, w = load_plain(sitivik_dirs["X"])
    W, dim, L, eps = cfg["width"], cfg["token_side"]["dim"], len(cfg["layers"]), cfg["norm"]["eps"]
    g = torch.Generator().manual_seed(3)
    n = 11
    toks = random_tokens(cfg["vocab"], n, 9)
    for dtype in (torch.float32, torch.bfloat16):
        for index in (0, L - 1):
            spec = PartSpec("token_side", {"hidden_size": W, "vocab_size": cfg["vocab"], "dim": dim, "slices": L, "index": index, "eps": eps},
                            {"table": "side.embed", "gate": f"l{index}.side.gate", "proj": f"l{index}.side.proj", "norm": f"l{index}.side.norm"})
            part = part_class("rewrite", "token_side")(spec, _env(dtype))
            part.bind({name: w[name].to(torch.bfloat16).to(DEV) for name in part.tensor_plan()})
            x = torch.randn(n, W, generator=g)
            if dtype == torch.bfloat16:
                x = x.to(dtype).float()
            ws = Workspace(DEV, ROWS)
            fed = list(toks)
            fed[4] = -1                                                  # a token still being chosen: read from the request's slot
            st = _Step([(1, 0, n, 0)], dtype, ws, tokens=fed)
            st.ctx.sampled = torch.tensor([0, toks[4], 0], dtype=torch.int32, device=DEV)
            # (only the bfloat16 engine's projections leave partial sums pending on the stream)
            pending = torch.randn(2, n, W, generator=g) * (0.1 if dtype == torch.bfloat16 else 0.0)
            h = ws.get("model.h", n, (W,), torch.float32)
            h.copy_((x - pending.sum(0)).to(DEV))
            stream = ResidualStream(h)
            if dtype == torch.bfloat16:
                stream.set_pending(pending.to(DEV))
            part.forward(st.ctx, stream)
            stream.fold()
            x64 = (x - pending.sum(0)).double() + pending.double().sum(0)
            want = x64 + plain.token_side(w, f"l{index}.", index, dim, torch.tensor(toks), x64, eps, dtype == torch.bfloat16)
            tol = 2e-4 if dtype == torch.float32 else 0.05
            assert (stream.h.cpu().double() - want).abs().max() <= tol * float(want.abs().max())
    # two branches, each normed over its row with its own gain, then their weighted sum
    n, W = 9, 100
    dst, a, b = (torch.randn(n, W, generator=g) for _ in range(3))
    pa, pb = torch.randn(3, n, W, generator=g), torch.randn(2, n, W, generator=g)
    ga, gb = torch.randn(W, generator=g), torch.randn(W, generator=g)
    ws = Workspace(DEV, ROWS)
    st = _Step([(0, 0, n, 0)], torch.bfloat16, ws)
    d, ad, bd, pad, pbd = (t.to(DEV).contiguous() for t in (dst, a, b, pa, pb))
    with ImmediateProgram(st.ctx, None) as program:
        program.add("branch", "sb_op_branch_pair_norm_fold", [d, ad, pad, 3, program.few_tokens, bd, pbd, 2, ga.to(DEV), gb.to(DEV), torch.float32, W],
                    [0.5, 0.25, 1e-3])
    A, B = a.double() + pa.double().sum(0), b.double() + pb.double().sum(0)
    want = dst.double() + 0.5 * plain.rms(A, 1e-3) * ga.double() + 0.25 * plain.rms(B, 1e-3) * gb.double()
    assert (d.cpu().double() - want).abs().max() <= 1e-5 * float(want.abs().max())
    assert float(ad.abs().max()) == 0.0 and float(bd.abs().max()) == 0.0       # the branches are empty again


# ---------------------------------------------------------------------------------------------- whole models
def _engine(model_dir, dtype, page, pages, rows=256, slots=4, **kw):
    from stride_b200.engine.engine import Engine, EngineOptions
    return Engine(model_dir, EngineOptions(dtype=dtype, max_rows=rows, max_full_rows=rows, max_slots=slots, kv_pages=pages,
                                           page_size=page, max_context=pages * page, device=DEV, **kw))


def _noise(cfg, w, tokens):
    """max and mean |plain with bfloat16 rounding - plain exact| over the sequence's logits."""
    d = (plain.forward(cfg, w, tokens, True) - plain.forward(cfg, w, tokens)).abs()
    return float(d.max()), float(d.mean())


def test_every_layer_against_the_plain_streams(sitivik_dirs):
    """The residual stream after every layer (behind its per-layer token input), in 32-bit, for a prompt in one step."""
    from stride_b200.engine.engine import StepEntry
    for name in ("X", "Y", "Z"):
        cfg, w = load_plain(sitivik_dirs[name])
        page = SITIVIK[name][2]
        toks = random_tokens(cfg["vocab"], 37, 12)
        streams = []
        plain.forward(cfg, w, toks, streams=streams)
        eng = _engine(sitivik_dirs[name], "float32", page, 8, native_step=False)
        slot = eng.cache.acquire_slot()
        eng.cache.ensure(slot, len(toks))
        seen = []
        side = "token_side" in cfg
        for block, layer in zip(eng.model.blocks, eng.model.spec.layers):
            if side != (layer.block == "rewrite"):        # with a token input the layer ends behind it
                continue

            def run(ctx, stream, cache, inner=block.forward):
                inner(ctx, stream, cache)
                stream.fold()
                seen.append(stream.h[:len(toks)].detach().cpu().double().clone())
            block.forward = run
        eng.step([StepEntry(slot, 0, toks, list(range(len(toks))))])
        assert len(seen) == len(streams)
        for k, (got, want) in enumerate(zip(seen, streams)):
            assert (got - want).abs().max() <= 2e-4 * max(1.0, float(want.abs().max())), f"{name}: the stream after layer {k} differs"


LENGTHS = {"X": [70, 130, 45, 33, 2], "Y": [300, 65, 140, 129, 40], "Z": [48, 90, 17, 64, 5]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["X", "Y", "Z"])
def test_replay_modes(name, dtype, sitivik_dirs, tmp_path):
    """Through bin/trace_run: whole; all but the last 32 tokens, then token by token; portions down to two tokens; mixed batches in a
    pool so small that pages are used again, four slots for five requests. Against the plain implementation (bfloat16: rounding at the
    same places; the largest deviation within the largest rounding noise of the same sequence), and all four in the same bits."""
    cfg, _, page = SITIVIK[name]
    vocab = cfg["vocab"]
    reqs = [random_tokens(vocab, n, 300 + i) for i, n in enumerate(LENGTHS[name])]
    pcfg, w = load_plain(sitivik_dirs[name])
    bf = dtype == "bfloat16"
    want = [plain.forward(pcfg, w, r, bf).float() for r in reqs]
    noise = [_noise(pcfg, w, r) if bf else None for r in reqs]
    per = lambda n: -(-n // page) * page
    longest = sorted((per(len(r)) for r in reqs), reverse=True)
    pool = max(longest[0] + longest[1] + page, 4 * page)
    tr = TraceRun(sitivik_dirs[name], dtype, tmp_path, pool, page, extra=("--kv-shuffle", "5"))
    bits = _Bits()

    def compare(got, i, a, b, what):
        tol = logit_tolerance(dtype, want[i]) if noise[i] is None else noise[i][0]
        diff = (got - want[i][a:b]).abs()
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


def test_window_and_chunk_edges_show_and_agree(sitivik_dirs):
    """With attention close to uniform every visible key carries weight: the plain implementation itself moves by far more than the
    tolerance when a window or a chunk is one token longer or shorter. The engine agrees with the right masks at every position, in a
    prompt whose windows and chunks straddle pages and decoding token by token with pages given back behind them."""
    from stride_b200.engine.engine import StepEntry
    cfg, w = load_plain(sitivik_dirs["XU"])
    toks = random_tokens(cfg["vocab"], 90, 77)
    want = plain.forward(cfg, w, toks).float()
    tol = logit_tolerance("float32", want)
    for layer, delta, least in ((1, 1, 20), (1, -1, 20), (2, 1, 20), (2, -1, 20), (3, -1, 5), (3, 1, 5)):     # (the last layer's window is 40 keys wide)
        other = copy.deepcopy(cfg)
        other["layers"][layer]["mixer"]["left"]["mask"]["size"] += delta
        moved = (plain.forward(other, w, toks).float() - want).abs().max(dim=1).values
        assert moved[45:].min() > least * tol, f"the yardstick does not notice layer {layer}'s mask {delta:+d}"
    eng = _engine(sitivik_dirs["XU"], "float32", 16, 12)
    slot = eng.cache.acquire_slot()
    eng.cache.ensure(slot, 50)
    got = [eng.step([StepEntry(slot, 0, toks[:50], list(range(50)))]).cpu().clone()]
    for t in range(50, 90):
        eng.cache.ensure(slot, t + 1)
        got.append(eng.step([StepEntry(slot, t, [toks[t]], [0])]).cpu().clone())
        eng.cache.trim(slot)
    assert (torch.cat(got) - want).abs().max() <= tol
    eng.cache.check()


def test_the_first_tokens_of_a_sequence(sitivik_dirs):
    """Positions 0, 1, 2, .. one by one in a slot that another request used: windows and chunks with fewer keys than their size, a sink
    beside a single key, a convolution with zeros in front of it, states that start from zero, position 0 of the rotations."""
    from stride_b200.engine.engine import StepEntry
    for name, page in (("Z", 8), ("X", 16), ("Y", 32)):
        cfg, w = load_plain(sitivik_dirs[name])
        eng = _engine(sitivik_dirs[name], "float32", page, 16)
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


def test_long_decoding_and_slot_reuse(sitivik_dirs):
    """A short prompt, then 400 tokens one by one (every window and chunk passes over decoded tokens, pages behind them are given back,
    the recurrent states run on), against the plain implementation; then the same slot again for another request, which must not see
    what the first left."""
    from stride_b200.engine.engine import StepEntry
    cfg, w = load_plain(sitivik_dirs["XU"])
    eng = _engine(sitivik_dirs["XU"], "float32", 16, 30)
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


def test_a_far_token_shows_through_the_states_and_the_unbounded_attention(sitivik_dirs, tmp_path):
    """The differential attention sees every earlier token and the recurrent states carry them. One early token's embedding is made
    large: another token in its place moves the plain logits 300 tokens later far beyond the tolerance, and the engine, fed in portions
    that cut pages and then token by token, agrees with the whole sequence."""
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
def test_batches_of_unequal_requests_against_each_alone(sitivik_dirs, native):
    """Four requests of unequal length in one step, then single tokens of some beside portions of others: every logit has the bits of
    the request run alone; the native step program and the part-by-part driver agree."""
    from stride_b200.engine.engine import StepEntry
    for name in ("Y", "X"):
        cfg, _, page = SITIVIK[name]
        reqs = [random_tokens(cfg["vocab"], n, 40 + n) for n in (150, 3, 64, 31)]
        for dtype in ("float32", "bfloat16"):
            eng = _engine(sitivik_dirs[name], dtype, page, 48, native_step=native)
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
                assert torch.equal(torch.cat(got[i]), alone[i]), f"{name} {dtype}: request {i} in company differs from the request alone"


def test_greedy_generation_through_the_entry_point(sitivik_dirs):
    """LLM.generate with its scheduler (three requests on two slots, prompts cut into portions, decode steps replayed from CUDA
    graphs, the per-layer token input reading tokens that are still being chosen): the tokens of greedy decoding with the plain
    implementation."""
    from stride_b200 import LLM
    cfg, w = load_plain(sitivik_dirs["X"])
    prompts = [random_tokens(cfg["vocab"], n, 500 + n) for n in (5, 41, 23)]
    llm = LLM(sitivik_dirs["X"], dtype="float32", concurrency=2, max_rows=32, prefill_chunk=8, kv_pages=12, page_size=16,
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
    bf = LLM(sitivik_dirs["Y"], dtype="bfloat16", concurrency=4, max_rows=64, prefill_chunk=16, kv_pages=16, page_size=32,
             max_slots=4, max_context=256, device=DEV)
    cfgy = SITIVIK["Y"][0]
    outs = bf.generate([random_tokens(cfgy["vocab"], n, n) for n in (70, 9, 33, 120, 64)], max_new_tokens=8)
    assert all(len(o.tokens) == 8 for o in outs)


def test_command_line_generates_what_the_entry_point_generates(sitivik_dirs, tmp_path):
    """bin/stride_cli on a Sitivik folder (greedy, float32 and bfloat16): the tokens of LLM.generate."""
    import json
    import subprocess
    import sys
    from conftest import ROOT
    from stride_b200 import LLM
    cfg = SITIVIK["Z"][0]
    prompts = [random_tokens(cfg["vocab"], n, 900 + n) for n in (3, 50, 21)]
    (tmp_path / "in.jsonl").write_text("".join(json.dumps({"id": i, "tokens": p}) + "\n" for i, p in enumerate(prompts)))
    for path, dtype in (("exact", "float32"), ("tc", "bfloat16")):
        out = tmp_path / f"out_{path}.jsonl"
        subprocess.run([sys.executable, str(ROOT / "bin" / "stride_cli"), "--model", str(sitivik_dirs["Z"]), "--input", str(tmp_path / "in.jsonl"),
                        "--output", str(out), "--max-new", "6", "--concurrency", "2", "--max-rows", "32", "--prefill-chunk", "16",
                        "--kv-blocks", "24", "--page-size", "8", "--max-slots", "4", "--max-context", "128", "--path", path], check=True, timeout=600)
        got = [json.loads(l) for l in out.read_text().splitlines()]
        llm = LLM(sitivik_dirs["Z"], dtype=dtype, concurrency=2, max_rows=32, prefill_chunk=16, kv_pages=24, page_size=8, max_slots=4,
                  max_context=128, device=DEV)
        want = llm.generate(prompts, max_new_tokens=6)
        assert [g["tokens"] for g in got] == [w.tokens for w in want] and all(g["finish"] == "length" for g in got)


def _drawn_configuration(seed):
    """A configuration drawn at random: sizes that are no multiple of four or eight, one tap, heads that are their own key heads, masks of
    one token and masks longer than the request, layers in any order, with and without the token input, feed-forward and rotation."""
    import random
    r = random.Random(seed)
    even = lambda lo, hi: 2 * r.randint(lo // 2, hi // 2)

    def rot(dim, scaled):
        if r.random() < 0.25:
            return None
        dims = even(2, dim)
        scaling = (r.choice([2.0, 8.0]), 1.0, r.choice([2.0, 4.0]), r.choice([16, 64, 512])) if scaled and r.random() < 0.6 else None
        out = {"dims": dims, "base": r.choice([50.0, 10000.0, 1000000.0])}
        if scaling:
            out["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
        return out

    def left(masked):
        kv = r.randint(1, 3)
        dim = even(4, 40)
        m = {"heads": kv * r.randint(1, 4), "kv_heads": kv, "dim": dim, "vdim": r.randint(3, 40), "scale": dim ** -0.5}
        if masked:
            m["mask"] = {"size": r.choice([1, 2, 5, 16, 33, 64, 500])}
        ro = rot(dim, True)
        if ro and masked:
            m["rot"] = ro
        return m

    layers = []
    for _ in range(r.randint(2, 4)):
        kind = r.choice(["parallel", "attention", "parallel_2"])
        mlp = {"kind": "dense", "ff": r.randint(5, 60)} if r.random() < 0.7 else None
        if kind == "attention":
            m = left(False)
            m["diff"] = r.choice([0.2, 0.5, 0.8])
            if r.random() < 0.6:
                m["q_temp"] = {"coef": r.choice([0.1, 0.5]), "every": r.choice([1, 3, 16, 1000])}
        elif kind == "parallel":
            heads, dim = r.randint(1, 4), even(4, 36)
            right = {"heads": heads, "dim": dim, "vdim": r.randint(2, 40), "decay": [r.choice([0.5, 0.9, 0.99, 1.0]) for _ in range(heads)]}
            ro = rot(dim, False)
            if ro:
                right["rot"] = ro
            m = {"left": left(True), "right": right}
        else:
            kv = r.randint(1, 3)
            right = {"heads": kv * r.randint(1, 3), "kv_heads": kv, "dim": r.randint(3, 40), "vdim": r.randint(2, 36), "conv": r.randint(1, 5),
                     "decay_rank": r.randint(1, 12), "gate_rank": r.randint(1, 12)}
            m = {"left": left(True), "right": right, "left_scale": r.choice([0.5, 1.0, 1.5]), "right_scale": r.choice([0.5, 1.0, 2.0])}
        layers.append({"type": kind, "mixer": m, "mlp": mlp})
    cfg = {"architecture": "Sitivik", "vocab": r.randint(30, 300), "width": r.choice([40, 50, 64, 72, 100, 136]), "norm": {"eps": r.choice([1e-6, 1e-4])},
           "layers": layers}
    if r.random() < 0.7:
        cfg["embedding"] = {"scale": r.choice([0.5, 1.0, 4.0])}
    if r.random() < 0.7:
        cfg["token_side"] = {"dim": r.randint(1, 20)}
    return cfg


@pytest.mark.parametrize("seed", [11, 12, 13, 14, 15, 16])
def test_configurations_drawn_at_random(seed, tmp_path):
    """Whole, and in portions down to one token with pages trimmed on the way, in 32-bit against the plain implementation and in bfloat16 in
    equal bits between the two ways of feeding."""
    from stride_b200.engine.engine import StepEntry
    import sitivik_cases
    cfg = _drawn_configuration(seed)
    sitivik_cases.SITIVIK[f"R{seed}"] = (cfg, seed, 16)
    try:
        folder = write_model(tmp_path / "m", f"R{seed}")
    finally:
        del sitivik_cases.SITIVIK[f"R{seed}"]
    pcfg, w = load_plain(folder)
    toks = random_tokens(cfg["vocab"], 75, seed)
    want = plain.forward(pcfg, w, toks).float()
    for dtype in ("float32", "bfloat16"):
        got = []
        for cuts in ([75], [9, 1, 2, 30, 1, 1, 17, 5, 1, 1, 7]):
            eng = _engine(folder, dtype, 16, 12)
            slot = eng.cache.acquire_slot()
            rows, at = [], 0
            for n in cuts:
                eng.cache.ensure(slot, at + n)
                rows.append(eng.step([StepEntry(slot, at, toks[at:at + n], list(range(n)))]).cpu().clone())
                eng.cache.trim(slot)
                at += n
            got.append(torch.cat(rows))
        assert torch.equal(got[0], got[1]), f"seed {seed} {dtype}: in portions it differs from the whole"
        if dtype == "float32":
            assert (got[0] - want).abs().max() <= logit_tolerance("float32", want), f"seed {seed}: {cfg}"
        else:
            noise = _noise(pcfg, w, toks)[0]
            assert (got[0] - plain.forward(pcfg, w, toks, True).float()).abs().max() <= 2.0 * noise
