"""A plain, slow implementation of the Pusisun design: one function per mechanism, whole sequences, no cache, no
batching, float64 arithmetic on the CPU. It shares no code with the engine; the tests hold the engine to it.

A model is (config dict, {tensor name: torch tensor}); weights are widened exactly. Notation: x [T, W] is the residual
stream of one sequence whose tokens stand at positions 0..T-1; W_foo y means y @ W_foo.T.

`rnd` (None or torch.bfloat16) rounds where an engine that serves in that precision may round: the inputs of the matrix
products (normed activations, the latents, queries, cached keys, values and latents, the mixers' outputs in front of
W_o, the experts' hidden activations). Everything the design wants in 32-bit stays unrounded. The difference between
the two is the size of the rounding noise that the tests measure the bfloat16 engine by.
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def w(tensors, name):
    return tensors[name].to(F)


def rounded(x, rnd):
    return x if rnd is None else x.to(rnd).to(F)


def rms_norm(x, gain, eps):
    """x / sqrt(mean(x^2) + eps) * gain along the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * gain


def silu(z):
    return z * torch.sigmoid(z)


def yarn_frequencies(dims, base, scaling):
    """The angle a position advances pair i by, and the factor on cos and sin. Pairs that turn fast keep their frequency,
    pairs that turn slowly are slowed by `factor`, with a linear ramp over the pair index between the two."""
    half = dims // 2
    freq = [base ** (-2.0 * i / dims) for i in range(half)]
    if not scaling:
        return freq, 1.0
    factor, original = scaling["factor"], scaling["original"]

    def pair_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(scaling["fast"])), 0)
    hi = min(math.ceil(pair_of(scaling["slow"])), dims - 1)
    out = []
    for i, f in enumerate(freq):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate(x, positions, freq, magnitude):
    """x [T, heads, dims]: element i is paired with i + dims/2 and the pair turns by position * freq[i]."""
    half = x.shape[-1] // 2
    angle = positions.to(F)[:, None] * torch.tensor(freq, dtype=F)[None, :]
    c, s = (torch.cos(angle) * magnitude)[:, None, :], (torch.sin(angle) * magnitude)[:, None, :]
    u, v = x[..., :half], x[..., half:]
    return torch.cat([u * c - v * s, v * c + u * s], dim=-1)


def latent_attention(h, tensors, prefix, m, eps, rnd=None):
    """Queries, keys and values come out of low-rank latents; one rotated key part is shared by all heads; causal softmax."""
    T = h.shape[0]
    H, D, R, V, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = rounded(rms_norm(h @ w(tensors, prefix + "dq").T, w(tensors, prefix + "dq.norm"), eps), rnd)
    q = rounded((cq @ w(tensors, prefix + "uq").T).view(T, H, D + R), rnd)
    down = h @ w(tensors, prefix + "dkv").T
    c = rounded(rms_norm(down[:, :C], w(tensors, prefix + "dkv.norm"), eps), rnd)
    rot = m["rot"]
    freq, magnitude = yarn_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    positions = torch.arange(T)
    shared = rounded(rotate(down[:, None, C:], positions, freq, magnitude), rnd)[:, 0]     # [T, R]
    q_rot = rounded(rotate(q[..., D:], positions, freq, magnitude), rnd)
    k = (c @ w(tensors, prefix + "uk").T).view(T, H, D)
    v = (c @ w(tensors, prefix + "uv").T).view(T, H, V)
    seen = torch.arange(T)[None, :] <= torch.arange(T)[:, None]
    out = torch.zeros(T, H, V, dtype=F)
    for head in range(H):
        score = (q[:, head, :D] @ k[:, head].T + q_rot[:, head] @ shared.T) * m["scale"]
        score = score.masked_fill(~seen, -math.inf)
        out[:, head] = torch.softmax(score, dim=-1) @ v[:, head]
    return rounded(out.reshape(T, H * V), rnd) @ w(tensors, prefix + "o").T


def sink_attention(h, tensors, prefix, m, eps, rnd=None):
    """Grouped heads with biased projections, q and k normed over the whole projection, no rotation, a penalty on distance per
    head, a window that also keeps the first tokens, and a softmax whose denominator holds one more term per head."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = h @ w(tensors, prefix + "q").T + w(tensors, prefix + "q.b")
    k = h @ w(tensors, prefix + "k").T + w(tensors, prefix + "k.b")
    v = h @ w(tensors, prefix + "v").T + w(tensors, prefix + "v.b")
    q = rounded(rms_norm(q, w(tensors, prefix + "q.norm"), eps), rnd).view(T, H, D)
    k = rounded(rms_norm(k, w(tensors, prefix + "k.norm"), eps), rnd).view(T, G, D)
    v = rounded(v, rnd).view(T, G, V)
    mask = m.get("mask") or {}
    window, keep = mask.get("size", 0), mask.get("keep_first", 0)
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = j <= i
    if window:
        seen = seen & ((i - j < window) | (j < keep))
    sink = w(tensors, prefix + "sink")
    out = torch.zeros(T, H, V, dtype=F)
    for head in range(H):
        g = head // (H // G)
        slope = 2.0 ** (-8.0 * (head + 1) / H)
        score = (q[:, head] @ k[:, g].T) * m["scale"] - slope * (i - j).to(F)
        score = score.masked_fill(~seen, -math.inf)
        top = torch.maximum(score.max(dim=-1, keepdim=True).values, sink[head])
        e = torch.exp(score - top)
        out[:, head] = (e / (e.sum(-1, keepdim=True) + torch.exp(sink[head] - top))) @ v[:, g]
    return rounded(out.reshape(T, H * V), rnd) @ w(tensors, prefix + "o").T


def routed_experts(h, tensors, prefix, mlp, rnd=None, leads=None):
    """Every token uses the `top` experts with the largest router logits, weighted by the softmax over those logits alone.
    `leads` (a list) receives, per token, by how much the last chosen logit leads the first one left out."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = h @ w(tensors, prefix + "router").T + w(tensors, prefix + "router.b")
    best = torch.topk(z, top, dim=-1)
    if leads is not None and top < E:
        leads.append((torch.topk(z, top + 1, dim=-1).values[:, top - 1:top + 1].diff(dim=-1).abs()[:, 0]))
    weight = torch.softmax(best.values, dim=-1)
    out = torch.zeros_like(h)
    for e in range(E):
        p = f"{prefix}e{e}."
        mid = rounded(silu(h @ w(tensors, p + "gate").T) * (h @ w(tensors, p + "up").T), rnd)
        share = (weight * (best.indices == e)).sum(-1, keepdim=True)
        out = out + share * (mid @ w(tensors, p + "down").T)
    return out


def layer(x, tensors, i, spec, eps, rnd=None, leads=None):
    """x + norm1b(mixer(norm1(x))), then the same around the feed-forward if the layer has one."""
    p = f"l{i}."
    h = rounded(rms_norm(x, w(tensors, p + "norm1"), eps), rnd)
    mixer = {"attention": sink_attention, "latent_attention": latent_attention}[spec["type"]]
    x = x + rms_norm(mixer(h, tensors, p + "mix.", spec["mixer"], eps, rnd), w(tensors, p + "norm1b"), eps)
    if spec.get("mlp"):
        h = rounded(rms_norm(x, w(tensors, p + "norm2"), eps), rnd)
        x = x + rms_norm(routed_experts(h, tensors, p + "mlp.", spec["mlp"], rnd, leads), w(tensors, p + "norm2b"), eps)
    return x


def layer_order(config):
    """[(layer, pass number or None, first of its pass)] in the order the layers run."""
    L = len(config["layers"])
    loop = config.get("loop")
    if not loop or loop["stop"] <= loop["start"]:
        return [(i, None, False) for i in range(L)]
    order = [(i, None, False) for i in range(loop["start"])]
    for t in range(loop["times"]):
        order += [(i, t, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return order + [(i, None, False) for i in range(loop["stop"], L)]


def forward(config, tensors, tokens, rnd=None, streams=None, leads=None):
    """Logits [T, vocab] of one sequence. `streams` (a list) receives the residual stream after every layer run."""
    eps = config["norm"]["eps"]
    first = w(tensors, "embed")[torch.as_tensor(tokens, dtype=torch.long)] * config["embedding"]["scale"]
    x = first
    for i, t, opens in layer_order(config):
        if opens:
            if t > 0:
                x = x + first
            x = x + w(tensors, "loop.step")[t]
        x = layer(x, tensors, i, config["layers"][i], eps, rnd, leads)
        if streams is not None:
            streams.append(x)
    h = rounded(rms_norm(x, w(tensors, "final.norm"), eps), rnd)
    return h @ w(tensors, "head").T
