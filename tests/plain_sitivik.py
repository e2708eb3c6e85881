"""Sitivik written out plainly in float64: one function per mechanism, a whole sequence at a time, no cache, no state carried
between calls, nothing shared with the engine. `config` is config.json as a dict, `w` maps tensor names to float64 tensors.

With `bf16=True` the places where the serving precision rounds (what enters a matrix product: normed activations, queries, keys and
values, the mixers' results in front of their output projections, hidden activations) are rounded to bfloat16 too, so that the
engine's bfloat16 path can be held to a tolerance that is its own rounding noise."""
from __future__ import annotations

import math

import torch

F = torch.float64


def rnd(x, bf16):
    return x.to(torch.bfloat16).to(F) if bf16 else x


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def frequencies(rot: dict):
    dims, base = rot["dims"], float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if sc:
        factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
        out = []
        for x in f:
            wave = 2.0 * math.pi / x
            if wave < orig / high:
                out.append(x)
            elif wave > orig / low:
                out.append(x / factor)
            else:
                s = (orig / wave - low) / (high - low)
                out.append((1.0 - s) * x / factor + s * x)
        f = out
    return torch.tensor(f, dtype=F)


def rotate(x, positions, rot: dict, interleaved: bool):
    """x [T, heads, dim]: the first rot.dims elements of every head turned by the position's angles (no `rot`: nothing is turned)."""
    if not rot:
        return x
    dims = rot["dims"]
    a = positions.to(F)[:, None] * frequencies(rot)[None, :]        # [T, dims / 2]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    out = x.clone()
    if interleaved:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    else:
        u, v = x[..., :dims // 2], x[..., dims // 2:dims]
        out[..., :dims // 2] = u * c - v * s
        out[..., dims // 2:dims] = v * c + u * s
    return out


def softmax_attention(q, k, v, scale, mask, sink: bool):
    """q [T, H, D], k [T, G, D], v [T, G, Dv]; mask [T, T] bool (row sees column); sink: one more term exp(0) in the denominator."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~mask, -math.inf)
        m = s.max(-1, keepdim=True).values
        if sink:
            m = torch.clamp(m, min=0.0)
        e = torch.exp(s - m)
        den = e.sum(-1, keepdim=True) + (torch.exp(-m) if sink else 0.0)
        out[:, h] = (e / den) @ v[:, g]
    return out


def causal_mask(T):
    i = torch.arange(T)
    return i[:, None] >= i[None, :]


def window_mask(T, size):
    i = torch.arange(T)
    d = i[:, None] - i[None, :]
    return (d >= 0) & (d < size)


def chunk_mask(T, size):
    i = torch.arange(T)
    return (i[:, None] >= i[None, :]) & ((i[:, None] // size) == (i[None, :] // size))


def linear(w, name, x, bf16, bias=True):
    y = rnd(x, bf16) @ w[name].T
    if bias and name + ".b" in w:
        y = y + w[name + ".b"]
    return y


def windowed_left(w, p, m, h, eps, bf16):
    """The left member of "parallel": biases, q/k norm over the whole projection, interleaved rotation, window, elementwise gate."""
    T, H, G, D, Dv = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q, k, v = linear(w, p + "q", h, bf16), linear(w, p + "k", h, bf16), linear(w, p + "v", h, bf16)
    q = rms(q, eps) * w[p + "q.norm"]
    k = rms(k, eps) * w[p + "k.norm"]
    q = rotate(q.view(T, H, D), pos, m.get("rot"), True)
    k = rotate(k.view(T, G, D), pos, m.get("rot"), True)
    o = softmax_attention(rnd(q, bf16), rnd(k, bf16), rnd(v.view(T, G, Dv), bf16), m["scale"], window_mask(T, m["mask"]["size"]), False)
    o = o.reshape(T, H * Dv) * torch.sigmoid(linear(w, p + "g", h, bf16))
    return linear(w, p + "o", o, bf16)


def retention_right(w, p, m, h, eps, bf16):
    T, H, D, Dv = h.shape[0], m["heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = rotate(linear(w, p + "q", h, bf16).view(T, H, D), pos, m.get("rot"), False)
    k = rotate(linear(w, p + "k", h, bf16).view(T, H, D), pos, m.get("rot"), False) * D ** -0.5
    v = linear(w, p + "v", h, bf16).view(T, H, Dv)
    o = torch.zeros(T, H, Dv, dtype=F)
    for hd in range(H):
        S = torch.zeros(D, Dv, dtype=F)
        for t in range(T):
            S = m["decay"][hd] * S + torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = S.T @ q[t, hd]
    o = rms(o, eps).reshape(T, H * Dv) * silu(linear(w, p + "g", h, bf16))
    return linear(w, p + "o", o, bf16)


def parallel_mixer(w, p, m, h, eps, bf16):
    left = windowed_left(w, p + "left.", m["left"], h, eps, bf16)
    right = retention_right(w, p + "right.", m["right"], h, eps, bf16)
    return 0.5 * (rms(left, eps) * w[p + "left.out"] + rms(right, eps) * w[p + "right.out"])


def differential_attention(w, p, m, h, eps, bf16):
    T, H, G, D, Dv = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = linear(w, p + "q", h, bf16).view(T, H, 2, D)
    k = linear(w, p + "k", h, bf16).view(T, G, 2, D)
    v = linear(w, p + "v", h, bf16).view(T, G, Dv)
    qt = m.get("q_temp")
    if qt:
        q = q * (1.0 + qt["coef"] * torch.log(torch.floor((pos + 1).to(F) / qt["every"]) + 1.0))[:, None, None, None]
    mask = causal_mask(T)
    a = [softmax_attention(rnd(q[:, :, i], bf16), rnd(k[:, :, i], bf16), rnd(v, bf16), m["scale"], mask, False) for i in range(2)]
    diff = m["diff"]
    lam = math.exp(float((w[p + "lq1"] * w[p + "lk1"]).sum())) - math.exp(float((w[p + "lq2"] * w[p + "lk2"]).sum())) + diff
    o = rms(a[0] - lam * a[1], eps) * (1.0 - diff)
    gate = torch.sigmoid(linear(w, p + "g", h, bf16))                # [T, H]
    o = (o * gate[:, :, None]).reshape(T, H * Dv)
    return linear(w, p + "o", o, bf16)


def chunked_left(w, p, m, h, eps, bf16):
    """The left member of "parallel_2": biases, q/k norm per head, interleaved rotation, chunks, a sink of score 0, elementwise gate."""
    T, H, G, D, Dv = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = rms(linear(w, p + "q", h, bf16).view(T, H, D), eps) * w[p + "q.norm"]
    k = rms(linear(w, p + "k", h, bf16).view(T, G, D), eps) * w[p + "k.norm"]
    v = linear(w, p + "v", h, bf16).view(T, G, Dv)
    q, k = rotate(q, pos, m.get("rot"), True), rotate(k, pos, m.get("rot"), True)
    o = softmax_attention(rnd(q, bf16), rnd(k, bf16), rnd(v, bf16), m["scale"], chunk_mask(T, m["mask"]["size"]), True)
    o = o.reshape(T, H * Dv) * torch.sigmoid(linear(w, p + "g", h, bf16))
    return linear(w, p + "o", o, bf16)


def short_convolution(x, taps_w):
    """x [T, C], taps_w [C, taps]: y_t = sum_j taps_w[:, j] x_(t - taps + 1 + j), zeros before the start."""
    T, taps = x.shape[0], taps_w.shape[1]
    y = torch.zeros_like(x)
    for j in range(taps):
        shift = taps - 1 - j
        if shift < T:
            y[shift:] += x[:T - shift] * taps_w[:, j]
    return y


def delta_right(w, p, m, h, eps, bf16):
    T, H, G, D, Dv = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_convolution(linear(w, p + "q", h, bf16, False), w[p + "q.conv"])).view(T, G, D)
    k = silu(short_convolution(linear(w, p + "k", h, bf16, False), w[p + "k.conv"])).view(T, G, D)
    v = silu(short_convolution(linear(w, p + "v", h, bf16, False), w[p + "v.conv"])).view(T, H, Dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(rnd(h, bf16) @ w[p + "b"].T)                # [T, H]
    a = rnd(rnd(h, bf16) @ w[p + "a1"].T, bf16) @ w[p + "a2"].T + w[p + "dt_bias"]
    decay = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * torch.nn.functional.softplus(a).view(T, H, D))
    o = torch.zeros(T, H, Dv, dtype=F)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(D, Dv, dtype=F)
        for t in range(T):
            S = decay[t, hd][:, None] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            o[t, hd] = S.T @ q[t, g]
    gate = torch.sigmoid(rnd(rnd(h, bf16) @ w[p + "g1"].T, bf16) @ w[p + "g2"].T).view(T, H, Dv)
    o = (rms(o, eps) * w[p + "norm"] * gate).reshape(T, H * Dv)
    return linear(w, p + "o", o, bf16)


def parallel_2_mixer(w, p, m, h, eps, bf16):
    return (m["left_scale"] * chunked_left(w, p + "left.", m["left"], h, eps, bf16)
            + m["right_scale"] * delta_right(w, p + "right.", m["right"], h, eps, bf16))


MIXERS = {"parallel": parallel_mixer, "attention": differential_attention, "parallel_2": parallel_2_mixer}


def dense_feed_forward(w, p, h, bf16):
    z = silu(rnd(h, bf16) @ w[p + "gate"].T) * (rnd(h, bf16) @ w[p + "up"].T)
    return rnd(z, bf16) @ w[p + "down"].T


def token_side(w, p, i, dim, tokens, x, eps, bf16):
    e = w["side.embed"][tokens][:, i * dim:(i + 1) * dim]
    g = gelu_tanh(rnd(x, bf16) @ w[p + "side.gate"].T) * e
    y = rnd(g, bf16) @ w[p + "side.proj"].T
    return rms(y, eps) * w[p + "side.norm"]


def forward(config: dict, w: dict, tokens, bf16: bool = False, streams: list = None):
    """Logits [T, vocab] for the whole sequence; `streams` (a list) receives the residual stream after every layer."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    eps = float(config["norm"]["eps"])
    x = w["embed"][tokens] * float((config.get("embedding") or {}).get("scale", 1.0))
    side = config.get("token_side")
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        r = MIXERS[layer["type"]](w, p + "mix.", layer["mixer"], rms(x, eps) * w[p + "norm1"], eps, bf16)
        x = x + (r * w[p + "ls1"] if p + "ls1" in w else r)
        if layer.get("mlp"):
            r = dense_feed_forward(w, p + "mlp.", rms(x, eps) * w[p + "norm2"], bf16)
            x = x + (r * w[p + "ls2"] if p + "ls2" in w else r)
        if side:
            x = x + token_side(w, p, i, side["dim"], tokens, x, eps, bf16)
        if streams is not None:
            streams.append(x.clone())
    return rnd(rms(x, eps) * w["final.norm"], bf16) @ w["embed"].T
