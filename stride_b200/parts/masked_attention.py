"""Softmax attention over the paged cache with score terms and masks as parameters (kernels: csrc/masked_attention.cu), and the two
mixers that use it.

"masked_attention": grouped-query attention. q, k, v = W x + b (biases optional); the whole query projection and the whole key projection
may each be RMS-normed as one vector, before the split into heads, with a gain of that size; score(i, j) = scale q_i.k_j - slope_h (i - j)
with slope_h = 2^(-slope_bits (h + 1) / H) (`distance_slopes`; None: no distance term); i sees j <= i with i - j < window or
j < keep_first (window 0: every earlier key); a learned number per head may join the softmax's denominator as a key without value
(`sink`). Key and value sizes may differ: a cache row holds the larger.

"latent_attention": queries and keys/values go through low-rank latents. c_q = norm(W_dq x), q = W_uq c_q, a head's q being
[dim unrotated | rot rotated]; W_dkv x = [c' | r]: c = norm(c') is the key/value latent, r, rotated, a key part that all heads share;
a head's key is [W_uk,h c | r] and its value W_uv,h c. Only [c | r] is cached, one row per token: the key projection is taken into the
query, q'_h = [W_uk,h^T q_h,unrotated | q_h,rotated], so that q'_h.[c | r] is the head's score, the attention's values are c itself, and
W_uv,h is applied to the result (per-head products: `head_linear`). Every earlier key is seen; ordinary softmax."""
from __future__ import annotations

import math

import torch

from ..kernels import ops
from ..kernels.linear import Linear
from .base import CacheNeed, Mixer, part_class, register_part
from .spec import TensorPlan


def distance_slopes(num_heads: int, bits: float) -> torch.Tensor:
    """slope_h = 2^(-bits (h + 1) / H), h = 0 .. H - 1, rounded to float32 from 64-bit."""
    return torch.tensor([math.pow(2.0, -bits * (h + 1) / num_heads) for h in range(num_heads)], dtype=torch.float64).to(torch.float32)


def _attend(q, out, cache, ctx, slopes, sinks, H, G, D, Dv, window, keep_first, scale, tiles):
    if tiles:
        ops.masked_attention_tiles(q, out, cache.pages, cache.block_table, ctx.entry_meta, ctx.entry_meta.shape[1], slopes, sinks, H, G, D, Dv,
                                   window, keep_first, scale)
    else:
        ops.masked_attention(q, out, cache.pages, cache.block_table, ctx.positions, ctx.slots, slopes, sinks, H, G, D, Dv, window, keep_first, scale)


def _page_where(pages, table):
    """The page arguments of the attention operations: pages per sequence, page size, page stride, offset of a token's values from its key
    (0: the key row's leading elements are the values), head stride."""
    return [table.shape[1], pages.shape[3], pages.stride(0), pages.stride(1) if pages.shape[1] > 1 else 0, pages.stride(2)]


def _emit_attend(program, q, out, cache, slopes, sinks, H, G, D, Dv, window, keep_first, scale, tiles):
    pages, table = cache.pages, cache.block_table
    if tiles:
        program.add("masked_attention", "sb_op_masked_attention_tiles",
                    [q, out, pages, table, *_page_where(pages, table), slopes, sinks, H, G, D, Dv, pages.shape[4], window, keep_first], [scale])
    else:
        program.add("masked_attention", "sb_op_masked_attention",
                    [q, out, q.dtype, pages, table, *_page_where(pages, table), slopes, sinks, H, G, D, Dv, pages.shape[4], window, keep_first],
                    [scale])


@register_part("mixer", "masked_attention")
class MaskedAttentionMixer(Mixer):
    """params: hidden_size, num_heads, num_kv_heads, key_dim, value_dim, scale, window (0 = all keys), keep_first, norm_eps,
    qk_norm (True: the whole q and the whole k projection are RMS-normed), bias (True: q, k, v have biases), slope_bits (None: no distance
    term), sink (True: a number per head in the denominator). tensors: q, k, v, o, and as the parameters say q_bias, k_bias, v_bias,
    q_norm [H D], k_norm [G D], sink [H]."""
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.num_heads, self.num_kv_heads = int(p["num_heads"]), int(p["num_kv_heads"])
        self.key_dim, self.value_dim = int(p["key_dim"]), int(p["value_dim"])
        self.window, self.keep_first = int(p.get("window", 0) or 0), int(p.get("keep_first", 0) or 0)
        self.scale, self.eps = float(p["scale"]), float(p.get("norm_eps", 1e-6))
        self.qk_norm, self.biased, self.has_sink = bool(p.get("qk_norm")), bool(p.get("bias")), bool(p.get("sink"))
        self.slope_bits = p.get("slope_bits")
        if self.num_heads % self.num_kv_heads:
            raise ValueError(f"masked attention: {self.num_heads} heads do not divide into {self.num_kv_heads} key/value heads")
        if max(self.key_dim, self.value_dim) > 640:
            raise ValueError(f"masked attention: key size {self.key_dim} / value size {self.value_dim} exceed 640, the most the kernel holds")
        if self.window == 0:
            self.keep_first = 0
        self.row = max(self.key_dim, self.value_dim)
        self.qkv = self.o = self.bias = self.q_gain = self.k_gain = self.slopes = self.sinks = None

    def tensor_plan(self):
        t, H, G, D, V = self.spec.tensors, self.num_heads, self.num_kv_heads, self.key_dim, self.value_dim
        plan = {t["q"]: TensorPlan((H * D, self.hidden)), t["k"]: TensorPlan((G * D, self.hidden)), t["v"]: TensorPlan((G * V, self.hidden)),
                t["o"]: TensorPlan((self.hidden, H * V))}
        if self.biased:
            plan.update({t["q_bias"]: TensorPlan((H * D,), zero_mean=True), t["k_bias"]: TensorPlan((G * D,), zero_mean=True),
                         t["v_bias"]: TensorPlan((G * V,), zero_mean=True)})
        if self.qk_norm:
            plan.update({t["q_norm"]: TensorPlan((H * D,)), t["k_norm"]: TensorPlan((G * D,))})
        if self.has_sink:
            plan[t["sink"]] = TensorPlan((H,), zero_mean=True)
        return plan

    def bind(self, tensors):
        t, f32 = self.spec.tensors, torch.float32
        ws = [tensors[t[r]] for r in ("q", "k", "v")]
        if len({w.dtype for w in ws}) > 1:
            ws = [w.to(f32) for w in ws]
        self.qkv = Linear(torch.cat(ws, dim=0), self.env.compute_dtype)
        self.o = Linear(tensors[t["o"]], self.env.compute_dtype)
        if self.biased:
            self.bias = torch.cat([tensors[t[r]].to(f32) for r in ("q_bias", "k_bias", "v_bias")]).contiguous()
        if self.qk_norm:
            self.q_gain, self.k_gain = tensors[t["q_norm"]].to(f32).contiguous(), tensors[t["k_norm"]].to(f32).contiguous()
        if self.has_sink:
            self.sinks = tensors[t["sink"]].to(f32).contiguous()
        if self.slope_bits is not None:
            self.slopes = distance_slopes(self.num_heads, float(self.slope_bits)).to(self.env.device)

    def weight_bytes(self):
        return self.qkv.weight_bytes() + self.o.weight_bytes()

    def cache_need(self):
        return CacheNeed("pages", kv_heads=self.num_kv_heads, head_dim=self.row, window=self.window, dtype=self.env.act_dtype,
                         keep_first=self.keep_first)

    def kernel_libraries(self):
        return {"masked_attention", "gemm_tc" if self.env.compute_dtype == torch.bfloat16 else "gemm_f32"}

    def _tiles(self, pages) -> bool:
        """The bfloat16 engine takes the tensor-core kernel where the shape allows it, the float32 engine and every other shape the
        kernel with a block per token and head."""
        return self.env.act_dtype == torch.bfloat16 and ops.masked_attention_tiles_supported(
            self.num_heads, self.num_kv_heads, self.key_dim, self.value_dim, pages.shape[4], pages.stride(1))

    def forward(self, ctx, x, stream, cache):
        n, ws, H, G, D, V = ctx.n, ctx.workspace, self.num_heads, self.num_kv_heads, self.key_dim, self.value_dim
        qkv = self.qkv.forward_partials(x, ws.raw("mattn.qkv", (self.qkv.partial_elems(ws.max_tokens),), torch.float32))
        q = ws.get("mattn.q", n, (H * D,), ctx.act_dtype)
        ops.qkv_norm_append(qkv, self.bias, self.q_gain, self.k_gain, self.eps, ctx.positions, ctx.slots, q, cache.pages, cache.block_table,
                            H, G, D, V, write_kv=cache.writes)
        mixed = ws.get("mattn.out", n, (H * V,), ctx.act_dtype)
        _attend(q, mixed, cache, ctx, self.slopes, self.sinks, H, G, D, V, self.window, self.keep_first, self.scale, self._tiles(cache.pages))
        self.o.forward_add(mixed, stream, ws.raw("mattn.o_partials", (self.o.partial_elems(ws.max_tokens),), torch.float32))

    def emit(self, program, x, cache):
        ws, H, G, D, V = program.workspace, self.num_heads, self.num_kv_heads, self.key_dim, self.value_dim
        act, T = self.env.act_dtype, ws.max_tokens
        qkv = ws.raw("mattn.qkv", (self.qkv.partial_elems(T),), torch.float32)
        S = self.qkv.emit_partials(program, x, qkv)
        q = ws.get("mattn.q", T, (H * D,), act)
        mixed = ws.get("mattn.out", T, (H * V,), act)
        pages, table = cache.pages, cache.block_table
        program.add("masked_attention", "sb_op_qkv_norm_append",
                    [qkv, S, program.few_tokens, self.bias, self.q_gain, self.k_gain, q, q.dtype, pages, table, *_page_where(pages, table),
                     H, G, D, V, pages.shape[4], int(cache.writes)], [self.eps])
        _emit_attend(program, q, mixed, cache, self.slopes, self.sinks, H, G, D, V, self.window, self.keep_first, self.scale, self._tiles(pages))
        self.o.emit_add(program, mixed, ws.raw("mattn.o_partials", (self.o.partial_elems(T),), torch.float32))


@register_part("mixer", "latent_attention")
class LatentAttentionMixer(Mixer):
    """params: hidden_size, num_heads, key_dim (a head's unrotated query/key elements), rot_dim (its rotated ones), value_dim, q_rank,
    kv_rank, scale, norm_eps, position (a PartSpec of category "position" offering cos_sin for rotary_dim = rot_dim, or None when
    rot_dim is 0). tensors: dq [q_rank, hidden], dq_norm, uq [H (key_dim + rot_dim), q_rank], dkv [kv_rank + rot_dim, hidden], dkv_norm,
    uk [H key_dim, kv_rank], uv [H value_dim, kv_rank], o [hidden, H value_dim]."""
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden, self.num_heads = int(p["hidden_size"]), int(p["num_heads"])
        self.key_dim, self.rot_dim, self.value_dim = int(p["key_dim"]), int(p.get("rot_dim", 0) or 0), int(p["value_dim"])
        self.q_rank, self.kv_rank = int(p["q_rank"]), int(p["kv_rank"])
        self.scale, self.eps = float(p["scale"]), float(p.get("norm_eps", 1e-6))
        if self.rot_dim % 2:
            raise ValueError(f"latent attention: {self.rot_dim} rotated elements (must be even)")
        self.row = self.kv_rank + self.rot_dim
        if self.row > 640:
            raise ValueError(f"latent attention: a cached row of {self.row} elements exceeds 640, the most the kernel holds")
        pos = p.get("position")
        if (pos is None) != (self.rot_dim == 0):
            raise ValueError("latent attention: a position part goes with rot_dim > 0, and only with it")
        self.position = part_class("position", pos.kind)(pos, env) if pos is not None else None
        self.down = self.uq = self.o = self.uk = self.uv = self.q_gain = self.kv_gain = None

    def tensor_plan(self):
        t, H = self.spec.tensors, self.num_heads
        plan = {t["dq"]: TensorPlan((self.q_rank, self.hidden)), t["dq_norm"]: TensorPlan((self.q_rank,)),
                t["uq"]: TensorPlan((H * (self.key_dim + self.rot_dim), self.q_rank)),
                t["dkv"]: TensorPlan((self.kv_rank + self.rot_dim, self.hidden)), t["dkv_norm"]: TensorPlan((self.kv_rank,)),
                t["uk"]: TensorPlan((H * self.key_dim, self.kv_rank)), t["uv"]: TensorPlan((H * self.value_dim, self.kv_rank)),
                t["o"]: TensorPlan((self.hidden, H * self.value_dim))}
        if self.position is not None:
            plan.update(self.position.tensor_plan())
        return plan

    def bind(self, tensors):
        t, f32, H = self.spec.tensors, torch.float32, self.num_heads
        ws = [tensors[t["dq"]], tensors[t["dkv"]]]
        if ws[0].dtype != ws[1].dtype:
            ws = [w.to(f32) for w in ws]
        self.down = Linear(torch.cat(ws, dim=0), self.env.compute_dtype)       # [q latent | key/value latent | shared rotated key part]
        self.uq = Linear(tensors[t["uq"]], self.env.compute_dtype)
        self.o = Linear(tensors[t["o"]], self.env.compute_dtype)
        act = self.env.act_dtype
        # per head: [key_dim, kv_rank] takes the unrotated query to the latent; [kv_rank, value_dim] takes the latent result to the values
        self.uk = tensors[t["uk"]].to(act).view(H, self.key_dim, self.kv_rank).contiguous()
        self.uv = tensors[t["uv"]].to(act).view(H, self.value_dim, self.kv_rank).transpose(1, 2).contiguous()
        self.q_gain, self.kv_gain = tensors[t["dq_norm"]].to(f32).contiguous(), tensors[t["dkv_norm"]].to(f32).contiguous()
        if self.position is None:
            self._cos_sin = torch.zeros(2, device=self.env.device)
        else:
            self.position.bind(tensors)
            table, rotary = getattr(self.position, "cos_sin", None), getattr(self.position, "rotary_dim", None)
            if not isinstance(table, torch.Tensor) or rotary != self.rot_dim or tuple(table.shape[1:]) != (self.rot_dim // 2, 2):
                raise TypeError(f"the position part '{self.spec.params['position'].kind}' does not offer cos_sin [positions, {self.rot_dim // 2}, 2] "
                                f"for rotary_dim = rot_dim {self.rot_dim} (see parts.base.PositionEncoding)")
            self._cos_sin = table

    def weight_bytes(self):
        return (self.down.weight_bytes() + self.uq.weight_bytes() + self.o.weight_bytes()
                + (self.uk.numel() + self.uv.numel()) * self.uk.element_size())

    def cache_need(self):
        return CacheNeed("pages", kv_heads=1, head_dim=self.row, window=0, dtype=self.env.act_dtype, planes=1)

    def kernel_libraries(self):
        return {"masked_attention", "gemm_tc" if self.env.compute_dtype == torch.bfloat16 else "gemm_f32"}

    def _tiles(self, pages) -> bool:
        return self.env.act_dtype == torch.bfloat16 and ops.masked_attention_tiles_supported(self.num_heads, 1, self.row, self.kv_rank,
                                                                                             pages.shape[4], 0)

    def _buffers(self, ws, rows):
        H, act = self.num_heads, self.env.act_dtype
        return (ws.get("lattn.cq", rows, (self.q_rank,), act), ws.get("lattn.q", rows, (H, self.key_dim + self.rot_dim), act),
                ws.get("lattn.ql", rows, (H, self.row), act), ws.get("lattn.ol", rows, (H, self.kv_rank), act),
                ws.get("lattn.out", rows, (H * self.value_dim,), act))

    def forward(self, ctx, x, stream, cache):
        n, ws, H, f32 = ctx.n, ctx.workspace, self.num_heads, torch.float32
        Dq, R, rot, V = self.key_dim + self.rot_dim, self.kv_rank, self.rot_dim, self.value_dim
        proj = self.down.forward_partials(x, ws.raw("lattn.proj", (self.down.partial_elems(ws.max_tokens),), f32))
        cq, q, ql, ol, mixed = self._buffers(ws, n)
        ops.latent_prepare(proj, self.q_gain, self.kv_gain, self.eps, ctx.positions, ctx.slots, self._cos_sin, cq, cache.pages, cache.block_table,
                           self.q_rank, R, rot, write_kv=cache.writes)
        qp = self.uq.forward_partials(cq, ws.raw("lattn.q_partials", (self.uq.partial_elems(ws.max_tokens),), f32))
        ops.rotate_heads(qp, ctx.positions, self._cos_sin, q.view(n, H * Dq), H, Dq, self.key_dim, rot)
        ops.head_linear(q, self.uk, ql, tail=rot)
        _attend(ql.view(n, H * self.row), ol.view(n, H * R), cache, ctx, None, None, H, 1, self.row, R, 0, 0, self.scale, self._tiles(cache.pages))
        ops.head_linear(ol, self.uv, mixed.view(n, H, V))
        self.o.forward_add(mixed, stream, ws.raw("lattn.o_partials", (self.o.partial_elems(ws.max_tokens),), f32))

    def emit(self, program, x, cache):
        ws, H, f32 = program.workspace, self.num_heads, torch.float32
        T = ws.max_tokens
        Dq, R, rot, V = self.key_dim + self.rot_dim, self.kv_rank, self.rot_dim, self.value_dim
        proj = ws.raw("lattn.proj", (self.down.partial_elems(T),), f32)
        S = self.down.emit_partials(program, x, proj)
        cq, q, ql, ol, mixed = self._buffers(ws, T)
        pages, table = cache.pages, cache.block_table
        program.add("masked_attention", "sb_op_latent_prepare",
                    [proj, S, program.few_tokens, self.q_gain, self.kv_gain, self._cos_sin, cq, cq.dtype, pages, table, table.shape[1], pages.shape[3],
                     pages.stride(0), self.q_rank, R, rot, pages.shape[4], int(cache.writes)], [self.eps])
        qp = ws.raw("lattn.q_partials", (self.uq.partial_elems(T),), f32)
        S = self.uq.emit_partials(program, cq, qp)
        program.add("masked_attention", "sb_op_rotate_heads", [qp, S, program.few_tokens, self._cos_sin, q, q.dtype, H, Dq, self.key_dim, rot])
        program.add("masked_attention", "sb_op_head_linear", [q, H * Dq, Dq, self.uk, ql, H * self.row, self.row, q.dtype, H, self.key_dim, R, rot])
        _emit_attend(program, ql, ol, cache, None, None, H, 1, self.row, R, 0, 0, self.scale, self._tiles(pages))
        program.add("masked_attention", "sb_op_head_linear", [ol, H * R, R, self.uv, mixed, H * V, V, ol.dtype, H, R, V, 0])
        self.o.emit_add(program, mixed, ws.raw("lattn.o_partials", (self.o.partial_elems(T),), f32))
