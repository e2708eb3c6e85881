"""Softmax attention over the paged cache with an output gate, put together from parameters (kernels: csrc/masked_attention.cu).

q, k, v = W x (+ b); q and k may be RMS-normed, over the whole projection (gains of that size) or per head (one gain of the head's size
for all heads); the first `rotary_dim` elements of every q and k head may be rotated by the position (a position part's table; pairs
(2i, 2i + 1) when `interleaved`, else (i, i + rotary_dim / 2)); q may grow with the position, times 1 + c ln(floor((p + 1) / every) + 1).
score = scale q.k; i sees j <= i with i - j < window (if a window is set) and floor(i / chunk) = floor(j / chunk) (if chunks are set:
their borders are absolute positions, wherever a prompt was cut); ordinary softmax, or with one more term exp(0) in the denominator (`sink` "zero": a key of score 0
without a value). The heads' results are multiplied by sigmoid(W_g x), one gate per element or one per head, and projected by W_o (+ b).

With `maps` 2 (differential attention) a head has two queries and a key head two keys, the second behind the first in the head's rows; the two
softmax maps share the values, and the head's result is a1 - lambda a2 with lambda = exp(lq1.lk1) - exp(lq2.lk2) + diff, RMS-normed over
the head's values (no gain), times 1 - diff. The kernels see 2 H query heads over 2 G key heads: the query rows are reordered so that
the heads of a (key head, map) lie side by side, and the value rows are stored once per map."""
from __future__ import annotations

import math

import torch

from ..kernels import ops
from ..kernels.linear import Linear
from ..kernels.native import ImmediateProgram
from .base import CacheNeed, Mixer, part_class, register_part
from .masked_attention import _page_where
from .spec import TensorPlan


@register_part("mixer", "gated_attention")
class GatedAttentionMixer(Mixer):
    """params: hidden_size, num_heads, num_kv_heads, key_dim, value_dim, scale, norm_eps, window (0: none), chunk (0: none), sink (None or
    "zero"), qk_norm (None, "projection" or "head"), bias (q, k, v have biases), o_bias, position (a PartSpec of category "position" offering
    cos_sin, or None), interleaved, gate ("element" or "head"), maps (1 or 2), diff (with two maps), q_temp ((coef, every) or None).
    tensors: q, k, v, g, o and, as the parameters say, q_bias, k_bias, v_bias, o_bias, q_norm, k_norm, lq1, lk1, lq2, lk2."""
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.H, self.G, self.D, self.V = int(p["num_heads"]), int(p["num_kv_heads"]), int(p["key_dim"]), int(p["value_dim"])
        self.scale, self.eps = float(p["scale"]), float(p.get("norm_eps", 1e-6))
        self.window, self.chunk = int(p.get("window", 0) or 0), int(p.get("chunk", 0) or 0)
        self.sink, self.qk_norm = p.get("sink"), p.get("qk_norm")
        self.biased, self.o_biased = bool(p.get("bias")), bool(p.get("o_bias"))
        self.interleaved, self.gate = bool(p.get("interleaved")), p.get("gate", "element")
        self.maps, self.diff = int(p.get("maps", 1)), float(p.get("diff", 0.0))
        self.q_temp = tuple(p["q_temp"]) if p.get("q_temp") else None
        if self.H % self.G:
            raise ValueError(f"gated attention: {self.H} heads do not divide into {self.G} key/value heads")
        if self.maps not in (1, 2) or self.gate not in ("element", "head") or self.sink not in (None, "zero") or \
                self.qk_norm not in (None, "projection", "head"):
            raise ValueError(f"gated attention: maps {self.maps}, gate {self.gate!r}, sink {self.sink!r}, qk_norm {self.qk_norm!r}")
        if max(self.D, self.V) > 640:
            raise ValueError(f"gated attention: key size {self.D} / value size {self.V} exceed 640, the most the kernel holds")
        pos = p.get("position")
        self.position = part_class("position", pos.kind)(pos, env) if pos is not None else None
        self.Hq, self.Hkv = self.maps * self.H, self.maps * self.G          # what the kernels see
        self.gates = self.H * self.V if self.gate == "element" else self.H
        self.g_off = self.Hq * self.D + self.Hkv * (self.D + self.V)
        self.width = self.g_off + self.gates
        self.proj = self.o = self.bias = self.o_bias = self.q_gain = self.k_gain = self.sinks = self.cos_sin = None
        self.rot, self.lam = 0, 0.0

    def tensor_plan(self):
        t, H, G, D, V, M, W = self.spec.tensors, self.H, self.G, self.D, self.V, self.maps, self.hidden
        plan = {t["q"]: TensorPlan((H * M * D, W)), t["k"]: TensorPlan((G * M * D, W)), t["v"]: TensorPlan((G * V, W)),
                t["g"]: TensorPlan((self.gates, W)), t["o"]: TensorPlan((W, H * V))}
        if self.biased:
            plan.update({t["q_bias"]: TensorPlan((H * M * D,), zero_mean=True), t["k_bias"]: TensorPlan((G * M * D,), zero_mean=True),
                         t["v_bias"]: TensorPlan((G * V,), zero_mean=True)})
        if self.o_biased:
            plan[t["o_bias"]] = TensorPlan((W,), zero_mean=True)
        if self.qk_norm == "projection":
            plan.update({t["q_norm"]: TensorPlan((H * M * D,)), t["k_norm"]: TensorPlan((G * M * D,))})
        elif self.qk_norm == "head":
            plan.update({t["q_norm"]: TensorPlan((D,)), t["k_norm"]: TensorPlan((D,))})
        if M == 2:
            plan.update({t[r]: TensorPlan((D,), zero_mean=True) for r in ("lq1", "lk1", "lq2", "lk2")})
        if self.position is not None:
            plan.update(self.position.tensor_plan())
        return plan

    def _by_map(self, q: torch.Tensor) -> torch.Tensor:
        """Query rows [H][maps][D] reordered to [G][maps][H / G][D]: the heads of a (key head, map) side by side."""
        if self.maps == 1:
            return q
        tail = q.shape[1:]
        return q.reshape(self.G, self.H // self.G, 2, self.D, *tail).transpose(1, 2).reshape(q.shape[0], *tail)

    def _per_map(self, v: torch.Tensor) -> torch.Tensor:
        """Value rows [G][V] stored once per map: [G][maps][V]."""
        if self.maps == 1:
            return v
        tail = v.shape[1:]
        return v.reshape(self.G, 1, self.V, *tail).expand(self.G, 2, self.V, *tail).reshape(2 * v.shape[0], *tail)

    def bind(self, tensors):
        t, f32 = self.spec.tensors, torch.float32
        ws = [self._by_map(tensors[t["q"]]), tensors[t["k"]], self._per_map(tensors[t["v"]]), tensors[t["g"]]]
        if len({w.dtype for w in ws}) > 1:
            ws = [w.to(f32) for w in ws]
        self.proj = Linear(torch.cat(ws, dim=0), self.env.compute_dtype)
        self.o = Linear(tensors[t["o"]], self.env.compute_dtype)
        if self.biased:
            self.bias = torch.cat([self._by_map(tensors[t["q_bias"]]).to(f32), tensors[t["k_bias"]].to(f32),
                                   self._per_map(tensors[t["v_bias"]]).to(f32)]).contiguous()
        if self.o_biased:
            self.o_bias = tensors[t["o_bias"]].to(f32).contiguous()
        if self.qk_norm is not None:
            qg, kg = tensors[t["q_norm"]].to(f32), tensors[t["k_norm"]].to(f32)
            self.q_gain, self.k_gain = (self._by_map(qg) if self.qk_norm == "projection" else qg).contiguous(), kg.contiguous()
        if self.sink == "zero":
            self.sinks = torch.zeros(self.Hq, dtype=f32, device=self.env.device)
        if self.maps == 2:
            dot = lambda a, b: float((tensors[t[a]].to(torch.float64) * tensors[t[b]].to(torch.float64)).sum())
            self.lam = math.exp(dot("lq1", "lk1")) - math.exp(dot("lq2", "lk2")) + self.diff
        if self.position is not None:
            self.position.bind(tensors)
            table, rot = getattr(self.position, "cos_sin", None), getattr(self.position, "rotary_dim", None)
            if not isinstance(table, torch.Tensor) or not rot or rot % 2 or rot > self.D or tuple(table.shape[1:]) != (rot // 2, 2):
                raise TypeError(f"the position part '{self.spec.params['position'].kind}' does not offer cos_sin [positions, rotary_dim / 2, 2] "
                                f"for an even rotary_dim <= {self.D} (see parts.base.PositionEncoding)")
            self.cos_sin, self.rot = table, int(rot)

    def weight_bytes(self):
        return self.proj.weight_bytes() + self.o.weight_bytes()

    def cache_need(self):
        return CacheNeed("pages", kv_heads=self.Hkv, head_dim=max(self.D, self.V), window=self.window or self.chunk, dtype=self.env.act_dtype)

    def kernel_libraries(self):
        return {"masked_attention", "branch", "gemm_tc" if self.env.compute_dtype == torch.bfloat16 else "gemm_f32"}

    def _tiles(self, pages) -> bool:
        return self.env.act_dtype == torch.bfloat16 and ops.masked_attention_tiles_supported(self.Hq, self.Hkv, self.D, self.V, pages.shape[4],
                                                                                             pages.stride(1))

    def forward(self, ctx, x, stream, cache):
        with ImmediateProgram(ctx, stream) as program:
            self.emit(program, x, cache)

    def emit(self, program, x, cache):
        ws, f32, act = program.workspace, torch.float32, self.env.act_dtype
        T, Hq, Hkv, D, V = ws.max_tokens, self.Hq, self.Hkv, self.D, self.V
        proj = ws.raw("gattn.proj", (self.proj.partial_elems(T),), f32)
        S = self.proj.emit_partials(program, x, proj)
        q = ws.get("gattn.q", T, (Hq * D,), act)
        pages, table = cache.pages, cache.block_table
        where = _page_where(pages, table)
        mode = {None: 0, "projection": 1, "head": 2}[self.qk_norm]
        coef, every = self.q_temp if self.q_temp else (0.0, 0)
        program.add("masked_attention", "sb_op_qkv_prepare",
                    [proj, self.width, S, program.few_tokens, self.bias, self.q_gain, self.k_gain, mode, self.cos_sin, self.rot, int(self.interleaved),
                     int(every), q, q.dtype, pages, table, *where, Hq, Hkv, D, V, pages.shape[4], int(cache.writes)], [self.eps, coef])
        a = ws.get("gattn.a", T, (Hq * V,), f32)
        if self._tiles(pages):
            program.add("masked_attention", "sb_op_masked_attention_tiles",
                        [q, a, pages, table, *where, None, self.sinks, Hq, Hkv, D, V, pages.shape[4], self.window, 0, self.chunk, 1], [self.scale])
        else:
            program.add("masked_attention", "sb_op_masked_attention",
                        [q, a, q.dtype, pages, table, *where, None, self.sinks, Hq, Hkv, D, V, pages.shape[4], self.window, 0, self.chunk, 1],
                        [self.scale])
        y = ws.get("gattn.y", T, (self.H * V,), act)
        program.add("masked_attention", "sb_op_head_gate",
                    [a, proj, self.width, S, program.few_tokens, self.g_off, y, y.dtype, self.H, self.G, V, self.maps, int(self.gate == "head")],
                    [self.lam, 1.0 - self.diff, self.eps])
        if self.o_bias is not None:      # onto the stream (or the branch this mixer runs on) in front of the projection's sums
            program.need_folded("an output bias")
            program.add("branch", "sb_op_stream_add", [program.h, None, 1, program.few_tokens, None, self.o_bias, self.o_bias.dtype, self.hidden])
        self.o.emit_add(program, y, ws.raw("gattn.o_partials", (self.o.partial_elems(T),), f32))
