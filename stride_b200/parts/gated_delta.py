"""The gated delta rule as a mixer with a state per request (kernels: csrc/delta_rule.cu).

q, k = W x (kv_heads x key_dim), v = W x (heads x value_dim), no biases; each passes a short causal convolution over time per channel (the
last tap the current token's, zeros before the start) and silu; q and k are made unit vectors per head, q also times key_dim^-1/2;
beta = sigmoid(W_b x), one per head; a decay per head and key channel, g = exp(-exp(A_h) softplus(W_a2 (W_a1 x) + dt)). Per head (head h
uses q/k head h / (heads / kv_heads)): S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q. Every head's o is divided by its root
mean square, times a gain of value_dim shared by the heads, times sigmoid(W_g2 (W_g1 x)), and projected by W_o.

The request's record is [S | the convolution's last taps - 1 inputs], float32. The projections that read x are one matrix product
(q | k | v | beta | a1 | g1); the two low-rank second halves are one more, a matrix of two blocks on the diagonal."""
from __future__ import annotations

import torch

from ..kernels.linear import Linear
from ..kernels.native import ImmediateProgram
from .base import CacheNeed, Mixer, register_part
from .spec import TensorPlan

MAX_TAPS = 8


@register_part("mixer", "gated_delta")
class GatedDeltaMixer(Mixer):
    """params: hidden_size, num_heads, num_kv_heads, key_dim, value_dim, taps, decay_rank, gate_rank, norm_eps.
    tensors: q, k, v, q_conv, k_conv, v_conv ([channels, taps]), beta [heads, hidden], a_log [heads], dt_bias [heads key_dim],
    a1 [decay_rank, hidden], a2 [heads key_dim, decay_rank], g1 [gate_rank, hidden], g2 [heads value_dim, gate_rank], norm [value_dim], o."""
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden, self.H, self.G = int(p["hidden_size"]), int(p["num_heads"]), int(p["num_kv_heads"])
        self.D, self.V, self.taps = int(p["key_dim"]), int(p["value_dim"]), int(p["taps"])
        self.ra, self.rg, self.eps = int(p["decay_rank"]), int(p["gate_rank"]), float(p["norm_eps"])
        if self.H % self.G:
            raise ValueError(f"gated delta rule: {self.H} heads do not divide into {self.G} query/key heads")
        if not 1 <= self.taps <= MAX_TAPS:
            raise ValueError(f"gated delta rule: {self.taps} taps (1 to {MAX_TAPS})")
        if self.D > 256:
            raise ValueError(f"gated delta rule: key_dim {self.D} exceeds 256, the most the recurrence kernel holds")
        self.C = 2 * self.G * self.D + self.H * self.V                     # channels that pass the convolution
        self.mid_off, self.width1 = self.C + self.H, self.C + self.H + self.ra + self.rg
        self.width2 = self.H * self.D + self.H * self.V
        self.state_elems = self.H * self.D * self.V
        self.record = self.state_elems + (self.taps - 1) * self.C
        self.cols = self.C + self.H + self.H * self.D                      # what the recurrence reads per token: q | k | v | beta | g
        self.first = self.second = self.o = self.conv = self.a_log = self.dt_bias = self.gain = None

    def tensor_plan(self):
        t, H, G, D, V, W = self.spec.tensors, self.H, self.G, self.D, self.V, self.hidden
        return {t["q"]: TensorPlan((G * D, W)), t["k"]: TensorPlan((G * D, W)), t["v"]: TensorPlan((H * V, W)),
                t["q_conv"]: TensorPlan((G * D, self.taps), zero_mean=True), t["k_conv"]: TensorPlan((G * D, self.taps), zero_mean=True),
                t["v_conv"]: TensorPlan((H * V, self.taps), zero_mean=True), t["beta"]: TensorPlan((H, W)),
                t["a_log"]: TensorPlan((H,), zero_mean=True), t["dt_bias"]: TensorPlan((H * D,), zero_mean=True),
                t["a1"]: TensorPlan((self.ra, W)), t["a2"]: TensorPlan((H * D, self.ra)), t["g1"]: TensorPlan((self.rg, W)),
                t["g2"]: TensorPlan((H * V, self.rg)), t["norm"]: TensorPlan((V,)), t["o"]: TensorPlan((W, H * V))}

    def bind(self, tensors):
        t, f32 = self.spec.tensors, torch.float32
        ws = [tensors[t[r]] for r in ("q", "k", "v", "beta", "a1", "g1")]
        if len({w.dtype for w in ws}) > 1:
            ws = [w.to(f32) for w in ws]
        self.first = Linear(torch.cat(ws, dim=0), self.env.compute_dtype)
        a2, g2 = tensors[t["a2"]], tensors[t["g2"]]
        if a2.dtype != g2.dtype:
            a2, g2 = a2.to(f32), g2.to(f32)
        both = torch.zeros(self.width2, self.ra + self.rg, dtype=a2.dtype, device=a2.device)
        both[:self.H * self.D, :self.ra] = a2
        both[self.H * self.D:, self.ra:] = g2
        self.second = Linear(both, self.env.compute_dtype)
        self.o = Linear(tensors[t["o"]], self.env.compute_dtype)
        self.conv = torch.cat([tensors[t[r]].to(f32) for r in ("q_conv", "k_conv", "v_conv")]).contiguous()
        self.a_log, self.dt_bias = tensors[t["a_log"]].to(f32).contiguous(), tensors[t["dt_bias"]].to(f32).contiguous()
        self.gain = tensors[t["norm"]].to(f32).contiguous()

    def weight_bytes(self):
        return self.first.weight_bytes() + self.second.weight_bytes() + self.o.weight_bytes()

    def cache_need(self):
        return CacheNeed("state", state_shape=(self.record,), state_dtype=torch.float32)

    def kernel_libraries(self):
        return {"delta_rule", "lightning", "elementwise", "gemm_tc" if self.env.compute_dtype == torch.bfloat16 else "gemm_f32"}

    def forward(self, ctx, x, stream, cache):
        with ImmediateProgram(ctx, stream) as program:
            self.emit(program, x, cache)

    def emit(self, program, x, cache):
        ws, f32, H, G, D, V = program.workspace, torch.float32, self.H, self.G, self.D, self.V
        T, few = ws.max_tokens, program.few_tokens
        p1 = ws.raw("delta.first", (self.first.partial_elems(T),), f32)
        S1 = self.first.emit_partials(program, x, p1)
        mid = ws.get("delta.mid", T, (self.ra + self.rg,), self.env.act_dtype)
        program.add("elementwise", "sb_op_cast_columns", [p1, self.width1, S1, few, self.mid_off, self.ra + self.rg, mid, mid.dtype])
        p2 = ws.raw("delta.second", (self.second.partial_elems(T),), f32)
        S2 = self.second.emit_partials(program, mid, p2)
        ready = ws.raw("delta.ready", (T * self.cols,), f32)
        program.add("delta_rule", "sb_op_delta_prepare", [p1, self.width1, S1, p2, self.width2, S2, few, self.conv, self.a_log, self.dt_bias,
                                                          cache.state, self.record, self.state_elems, ready, H, G, D, V, self.taps])
        o = ws.get("delta.o", T, (H * V,), f32)
        program.add("delta_rule", "sb_op_delta_scan", [ready, cache.state, self.record, o, H, G, D, V])
        y = ws.get("delta.y", T, (H * V,), self.env.act_dtype)
        program.add("lightning", "sb_op_group_norm_gate", [o, p2, self.width2, S2, few, H * D, self.gain, self.gain.dtype, y, y.dtype, H, V, 0],
                    [self.eps])
        self.o.emit_add(program, y, ws.raw("delta.o_partials", (self.o.partial_elems(T),), f32))
