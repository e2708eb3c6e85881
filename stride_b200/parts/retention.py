"""Retention: linear attention with a fixed decay per head and no softmax or denominator, as a mixer with a state per request.

Per head: q, k = W x rotated by the position in the first `rotary_dim` elements (pairs (i, i + rotary_dim / 2)), k times key_dim^-1/2 behind
the rotation, v = W x; S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t. Every head's o is divided by its root mean square (no gain), the
heads side by side are multiplied by silu(W_g x) and projected by W_o. The recurrence is the decayed linear-attention kernel
(csrc/lightning.cu) fed with ready-made q, k, v; rotation, recurrence, norm and gate are 32-bit in both precisions of the engine."""
from __future__ import annotations

import torch

from ..kernels.linear import Linear
from ..kernels.native import ImmediateProgram
from .base import CacheNeed, Mixer, part_class, register_part
from .spec import TensorPlan


@register_part("mixer", "retention")
class RetentionMixer(Mixer):
    """params: hidden_size, num_heads, key_dim, value_dim, decay (one factor per head), norm_eps, position (a PartSpec of category "position"
    offering cos_sin, or None). tensors: q, k, v, g, o."""
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden, self.H, self.D, self.V = int(p["hidden_size"]), int(p["num_heads"]), int(p["key_dim"]), int(p["value_dim"])
        self.eps = float(p["norm_eps"])
        decay = [float(d) for d in p["decay"]]
        if len(decay) != self.H:
            raise ValueError(f"retention: {len(decay)} decay factors for {self.H} heads")
        if self.D > 256:
            raise ValueError(f"retention: key_dim {self.D} exceeds 256, the most the recurrence kernel holds")
        self._decay_host = torch.tensor(decay, dtype=torch.float64).to(torch.float32)
        pos = p.get("position")
        self.position = part_class("position", pos.kind)(pos, env) if pos is not None else None
        H, D, V = self.H, self.D, self.V
        self.k_off, self.v_off, self.g_off, self.width = H * D, 2 * H * D, 2 * H * D + H * V, 2 * H * D + 2 * H * V
        self.proj = self.o = self.decay = self.cos_sin = None
        self.rot = 0

    def tensor_plan(self):
        t, H, D, V, W = self.spec.tensors, self.H, self.D, self.V, self.hidden
        plan = {t["q"]: TensorPlan((H * D, W)), t["k"]: TensorPlan((H * D, W)), t["v"]: TensorPlan((H * V, W)), t["g"]: TensorPlan((H * V, W)),
                t["o"]: TensorPlan((W, H * V))}
        if self.position is not None:
            plan.update(self.position.tensor_plan())
        return plan

    def bind(self, tensors):
        t = self.spec.tensors
        ws = [tensors[t[r]] for r in ("q", "k", "v", "g")]
        if len({w.dtype for w in ws}) > 1:
            ws = [w.to(torch.float32) for w in ws]
        self.proj = Linear(torch.cat(ws, dim=0), self.env.compute_dtype)
        self.o = Linear(tensors[t["o"]], self.env.compute_dtype)
        self.decay = self._decay_host.to(self.env.device)
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
        return CacheNeed("state", state_shape=(self.H, self.D, self.V), state_dtype=torch.float32)

    def kernel_libraries(self):
        return {"lightning", "gemm_tc" if self.env.compute_dtype == torch.bfloat16 else "gemm_f32"}

    def forward(self, ctx, x, stream, cache):
        with ImmediateProgram(ctx, stream) as program:
            self.emit(program, x, cache)

    def emit(self, program, x, cache):
        ws, f32, H, D, V = program.workspace, torch.float32, self.H, self.D, self.V
        T, few = ws.max_tokens, program.few_tokens
        proj = ws.raw("retention.proj", (self.proj.partial_elems(T),), f32)
        S = self.proj.emit_partials(program, x, proj)
        ready = ws.raw("retention.qkv", (T * self.g_off,), f32)
        program.add("lightning", "sb_op_rotate_qk", [proj, self.width, S, few, 0, self.k_off, self.v_off, self.cos_sin, self.rot, 0, ready, H, D, V],
                    [float(D) ** -0.5])
        o = ws.get("retention.o", T, (H * V,), f32)
        program.add("lightning", "sb_op_lightning_scan", [ready, self.g_off, 1, few, 0, self.k_off, self.v_off, self.decay, cache.state, o, H, D, V, None, 1])
        y = ws.get("retention.y", T, (H * V,), self.env.act_dtype)
        program.add("lightning", "sb_op_group_norm_gate", [o, proj, self.width, S, few, self.g_off, None, 0, y, y.dtype, H, V, 1], [self.eps])
        self.o.emit_add(program, y, ws.raw("retention.o_partials", (self.o.partial_elems(T),), f32))
