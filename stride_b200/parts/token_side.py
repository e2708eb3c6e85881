"""A per-layer input that depends on the token alone (category "rewrite", kind "token_side").

A second embedding table, narrow, holds a slice of `dim` elements per layer for every token. Behind a layer's sublayers, with x the stream:
e = table[token][index dim : (index + 1) dim]; g = act(W_gate x) * e; y = W_proj g; x <- x + gain * y / sqrt(mean(y^2) + eps). The projection
W_gate reads the stream itself (a copy in the activations' dtype), not a normed copy; the last step is the fold of a branch with a norm on
the way that layers with a norm behind their sublayers use (csrc/branch.cu)."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..kernels.linear import Linear
from ..kernels.native import ImmediateProgram
from .base import Rewrite, register_part
from .branch import emit_fold, emit_on_branch
from .spec import TensorPlan


@register_part("rewrite", "token_side")
class TokenSide(Rewrite):
    """params: hidden_size, vocab_size, dim, slices (of the table's row), index (this layer's slice), eps, activation ("gelu_tanh" or "silu").
    tensors: table [vocab, slices dim], gate [dim, hidden], proj [hidden, dim], norm [hidden]."""
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden, self.vocab, self.dim = int(p["hidden_size"]), int(p["vocab_size"]), int(p["dim"])
        self.slices, self.index, self.eps = int(p["slices"]), int(p["index"]), float(p["eps"])
        self.activation = str(p.get("activation", "gelu_tanh"))
        if not 0 <= self.index < self.slices or self.activation not in ops.GATE_ACTIVATIONS:
            raise ValueError(f"token side input: slice {self.index} of {self.slices}, activation {self.activation!r}")
        self.table = self.gate = self.proj = self.gain = None

    def tensor_plan(self):
        t = self.spec.tensors
        return {t["table"]: TensorPlan((self.vocab, self.slices * self.dim), zero_mean=True), t["gate"]: TensorPlan((self.dim, self.hidden)),
                t["proj"]: TensorPlan((self.hidden, self.dim)), t["norm"]: TensorPlan((self.hidden,))}

    def bind(self, tensors):
        t = self.spec.tensors
        self.table = tensors[t["table"]].contiguous()
        self.gate = Linear(tensors[t["gate"]], self.env.compute_dtype)
        self.proj = Linear(tensors[t["proj"]], self.env.compute_dtype)
        self.gain = tensors[t["norm"]].contiguous()

    def weight_bytes(self):
        return self.gate.weight_bytes() + self.proj.weight_bytes()

    def kernel_libraries(self):
        return {"elementwise", "branch", "gemm_tc" if self.env.compute_dtype == torch.bfloat16 else "gemm_f32"}

    def forward(self, ctx, stream):
        with ImmediateProgram(ctx, stream) as program:
            self.emit(program)

    def emit(self, program):
        ws, f32, act = program.workspace, torch.float32, self.env.act_dtype
        T, few = ws.max_tokens, program.few_tokens
        x = ws.get("side.x", T, (self.hidden,), act)
        flat, S, _ = program.take_pending() or (None, 1, 0)
        program.add("elementwise", "sb_op_stream_cast", [program.h, flat, S, few, x, x.dtype, self.hidden])
        sums = ws.raw("side.gate", (self.gate.partial_elems(T),), f32)
        Sg = self.gate.emit_partials(program, x, sums)
        g = ws.get("side.g", T, (self.dim,), act)
        program.add("elementwise", "sb_op_token_gate", [sums, self.dim, Sg, few, self.table, self.table.dtype, self.slices * self.dim,
                                                        self.index * self.dim, self.vocab, getattr(program, "sampled", None), g, g.dtype,
                                                        ops.GATE_ACTIVATIONS[self.activation]])
        branch = ws.get("block.branch", T, (self.hidden,), f32)
        source = emit_on_branch(program, branch, lambda: self.proj.emit_add(program, g, ws.raw("side.proj", (self.proj.partial_elems(T),), f32)))
        emit_fold(program, [(*source, 1.0)], self.gain, self.hidden, norm_eps=self.eps)
