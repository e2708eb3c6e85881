"""Re-entry of the embedding into the residual stream: h <- W [h; e], e being the embedding output of the same
token and W a [hidden, 2 hidden] matrix whose first half of columns meets h. Models that run a group of layers
several times put it in front of every pass, so that each pass sees the token itself beside what the pass before made
of it. The two streams are laid side by side in the activation dtype (the stream's pending partial sums folded in on the
way, and h set to zero behind the read) and go through one matrix product, whose K ranges' partial sums are left pending
on the now empty stream like those of any other projection: the next norm adds them, h = 0 + (r0 + r1 + ..).

"embedding_add": h <- (h + e) + s, the plain form of the same idea: the embedding output is added (not mixed in through a matrix; a
pass may also go without it) and a stored vector s, one row of a [passes, hidden] table, marks the pass. All in 32-bit."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..kernels.linear import Linear
from .base import Rewrite, register_part
from .spec import TensorPlan


@register_part("rewrite", "embedding_mix")
class EmbeddingMix(Rewrite):
    """params: hidden_size, optional (True: the matrix may be absent, for a part that no schedule entry runs).
    tensors: weight [hidden, 2 hidden]."""
    graph_safe = True
    reads_embedding = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec.params["hidden_size"])
        self.linear = None

    def tensor_plan(self):
        return {self.spec.tensors["weight"]: TensorPlan((self.hidden, 2 * self.hidden), optional=bool(self.spec.params.get("optional", False)))}

    def bind(self, tensors):
        weight = tensors.get(self.spec.tensors["weight"])
        if weight is not None:
            self.linear = Linear(weight, self.env.compute_dtype)

    def weight_bytes(self):
        return self.linear.weight_bytes() if self.linear is not None else 0

    def kernel_libraries(self):
        return {"elementwise", "gemm_tc" if self.env.compute_dtype == torch.bfloat16 else "gemm_f32"}

    def forward(self, ctx, stream):
        if ctx.embedding_output is None:
            raise RuntimeError("embedding_mix: the model did not keep the embedding output")
        both = ctx.workspace.get("reentry.both", ctx.n, (2 * self.hidden,), ctx.act_dtype)
        ops.concat_rows(stream.h, ctx.embedding_output, both, partials=stream.take_pending(), clear_a=True)
        self.linear.forward_add(both, stream, ctx.workspace.raw("reentry.partials", (self.linear.partial_elems(ctx.workspace.max_tokens),), torch.float32))

    def emit(self, program):
        ws = program.workspace
        both = ws.get("reentry.both", ws.max_tokens, (2 * self.hidden,), self.env.act_dtype)
        flat, S, _ = program.take_pending() or (None, 1, 0)
        program.add("elementwise", "sb_op_concat_rows", [program.h, flat, S, program.few_tokens, program.embedding_output, both, both.dtype,
                                                          self.hidden, 1])
        self.linear.emit_add(program, both, ws.raw("reentry.partials", (self.linear.partial_elems(ws.max_tokens),), torch.float32))


@register_part("rewrite", "embedding_add")
class EmbeddingAdd(Rewrite):
    """params: hidden_size, rows (of the table), row (the one this part adds), add_embedding (False: only the vector is added).
    tensors: table [rows, hidden] (optional when `row` is None: a part that adds the embedding alone)."""
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden, self.rows = int(p["hidden_size"]), int(p.get("rows", 0))
        self.row = p.get("row")
        self.reads_embedding = bool(p.get("add_embedding", True))
        if self.row is not None and not 0 <= int(self.row) < self.rows:
            raise ValueError(f"embedding_add: row {self.row} of a table of {self.rows}")
        self.vector = None

    def tensor_plan(self):
        if self.row is None:
            return {}
        return {self.spec.tensors["table"]: TensorPlan((self.rows, self.hidden), zero_mean=True)}

    def bind(self, tensors):
        if self.row is not None:
            self.vector = tensors[self.spec.tensors["table"]][int(self.row)].contiguous()

    def kernel_libraries(self):
        return {"branch"}

    def forward(self, ctx, stream):
        if self.reads_embedding and ctx.embedding_output is None:
            raise RuntimeError("embedding_add: the model did not keep the embedding output")
        ops.stream_add(stream.h, ctx.embedding_output if self.reads_embedding else None, self.vector, partials=stream.take_pending())

    def emit(self, program):
        flat, S, _ = program.take_pending() or (None, 1, 0)
        program.add("branch", "sb_op_stream_add", [program.h, flat, S, program.few_tokens, program.embedding_output if self.reads_embedding else None,
                                                   self.vector, self.vector.dtype if self.vector is not None else 0, self.hidden])
