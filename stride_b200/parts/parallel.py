"""Several mixers side by side: all read the same normed activations, and the result is the sum of theirs, each times a
constant, r = c_0 m_0(x) + c_1 m_1(x). Every member keeps its own cache or state (the schedule entry asks the cache
manager with a list of needs), runs on a branch of its own, and one pass takes the branches into the stream."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Mixer, part_class, register_part
from .branch import Branch, emit_fold, emit_on_branch


@register_part("mixer", "parallel")
class ParallelMixer(Mixer):
    """params: hidden_size, members (PartSpecs of category "mixer"; two), scales (one constant per member)."""
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec.params["hidden_size"])
        members = list(spec.params["members"])
        self.scales = [float(c) for c in spec.params["scales"]]
        if len(members) != 2 or len(self.scales) != 2:
            raise ValueError(f"parallel mixer: {len(members)} members with {len(self.scales)} scales (two of each)")
        self.members = [part_class("mixer", m.kind)(m, env) for m in members]
        self.graph_safe = all(m.graph_safe for m in self.members)

    def tensor_plan(self):
        plan = {}
        for m in self.members:
            plan.update(m.tensor_plan())
        return plan

    def bind(self, tensors):
        for m in self.members:
            m.bind(tensors)

    def weight_bytes(self):
        return sum(m.weight_bytes() for m in self.members)

    def cache_need(self):
        return [m.cache_need() for m in self.members]

    def kernel_libraries(self):
        return set().union({"branch"}, *(m.kernel_libraries() for m in self.members))

    def _buffers(self, ws, rows):
        return [ws.get(f"parallel.branch{k}", rows, (self.hidden,), torch.float32) for k in range(2)]

    def forward_sources(self, ctx, x, cache):
        """The members' results as [(Branch, constant)], left to the caller to fold."""
        branches = [Branch(b) for b in self._buffers(ctx.workspace, ctx.n)]
        for m, b, c in zip(self.members, branches, cache.parts):
            m.forward(ctx, x, b, c)
        return list(zip(branches, self.scales))

    def forward(self, ctx, x, stream, cache):
        (a, ca), (b, cb) = self.forward_sources(ctx, x, cache)
        stream.fold()
        (ah, ap), (bh, bp) = a.source(), b.source()
        ops.branch_fold(stream.h, a=ah, a_partials=ap, ca=ca, b=bh, b_partials=bp, cb=cb)

    def emit_sources(self, program, x, cache):
        buffers = self._buffers(program.workspace, program.workspace.max_tokens)
        return [(*emit_on_branch(program, buf, lambda m=m, c=c: m.emit(program, x, c)), scale)
                for m, buf, c, scale in zip(self.members, buffers, cache.parts, self.scales)]

    def emit(self, program, x, cache):
        emit_fold(program, self.emit_sources(program, x, cache), None, self.hidden)


@register_part("mixer", "parallel_normed")
class NormedParallelMixer(Mixer):
    """Two mixers side by side whose results are each RMS-normed over the model width, with a gain of its own, before their weighted sum:
    r = c_0 g_0 * m_0(x) / rms(m_0(x)) + c_1 g_1 * m_1(x) / rms(m_1(x)). params: hidden_size, members (two PartSpecs of category "mixer"),
    scales (a constant per member), eps. tensors: norms (the two gains' names)."""
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden, self.eps = int(spec.params["hidden_size"]), float(spec.params["eps"])
        members = list(spec.params["members"])
        self.scales = [float(c) for c in spec.params["scales"]]
        if len(members) != 2 or len(self.scales) != 2 or len(spec.tensors["norms"]) != 2:
            raise ValueError("parallel mixer with norms: two members, two constants and two gains")
        self.members = [part_class("mixer", m.kind)(m, env) for m in members]
        self.graph_safe = all(m.graph_safe for m in self.members)
        self.gains = self._outer = None

    def tensor_plan(self):
        from .spec import TensorPlan
        plan = {name: TensorPlan((self.hidden,)) for name in self.spec.tensors["norms"]}
        for m in self.members:
            plan.update(m.tensor_plan())
        return plan

    def bind(self, tensors):
        for m in self.members:
            m.bind(tensors)
        self.gains = [tensors[name].to(torch.float32).contiguous() for name in self.spec.tensors["norms"]]

    def weight_bytes(self):
        return sum(m.weight_bytes() for m in self.members)

    def cache_need(self):
        return [m.cache_need() for m in self.members]

    def kernel_libraries(self):
        return set().union({"branch"}, *(m.kernel_libraries() for m in self.members))

    def forward(self, ctx, x, stream, cache):
        from ..kernels.native import ImmediateProgram
        with ImmediateProgram(ctx, stream) as program:
            self.emit(program, x, cache)

    def forward_scaled(self, ctx, x, stream, cache, gain):
        from ..kernels.native import ImmediateProgram
        with ImmediateProgram(ctx, stream) as program:
            self.emit_scaled(program, x, cache, gain)

    def emit_scaled(self, program, x, cache, gain):
        """The result times a gain vector of the width (a layer scale), added to the program's stream by the same pass that norms the members."""
        key = id(gain)
        if self._outer is None or self._outer[0] != key:
            self._outer = (key, gain.to(torch.float32).contiguous())
        self.emit(program, x, cache, self._outer[1])

    def emit(self, program, x, cache, outer=None):
        ws = program.workspace
        buffers = [ws.get(f"parallel.branch{k}", ws.max_tokens, (self.hidden,), torch.float32) for k in range(2)]
        (a, pa), (b, pb) = [emit_on_branch(program, buf, lambda m=m, c=c: m.emit(program, x, c))
                            for m, buf, c in zip(self.members, buffers, cache.parts)]
        (fa, Sa, _), (fb, Sb, _) = pa or (None, 1, 0), pb or (None, 1, 0)
        program.need_folded("mixers side by side")
        program.add("branch", "sb_op_branch_pair_norm_fold",
                    [program.h, a, fa, Sa, program.few_tokens, b, fb, Sb, self.gains[0], self.gains[1], self.gains[0].dtype, self.hidden, outer],
                    [self.scales[0], self.scales[1], self.eps])
