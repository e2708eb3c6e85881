"""Sublayers whose result is scaled before it joins the residual stream.

"layer_scale" (category "branch_scale"): h += w * r, w a vector of the stream's width stored per sublayer, r the
sublayer's result. Blocks "prenorm_scaled" and "prenorm_scaled_mixer": h += w1 * mixer(norm(h)), then (the first kind)
h += w2 * feed_forward(norm(h)). The mixer and the feed-forward are the same parts that other blocks use: they are
handed a branch, a `ResidualStream` over a float32 buffer that is zero between uses, instead of the stream, so their
last projection adds into the branch or leaves its K ranges' partial sums pending on it; the scale then takes
both into the stream in one pass (csrc/branch.cu) and leaves the branch zero again. A part that is several parts side by
side may hand its members' branches over unfolded (`forward_sources` / `emit_sources`), so that one pass scales and adds them all.

"rmsnorm" (category "branch_scale" too): h += w * r / sqrt(mean(r^2) + eps), a norm on the sublayer's result, for designs that norm a
sublayer on both sides; the same blocks, the same branches, one kernel that norms on the way."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Block, BranchScale, register_part
from .context import ResidualStream
from .spec import TensorPlan


class Branch(ResidualStream):
    """A residual stream over a branch buffer that notes whether anything asked for the buffer: a sublayer whose last projection
    only leaves partial sums pending never does, and the fold then neither reads nor clears the buffer."""

    def __init__(self, buffer: torch.Tensor):
        self._buffer, self.pending, self.touched = buffer, None, False

    @property
    def h(self):
        self.touched = True
        return self._buffer

    def source(self):
        """(buffer or None, pending partial sums or None), what a fold takes."""
        return (self._buffer if self.touched else None), self.take_pending()


def emit_on_branch(program, branch: torch.Tensor, emit) -> tuple:
    """Run `emit()` (a part's `emit` that adds to the program's stream) with `branch` in the stream's place; returns (the branch if an
    operation wrote into it, else None; the partial sums left pending, or None)."""
    program.need_folded("a sublayer on a branch")
    main = program._h
    program.h = branch
    try:
        emit()
        return (branch if program.h_touched else None), program.take_pending()
    finally:
        program.h = main


@register_part("branch_scale", "layer_scale")
class LayerScale(BranchScale):
    """params: size. tensors: weight [size]."""
    graph_safe = True
    gain_only = True          # nothing but a gain vector: a part that folds its own result (`emit_scaled`) may apply it on the way

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.size = int(spec.params["size"])
        self.weight = None

    def tensor_plan(self):
        return {self.spec.tensors["weight"]: TensorPlan((self.size,))}

    def bind(self, tensors):
        self.weight = tensors[self.spec.tensors["weight"]].contiguous()

    def weight_bytes(self):
        return self.weight.numel() * self.weight.element_size()

    def kernel_libraries(self):
        return {"branch"}

    def forward(self, ctx, sources, stream):
        """sources: one or two (Branch, constant)."""
        stream.fold()
        (a, pa), ca = sources[0][0].source(), sources[0][1]
        (b, pb), cb = (sources[1][0].source(), sources[1][1]) if len(sources) > 1 else ((None, None), 1.0)
        ops.branch_fold(stream.h, a=a, a_partials=pa, ca=ca, b=b, b_partials=pb, cb=cb, gain=self.weight)

    def emit(self, program, sources):
        """sources: one or two (buffer or None, pending partial sums or None, constant)."""
        program.need_folded("a layer scale")
        emit_fold(program, sources, self.weight, self.size)


@register_part("branch_scale", "rmsnorm")
class BranchRMSNorm(BranchScale):
    """The sublayer's result joins the residual RMS-normed over its row, times a gain. params: size, eps, offset (0 by default: the stored
    vector is the gain's distance from it). tensors: weight [size]."""
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.size, self.eps = int(spec.params["size"]), float(spec.params["eps"])
        self.offset = float(spec.params.get("offset", 0.0))
        self.weight = None

    def tensor_plan(self):
        return {self.spec.tensors["weight"]: TensorPlan((self.size,), zero_mean=self.offset != 0.0)}

    def bind(self, tensors):
        self.weight = tensors[self.spec.tensors["weight"]].contiguous()
        if self.offset != 0.0:
            self.weight = (self.weight.to(torch.float32) + self.offset).contiguous()

    def weight_bytes(self):
        return self.weight.numel() * self.weight.element_size()

    def kernel_libraries(self):
        return {"branch"}

    def forward(self, ctx, sources, stream):
        """sources: one or two (Branch, constant)."""
        stream.fold()
        (a, pa), ca = sources[0][0].source(), sources[0][1]
        (b, pb), cb = (sources[1][0].source(), sources[1][1]) if len(sources) > 1 else ((None, None), 1.0)
        ops.branch_norm_fold(stream.h, self.weight, self.eps, a=a, a_partials=pa, ca=ca, b=b, b_partials=pb, cb=cb)

    def emit(self, program, sources):
        program.need_folded("a norm behind a sublayer")
        emit_fold(program, sources, self.weight, self.size, norm_eps=self.eps)


def emit_fold(program, sources, gain, width: int, norm_eps: float = None) -> None:
    """The operation that takes one or two branches (buffer or None, pending or None, constant) into the program's stream; with
    `norm_eps` their sum is RMS-normed over its row before the gain."""
    if not 1 <= len(sources) <= 2:
        raise ValueError("a fold takes one or two branches")
    (a, pa, ca), (b, pb, cb) = sources[0], sources[1] if len(sources) > 1 else (None, None, 1.0)
    (fa, Sa, _), (fb, Sb, _) = pa or (None, 1, 0), pb or (None, 1, 0)
    if a is None and fa is None:
        raise ValueError("a branch that nothing wrote into")
    ints = [program.h, a, fa, Sa, program.few_tokens, b, fb, Sb, gain, gain.dtype if gain is not None else 0, width]
    if norm_eps is None:
        program.add("branch", "sb_op_branch_fold", ints, [ca, cb])
    else:       # the branches' sum is RMS-normed over its row on the way
        program.add("branch", "sb_op_branch_norm_fold", ints, [ca, cb, norm_eps])


class _ScaledBlock(Block):
    graph_safe = True

    def _branch(self, ws, rows, width):
        return ws.get("block.branch", rows, (width,), torch.float32)

    def _sublayer(self, ctx, stream, norm, part, run, scale):
        """`part` may offer `forward_sources(ctx, x, ...)`: its result as branches with constants that it leaves to the caller to
        fold (several mixers side by side do); every other part runs on one branch."""
        width = stream.h.shape[1]
        x = ctx.workspace.get("block.x", ctx.n, (width,), ctx.act_dtype)
        norm.forward(ctx, stream, x)
        if hasattr(part, "forward_scaled") and getattr(scale, "gain_only", False):
            stream.fold()
            return run(lambda c, x_, *rest: part.forward_scaled(c, x_, stream, *rest, scale.weight), x)
        if hasattr(part, "forward_sources"):
            sources = run(part.forward_sources, x)
        else:
            branch = Branch(self._branch(ctx.workspace, ctx.n, width))
            run(part.forward, x, branch)
            sources = [(branch, 1.0)]
        scale.forward(ctx, sources, stream)

    def _emit_sublayer(self, program, norm, part, run, scale):
        ws, width = program.workspace, program.h.shape[1]
        x = ws.get("block.x", ws.max_tokens, (width,), self.env.act_dtype)
        norm.emit(program, x)
        if hasattr(part, "emit_scaled") and getattr(scale, "gain_only", False):
            program.need_folded("a sublayer that folds its own result")
            return run(lambda pr, x_, *rest: part.emit_scaled(pr, x_, *rest, scale.weight), x)
        if hasattr(part, "emit_sources"):
            sources = run(part.emit_sources, x)
        else:
            branch = self._branch(ws, ws.max_tokens, width)
            sources = [(*emit_on_branch(program, branch, lambda: run(part.emit, x)), 1.0)]
        scale.emit(program, sources)


@register_part("block", "prenorm_scaled")
class PreNormScaledBlock(_ScaledBlock):
    ROLES = {"mixer_norm": "norm", "mixer": "mixer", "mixer_scale": "branch_scale",
             "feed_forward_norm": "norm", "feed_forward": "feed_forward", "feed_forward_scale": "branch_scale"}

    def forward(self, ctx, stream, cache):
        self._sublayer(ctx, stream, self.mixer_norm, self.mixer, lambda f, x, *b: f(ctx, x, *b, cache), self.mixer_scale)
        self._sublayer(ctx, stream, self.feed_forward_norm, self.feed_forward, lambda f, x, *b: f(ctx, x, *b), self.feed_forward_scale)

    def emit(self, program, cache):
        self._emit_sublayer(program, self.mixer_norm, self.mixer, lambda f, x: f(program, x, cache), self.mixer_scale)
        self._emit_sublayer(program, self.feed_forward_norm, self.feed_forward, lambda f, x: f(program, x), self.feed_forward_scale)


@register_part("block", "prenorm_scaled_mixer")
class PreNormScaledMixerBlock(_ScaledBlock):
    """The first half alone: a layer without a feed-forward."""
    ROLES = {"mixer_norm": "norm", "mixer": "mixer", "mixer_scale": "branch_scale"}

    def forward(self, ctx, stream, cache):
        self._sublayer(ctx, stream, self.mixer_norm, self.mixer, lambda f, x, *b: f(ctx, x, *b, cache), self.mixer_scale)

    def emit(self, program, cache):
        self._emit_sublayer(program, self.mixer_norm, self.mixer, lambda f, x: f(program, x, cache), self.mixer_scale)
