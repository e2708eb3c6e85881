"""Feed-forwards that are no plain gated product.

"polynorm": W_down act(W_up x) with act(z) = a N(z) + b N(z^2) + c N(z^3) + e, powers element by element, N(y) =
y / sqrt(mean(y^2) + eps) over a token's row, and a, b, c, e four stored numbers.

"routed": `experts` small feed-forwards W_down relu(W_up x)^2 of which every token uses `top`, plus `identity` experts
without weights whose output is their input. Router logits z = W_r x in true float32; scores s = softmax(z) over all
experts; the `top` experts with the largest s + correction are chosen; a chosen expert weighs s / (sum of the chosen
s + 1e-20) * scale. The experts' up matrices lie side by side as one matrix, so do the down matrices: the hidden
activations of experts that a token did not choose are exact zeros (times weight 0), so one product each way is the
weighted sum of the chosen experts; identity experts add their weight times x. Kernels between the products:
csrc/feed_forward.cu; the identity experts' share: csrc/branch.cu.

Two parameters make other routed designs of it. `weights_from` "logits": the stored vector is the router's bias, z = W_r x + b, the
`top` largest z are chosen and weigh by the softmax over the chosen z alone. `expert` "silu_gated": an expert is
W_down (silu(W_gate x) * (W_up x)); its gate and up matrices lie one above the other in the side-by-side product."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..kernels.linear import Linear
from .base import FeedForward, register_part
from .spec import TensorPlan


@register_part("feed_forward", "polynorm")
class PolyNormFeedForward(FeedForward):
    """params: hidden_size, intermediate_size, eps. tensors: up, down, coefficients [4]."""
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden, self.intermediate = int(spec.params["hidden_size"]), int(spec.params["intermediate_size"])
        self.eps = float(spec.params["eps"])
        self.up = self.down = None
        self.coefficients = (0.0, 0.0, 0.0, 0.0)

    def tensor_plan(self):
        t = self.spec.tensors
        return {t["up"]: TensorPlan((self.intermediate, self.hidden)), t["down"]: TensorPlan((self.hidden, self.intermediate)),
                t["coefficients"]: TensorPlan((4,))}

    def bind(self, tensors):
        t = self.spec.tensors
        self.up = Linear(tensors[t["up"]], self.env.compute_dtype)
        self.down = Linear(tensors[t["down"]], self.env.compute_dtype)
        self.coefficients = tuple(float(v) for v in tensors[t["coefficients"]].to(torch.float32).cpu().tolist())

    def weight_bytes(self):
        return self.up.weight_bytes() + self.down.weight_bytes()

    def kernel_libraries(self):
        return {"feed_forward", "gemm_tc" if self.env.compute_dtype == torch.bfloat16 else "gemm_f32"}

    def forward(self, ctx, x, stream):
        n, ws = ctx.n, ctx.workspace
        up = self.up.forward_partials(x, ws.raw("polynorm.up", (self.up.partial_elems(ws.max_tokens),), torch.float32))
        z = ws.get("polynorm.z", n, (self.intermediate,), ctx.act_dtype)
        ops.polynorm(up, z, self.coefficients, self.eps)
        self.down.forward_add(z, stream, ws.raw("polynorm.down_partials", (self.down.partial_elems(ws.max_tokens),), torch.float32))

    def emit(self, program, x):
        ws = program.workspace
        T = ws.max_tokens
        up = ws.raw("polynorm.up", (self.up.partial_elems(T),), torch.float32)
        S = self.up.emit_partials(program, x, up)
        z = ws.get("polynorm.z", T, (self.intermediate,), self.env.act_dtype)
        eps_bits = int(torch.tensor(self.eps, dtype=torch.float32).view(torch.int32).item())
        program.add("feed_forward", "sb_op_polynorm", [up, S, program.few_tokens, z, z.dtype, self.intermediate, eps_bits], self.coefficients)
        self.down.emit_add(program, z, ws.raw("polynorm.down_partials", (self.down.partial_elems(T),), torch.float32))


@register_part("feed_forward", "routed")
class RoutedFeedForward(FeedForward):
    """params: hidden_size, intermediate_size (of one expert), experts, identity (experts without weights, listed last by the
    router), top, scale (1 by default), weights_from ("scores" by default, or "logits"), expert ("relu2" by default, or "silu_gated").
    tensors: router [experts + identity, hidden], correction [experts + identity], up and down (lists of names, one per expert), gate
    (the same, for gated experts)."""
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden, self.intermediate = int(p["hidden_size"]), int(p["intermediate_size"])
        self.experts, self.identity, self.top = int(p["experts"]), int(p.get("identity", 0)), int(p["top"])
        self.scale = float(p.get("scale", 1.0))
        self.biased = {"scores": False, "logits": True}[p.get("weights_from", "scores")]
        self.gated = {"relu2": False, "silu_gated": True}[p.get("expert", "relu2")]
        self.outputs = self.experts + self.identity
        if not 0 < self.top <= self.outputs or self.outputs > 256:
            raise ValueError(f"routed feed-forward: {self.top} of {self.outputs} experts (at most 256)")
        self.router = self.correction = self.up = self.down = None

    def tensor_plan(self):
        t = self.spec.tensors
        plan = {t["router"]: TensorPlan((self.outputs, self.hidden)), t["correction"]: TensorPlan((self.outputs,), zero_mean=True)}
        for name in (*t["up"], *(t["gate"] if self.gated else ())):
            plan[name] = TensorPlan((self.intermediate, self.hidden))
        for name in t["down"]:
            plan[name] = TensorPlan((self.hidden, self.intermediate))
        return plan

    def bind(self, tensors):
        t = self.spec.tensors

        def side_by_side(names, dim):
            ws = [tensors[n] for n in names]
            if len({w.dtype for w in ws}) > 1:
                ws = [w.to(torch.float32) for w in ws]
            return torch.cat(ws, dim=dim)

        self.router = tensors[t["router"]].contiguous()
        self.correction = tensors[t["correction"]].to(torch.float32).contiguous()
        if self.experts:
            rows = t["up"] if not self.gated else [name for pair in zip(t["gate"], t["up"]) for name in pair]
            self.up = Linear(side_by_side(rows, 0), self.env.compute_dtype)
            self.down = Linear(side_by_side(t["down"], 1), self.env.compute_dtype)

    def weight_bytes(self):
        own = self.router.numel() * self.router.element_size()
        return own + (self.up.weight_bytes() + self.down.weight_bytes() if self.experts else 0)

    def kernel_libraries(self):
        return {"feed_forward", "branch", "gemm_f32", "gemm_tc" if self.env.compute_dtype == torch.bfloat16 else "gemm_f32"}

    def forward(self, ctx, x, stream):
        n, ws, E, F = ctx.n, ctx.workspace, self.experts, self.intermediate
        logits = ws.get("routed.logits", n, (self.outputs,), torch.float32)
        ops.gemm_f32(x, self.router, logits)
        weights = ws.get("routed.weights", n, (self.outputs,), torch.float32)
        ops.moe_route(logits, self.correction, weights, self.top, self.scale, self.biased)
        if self.identity:
            stream.fold()
            ops.row_scaled_add(stream.h, x, weights, E, self.identity)
        if E:
            up = self.up.forward_partials(x, ws.raw("routed.up", (self.up.partial_elems(ws.max_tokens),), torch.float32))
            z = ws.get("routed.z", n, (E * F,), ctx.act_dtype)
            ops.moe_activate(up, weights, z, E, F, self.gated)
            self.down.forward_add(z, stream, ws.raw("routed.down_partials", (self.down.partial_elems(ws.max_tokens),), torch.float32))

    def emit(self, program, x):
        ws, E, F, X = program.workspace, self.experts, self.intermediate, self.outputs
        T, f32 = ws.max_tokens, torch.float32
        logits = ws.get("routed.logits", T, (X,), f32)
        program.add("gemm_f32", "sb_op_linear_f32", [x, x.dtype, x.stride(0), self.router, self.router.dtype, self.router.stride(0), logits, X, X,
                                                     self.hidden, 0, 0])
        weights = ws.get("routed.weights", T, (X,), f32)
        program.add("feed_forward", "sb_op_moe_route", [logits, X, self.correction, self.correction.dtype, weights, X, self.top, int(self.biased)],
                    [self.scale])
        if self.identity:
            program.need_folded("identity experts")
            program.add("branch", "sb_op_row_scaled_add", [program.h, x, x.dtype, weights, X, E, self.identity, self.hidden])
        if E:
            up = ws.raw("routed.up", (self.up.partial_elems(T),), f32)
            S = self.up.emit_partials(program, x, up)
            z = ws.get("routed.z", T, (E * F,), self.env.act_dtype)
            program.add("feed_forward", "sb_op_moe_activate", [up, S, program.few_tokens, weights, X, z, z.dtype, E, F, int(self.gated)])
            self.down.emit_add(program, z, ws.raw("routed.down_partials", (self.down.partial_elems(T),), f32))
