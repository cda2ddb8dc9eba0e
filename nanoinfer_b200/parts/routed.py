"""A routed feed-forward (mixture of experts): every row goes through ``top`` of ``n_expert`` small
two-layer experts without biases, chosen by a router whose logits and softmax are 32-bit.

z = W_router h, s = softmax(z) over ALL experts (``score`` "sigmoid": each logit's sigmoid instead), the ``top``
largest are chosen; their weights are the scores s themselves (``renorm`` divides them by their sum);
out = sum_e s_e W_down[e] act(W_up[e] h), plus, with ``shared_inner`` > 0, one expert of the same form
that every row goes through unweighted.  Routing happens on the device (csrc/moe.cu): nothing of it is
read by the host, so a step's launches depend on its shape only.

Variants, each a constructor argument: ``gated`` experts W_down (act(W_gate h) * (W_up h)) (one more matrix an
expert; gate and value rows are interleaved into one matrix at load, so that one product makes both);
``weight_on`` "input": the score multiplies what the expert READS, out = sum_e expert_e(s_e h), which for these
experts is not the same as scaling the output (the first product is linear, so the kernels scale its results
before the activation); ``shared_row_gate``: the shared expert's output times sigmoid(w_sg . h), one number a row
(its row rides in the shared expert's first product); ``choice_bias``: a learned number per expert that is added
to the scores for the CHOICE only (the weights stay the scores); ``n_identity`` > 0: the router has that many outputs
more than there are experts with matrices, and a row that chooses one of them gets its own input back, times the
score (the routing kernel adds it, the expert kernels skip the choice); activation "swiglu_capped" (gated experts):
g' = min(g, act_limit), u' = clamp(u, -act_limit, act_limit), g' sigmoid(1.702 g') (u' + 1).
"""
from __future__ import annotations

import itertools
from typing import List, Optional

import torch

from ..kernels import ops
from .base import MATRIX, VECTOR, FeedForward, ParamSpec, StepContext, register_feed_forward


_instances = itertools.count()


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    def __init__(self, width: int, n_expert: int, top: int, inner: int, activation: str = "erf",
                 renorm: bool = False, shared_inner: int = 0, shared_activation: str = "erf",
                 score: str = "softmax", gated: bool = False, weight_on: str = "output", shared_row_gate: bool = False,
                 choice_bias: bool = False, n_identity: int = 0, act_limit: float = 0.0):
        if n_identity < 0 or not 0 < top <= n_expert + n_identity:
            raise ValueError(f"routed_experts: top {top} must be between 1 and the number of experts {n_expert} "
                             f"(+ {n_identity} without matrices)")
        for a in (activation, shared_activation):
            if a not in (("tanh", "erf", "relu2", "silu", "swiglu_capped") if gated else ("tanh", "erf")):
                raise ValueError(f"routed_experts: activation {a!r} is not one of 'tanh', 'erf' (gated experts: "
                                 "also 'relu2', 'silu', 'swiglu_capped')")
        if activation == "swiglu_capped" and not act_limit > 0.0:
            raise ValueError("routed_experts: 'swiglu_capped' needs a positive act_limit")
        if shared_inner and shared_activation == "swiglu_capped":
            raise ValueError("routed_experts: the shared expert does not take 'swiglu_capped'")
        if n_identity and weight_on == "input":
            raise ValueError("routed_experts: experts without matrices go with weights on the output")
        if score not in ("softmax", "sigmoid") or weight_on not in ("input", "output"):
            raise ValueError("routed_experts: score is 'softmax' or 'sigmoid', weight_on 'input' or 'output'")
        if weight_on == "input" and not gated:
            raise ValueError("routed_experts: weight_on 'input' is built for gated experts")
        if shared_row_gate and not (gated and shared_inner):
            raise ValueError("routed_experts: shared_row_gate needs a gated shared expert")
        self.width, self.n_expert, self.top, self.inner = int(width), int(n_expert), int(top), int(inner)
        self.activation, self.renorm = activation, bool(renorm)
        self.shared_inner, self.shared_activation = int(shared_inner), shared_activation
        self.score, self.gated, self.weight_on = score, bool(gated), weight_on
        # every part keeps the experts it chose in a buffer of its own: after a step (replayed from a graph or not)
        # ``last_ids[:rows]`` says which experts each row of that step went to
        self._ids_name = f"moe.ids.{next(_instances)}"
        self.last_ids: Optional[torch.Tensor] = None
        self.shared_row_gate = bool(shared_row_gate)
        self.choice_bias, self.n_identity, self.act_limit = bool(choice_bias), int(n_identity), float(act_limit)
        #: outputs of the router: the experts with matrices, then those without
        self.n_routes = self.n_expert + self.n_identity

    def param_specs(self) -> List[ParamSpec]:
        specs = [ParamSpec("router", (self.n_routes, self.width), MATRIX)]
        if self.choice_bias:
            specs.append(ParamSpec("choice_bias", (self.n_routes,), VECTOR))
        for e in range(self.n_expert):
            if self.gated:
                specs.append(ParamSpec(f"expert{e}_gate", (self.inner, self.width), MATRIX))
            specs += [ParamSpec(f"expert{e}_up", (self.inner, self.width), MATRIX),
                      ParamSpec(f"expert{e}_down", (self.width, self.inner), MATRIX)]
        if self.shared_inner:
            if self.gated:
                specs.append(ParamSpec("shared_gate", (self.shared_inner, self.width), MATRIX))
            specs += [ParamSpec("shared_up", (self.shared_inner, self.width), MATRIX),
                      ParamSpec("shared_down", (self.width, self.shared_inner), MATRIX)]
            if self.shared_row_gate:
                specs.append(ParamSpec("shared_row_gate", (1, self.width), MATRIX))
        return specs

    def matrix_flops_per_row(self) -> float:
        n_mat = 3 if self.gated else 2
        per_expert = 2.0 * n_mat * self.inner * self.width
        return 2.0 * self.n_routes * self.width + self.top * per_expert + 2.0 * n_mat * self.shared_inner * self.width

    def prepare(self, dtype, device) -> None:
        super().prepare(dtype, device)
        p, E = self.params, self.n_expert
        # the experts' matrices stacked, [E, F, C] and [E, C, F]: a kernel finds expert e at a fixed stride, and
        # the first matrices of all experts are one matrix [E * F, C]; the parameters by name become views of
        # the stacks (no second copy stays behind)
        if self.gated:
            # gate and value rows interleaved, [E, 2F, C]: row 2f the gate's, row 2f + 1 the value's
            self.w_up = torch.stack([torch.stack([p[f"expert{e}_gate"], p[f"expert{e}_up"]], 1).reshape(
                2 * self.inner, self.width) for e in range(E)], 0).contiguous()
        else:
            self.w_up = torch.stack([p[f"expert{e}_up"] for e in range(E)], 0).contiguous()
        self.w_down = torch.stack([p[f"expert{e}_down"] for e in range(E)], 0).contiguous()
        for e in range(E):
            if self.gated:
                p[f"expert{e}_gate"], p[f"expert{e}_up"] = self.w_up[e, 0::2], self.w_up[e, 1::2]
            else:
                p[f"expert{e}_up"] = self.w_up[e]
            p[f"expert{e}_down"] = self.w_down[e]
        if self.shared_inner and self.gated:
            # the shared expert's first product: (gate, value) rows interleaved, then the row gate's row, zero rows
            # up to a multiple of 8; its result is 32-bit
            Fs = self.shared_inner
            self.shared_cols = -(-(2 * Fs + 1) // 8) * 8
            w = torch.zeros(self.shared_cols, self.width, dtype=self.w_up.dtype, device=self.w_up.device)
            w[0:2 * Fs:2], w[1:2 * Fs:2] = p["shared_gate"], p["shared_up"]
            p["shared_gate"], p["shared_up"] = w[0:2 * Fs:2], w[1:2 * Fs:2]
            if self.shared_row_gate:
                w[2 * Fs] = p["shared_row_gate"][0]
                p["shared_row_gate"] = w[2 * Fs:2 * Fs + 1]
            self.w_shared = w

    def reserve(self, workspace, limits) -> None:
        n = limits.max_rows
        workspace.reserve(self._ids_name, n * self.top, torch.int32)
        workspace.reserve("moe.weights", n * self.top, torch.float32)
        workspace.reserve("moe.inner", n * self.top * self.inner, self.dtype)
        workspace.reserve("moe.parts", n * self.top * self.width, torch.float32)
        if self.n_expert <= ops.MOE_DENSE_MAX_RATIO * self.top:
            workspace.reserve("moe.inner_all", n * self.n_expert * self.inner, self.dtype)
            if self.gated:
                workspace.reserve("moe.pre_all", n * self.n_expert * 2 * self.inner, torch.float32)
        if self.shared_inner:
            workspace.reserve("moe.shared", n * self.shared_inner, self.dtype)
            if self.gated:
                workspace.reserve("moe.shared_pre", n * self.shared_cols, torch.float32)

    def forward(self, xn: torch.Tensor, x: torch.Tensor, ctx: StepContext) -> None:
        if isinstance(xn, ops.NormInput):
            xn = xn.materialise(ctx.n_rows)
        T, p, ws, n = ctx.n_rows, self.params, ctx.workspace, ctx.max_rows
        ids = self.last_ids = ws.get(self._ids_name, (n, self.top), torch.int32)
        weights = ws.get("moe.weights", (n, self.top), torch.float32)
        ops.trace_scope(ctx.layer, "router")
        ops.moe_route(xn, p["router"], T, self.top, self.renorm, ids, weights, score=self.score,
                      choice_bias=p.get("choice_bias"), n_real=self.n_expert, x=x)
        inner = ws.get("moe.inner", (n * self.top, self.inner), self.dtype)
        ops.trace_scope(ctx.layer, "experts")
        ops.moe_experts(xn, self.w_up, self.w_down, ids, weights, inner, x, T, self.top,
                        ops.ACT_CODES[self.activation], ws, gated=self.gated, weight_on_input=self.weight_on == "input",
                        act_prm=self.act_limit)
        if self.shared_inner:
            hs = ws.get("moe.shared", (n, self.shared_inner), self.dtype)
            ops.trace_scope(ctx.layer, "shared_fc")
            if self.gated:
                pre = ws.get("moe.shared_pre", (n, self.shared_cols), torch.float32)
                ops.linear(xn, self.w_shared, None, pre, T)
                # (the row gate multiplies the expert's output; the second product is linear, so it may scale its input)
                ops.glu(pre, hs, T, self.shared_inner, ops.ACT_CODES[self.shared_activation],
                        2 * self.shared_inner if self.shared_row_gate else -1)
            else:
                ops.linear(xn, p["shared_up"], None, hs, T, act=ops.ACT_CODES[self.shared_activation])
            ops.trace_scope(ctx.layer, "shared_proj")
            ops.linear(hs, p["shared_down"], None, x, T, residual=True)
