"""The dense feed-forward: x += act(xn . W_fc^T + b_fc) . W_proj^T + b_proj
(reference: crates/core/src/stages/blocks.rs:113-137).  The reference fixes the inner width
at 4C (crates/core/src/weights.rs:95-98) and the activation at tanh-GELU
(crates/core/src/kernels/reference.rs:53-61); both are parameters here, and the exact
erf-GELU is offered beside the tanh form, the square of relu ("relu2": max(z, 0)^2), and xIELU, an
activation with two learned numbers p, q:
z > 0: softplus(p) z^2 + z / 2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2."""
from __future__ import annotations

from typing import List

import torch

from ..kernels import ops
from .base import MATRIX, TABLE, VECTOR, FeedForward, ParamSpec, StepContext, register_feed_forward


@register_feed_forward("dense_mlp")
class DenseMLP(FeedForward):
    takes_norm_input = True

    def __init__(self, width: int, inner: int, activation: str, bias: bool = True):
        if activation not in ("tanh", "erf", "relu2", "xielu"):
            raise ValueError(f"activation {activation!r} is not one of 'tanh', 'erf' (the two GELU forms), 'relu2', "
                             "'xielu'")
        self.width, self.inner, self.activation, self.bias = int(width), int(inner), activation, bool(bias)

    def param_specs(self) -> List[ParamSpec]:
        specs = [ParamSpec("fc_weight", (self.inner, self.width), MATRIX),
                 ParamSpec("proj_weight", (self.width, self.inner), MATRIX)]
        if self.bias:
            specs += [ParamSpec("fc_bias", (self.inner,), VECTOR), ParamSpec("proj_bias", (self.width,), VECTOR)]
        if self.activation == "xielu":
            specs.append(ParamSpec("act_params", (2,), VECTOR))
        return specs

    def reserve(self, workspace, limits) -> None:
        workspace.reserve("mlp.fc", limits.max_rows * self.inner, self.dtype)

    def forward(self, xn: torch.Tensor, x: torch.Tensor, ctx: StepContext) -> None:
        T, p = ctx.n_rows, self.params
        fc = ctx.workspace.get("mlp.fc", (ctx.max_rows, self.inner), self.dtype)
        xn, norm = (None, xn) if isinstance(xn, ops.NormInput) else (xn, None)
        ops.trace_scope(ctx.layer, "fc")
        if self.activation == "xielu":
            ops.linear(xn, p["fc_weight"], p.get("fc_bias"), fc, T, norm=norm)
            ops.unary(fc, fc, T, ops.UNARY_XIELU, p["act_params"])
        else:
            ops.linear(xn, p["fc_weight"], p.get("fc_bias"), fc, T, act=ops.ACT_CODES[self.activation], norm=norm)
        ops.trace_scope(ctx.layer, "fc_proj")
        ops.linear(fc, p["proj_weight"], p.get("proj_bias"), x, T, residual=True)


@register_feed_forward("gated_mlp")
class GatedMLP(FeedForward):
    """The gated dense feed-forward: x += W_down (act(W_gate h) * (W_up h)), without biases; ``activation`` is
    "silu" (z * sigmoid(z)) or one of the dense feed-forward's.  Gate and value rows are interleaved into one
    matrix at load ([2F, C]: row 2f the gate's, row 2f + 1 the value's), so that one product makes both as 32-bit
    floats; one kernel makes act(g) * u in 32-bit and casts; the second product adds into the stream."""

    def __init__(self, width: int, inner: int, activation: str = "silu"):
        if activation not in ("silu", "tanh", "erf", "relu2"):
            raise ValueError(f"gated_mlp: activation {activation!r} is not one of 'silu', 'tanh', 'erf', 'relu2'")
        if width <= 0 or inner <= 0:
            raise ValueError("gated_mlp: sizes must be positive")
        self.width, self.inner, self.activation = int(width), int(inner), activation

    def param_specs(self) -> List[ParamSpec]:
        return [ParamSpec("gate_weight", (self.inner, self.width), MATRIX),
                ParamSpec("up_weight", (self.inner, self.width), MATRIX),
                ParamSpec("down_weight", (self.width, self.inner), MATRIX)]

    def prepare(self, dtype, device) -> None:
        super().prepare(dtype, device)
        p = self.params
        w = torch.empty(self.inner, 2, self.width, dtype=p["gate_weight"].dtype, device=p["gate_weight"].device)
        w[:, 0], w[:, 1] = p["gate_weight"], p["up_weight"]
        p["gate_weight"], p["up_weight"] = w[:, 0], w[:, 1]
        self.w_in = w.view(2 * self.inner, self.width)

    def reserve(self, workspace, limits) -> None:
        workspace.reserve("gated_mlp.pre", limits.max_rows * 2 * self.inner, torch.float32)
        workspace.reserve("mlp.fc", limits.max_rows * self.inner, self.dtype)

    def forward(self, xn: torch.Tensor, x: torch.Tensor, ctx: StepContext) -> None:
        if isinstance(xn, ops.NormInput):
            xn = xn.materialise(ctx.n_rows)
        T, ws = ctx.n_rows, ctx.workspace
        pre = ws.get("gated_mlp.pre", (ctx.max_rows, 2 * self.inner), torch.float32)
        ops.trace_scope(ctx.layer, "fc")
        ops.linear(xn, self.w_in, None, pre, T)
        fc = ws.get("mlp.fc", (ctx.max_rows, self.inner), self.dtype)
        ops.glu(pre, fc, T, self.inner, ops.ACT_CODES[self.activation])
        ops.trace_scope(ctx.layer, "fc_proj")
        ops.linear(fc, self.params["down_weight"], None, x, T, residual=True)


@register_feed_forward("token_gated_input")
class TokenGatedInput(FeedForward):
    """What a row's own token adds late in a layer: a second embedding table holds ``dim`` values for every
    (token, layer); with e the slice [offset, offset + dim) of the token's row,
        y = W_proj (act(W_gate h) * e),
    added into the buffer it is given (the arrangement norms and sums it).  ``table`` may be one tensor shared by
    all layers, each reading its own slice.  act(W_gate h) is made in 32-bit."""

    def __init__(self, width: int, dim: int, table_width: int, offset: int, vocab_size: int, activation: str = "tanh"):
        if min(width, dim, vocab_size) <= 0 or offset < 0 or offset + dim > table_width:
            raise ValueError("token_gated_input: the slice [offset, offset + dim) must lie within the table's rows")
        if activation not in ("tanh", "erf", "silu", "relu2"):
            raise ValueError(f"token_gated_input: activation {activation!r} is not known")
        self.width, self.dim, self.table_width, self.offset = int(width), int(dim), int(table_width), int(offset)
        self.vocab_size, self.activation = int(vocab_size), activation

    def param_specs(self) -> List[ParamSpec]:
        return [ParamSpec("table", (self.vocab_size, self.table_width), TABLE),
                ParamSpec("gate_weight", (self.dim, self.width), MATRIX),
                ParamSpec("proj_weight", (self.width, self.dim), MATRIX)]

    def matrix_flops_per_row(self) -> float:
        return 4.0 * self.dim * self.width

    def reserve(self, workspace, limits) -> None:
        workspace.reserve("token_input.pre", limits.max_rows * self.dim, torch.float32)
        workspace.reserve("token_input.g", limits.max_rows * self.dim, self.dtype)

    def forward(self, xn: torch.Tensor, x: torch.Tensor, ctx: StepContext) -> None:
        if isinstance(xn, ops.NormInput):
            xn = xn.materialise(ctx.n_rows)
        T, ws, p = ctx.n_rows, ctx.workspace, self.params
        pre = ws.get("token_input.pre", (ctx.max_rows, self.dim), torch.float32)
        ops.trace_scope(ctx.layer, "token_gate")
        ops.linear(xn, p["gate_weight"], None, pre, T)
        g = ws.get("token_input.g", (ctx.max_rows, self.dim), self.dtype)
        ops.gate_by_table(pre, ctx.tokens, ctx.token_feedback, p["table"], self.offset, self.dim,
                          ops.ACT_CODES[self.activation], g, T)
        ops.trace_scope(ctx.layer, "token_proj")
        ops.linear(g, p["proj_weight"], None, x, T, residual=True)
