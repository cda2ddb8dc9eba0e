"""Mamba's selective scan as a mixer: a state [inner, state] per request whose decay, input and read-out depend on
the token.

W_in h is laid out [x: inner | z: inner].  x passes a causal convolution over time per channel (``taps`` taps, the
last the current token's, zeros before the start, a bias) and SiLU.  W_x x is laid out [dt: dt_rank | B: state |
C: state]; dt <- softplus(W_dt dt + dt_bias), one step size per channel; A = -exp(A_log) [inner, state].  Per channel
c and state index n:   S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n;   y_c = sum_n S[c, n] C_n + D_c x_c.
Then y * silu(z), and W_o.

What a request keeps between steps, in its state slot, 32-bit: the convolution's last ``taps - 1`` inputs and S.
Step sizes, decays, the recurrence and the gate are computed in 32-bit whatever the engine's dtype: the products that
feed them leave 32-bit results.  W_x is cut in two at load: its first dt_rank rows (their product is the next
product's input, in the engine's dtype, padded with zero rows to a multiple of 8) and the rows of B and C.  The
device's work is shaped by the step's shape alone, so steps are captured in graphs.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..kernels import ops
from .base import (INIT_ONE_PLUS_NORMAL, MATRIX, VECTOR, KVCacheView, Mixer, ParamSpec, StateSpec, StepContext,
                   StepLimits, Workspace, register_mixer)


def _round_up(n: int, m: int) -> int:
    return -(-n // m) * m


@register_mixer("selective_scan")
class SelectiveScan(Mixer):
    capture_safe = True

    def __init__(self, width: int, inner: int, state: int, dt_rank: int, taps: int, out_scale: float = 1.0):
        if min(width, inner, state, dt_rank, taps) <= 0:
            raise ValueError("selective_scan: sizes must be positive")
        if ops.selective_scan_padded(state) == 0:
            raise ValueError(f"selective_scan: a state of {state} values per channel is not supported (at most 256)")
        self.width, self.inner, self.n_state, self.dt_rank, self.taps = int(width), int(inner), int(state), \
            int(dt_rank), int(taps)
        self.out_scale = float(out_scale)
        self.rank_pad = _round_up(self.dt_rank, 8)
        self.bc_cols = _round_up(2 * self.n_state, 8)
        #: floats from the start of a request's row to S (the convolution's inputs come first)
        self.s_off = _round_up((self.taps - 1) * self.inner, 4)
        self.state_floats = self.s_off + self.inner * ops.selective_scan_padded(self.n_state)

    def param_specs(self) -> List[ParamSpec]:
        c, n, r = self.width, self.n_state, self.dt_rank
        return [ParamSpec("in_weight", (2 * self.inner, c), MATRIX),
                ParamSpec("conv_weight", (self.inner, self.taps), VECTOR), ParamSpec("conv_bias", (self.inner,), VECTOR),
                ParamSpec("x_weight", (r + 2 * n, self.inner), MATRIX), ParamSpec("dt_weight", (self.inner, r), MATRIX),
                ParamSpec("dt_bias", (self.inner,), VECTOR), ParamSpec("A_log", (self.inner, n), VECTOR),
                ParamSpec("D", (self.inner,), VECTOR, INIT_ONE_PLUS_NORMAL),
                ParamSpec("out_weight", (c, self.inner), MATRIX)]

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((self.state_floats,), torch.float32)

    def prepare(self, dtype, device) -> None:
        super().prepare(dtype, device)
        p, r, n = self.params, self.dt_rank, self.n_state
        wx = p["x_weight"]
        # the step sizes' rows, zero rows up to a multiple of 8, then B's and C's rows: the parameter becomes two views
        self.w_x = torch.zeros(self.rank_pad + self.bc_cols, self.inner, dtype=wx.dtype, device=wx.device)
        self.w_x[:r] = wx[:r]
        self.w_x[self.rank_pad:self.rank_pad + 2 * n] = wx[r:]
        self.w_dt = torch.zeros(self.inner, self.rank_pad, dtype=wx.dtype, device=wx.device)
        self.w_dt[:, :r] = p["dt_weight"]
        p["dt_weight"] = self.w_dt[:, :r]
        del p["x_weight"]
        self.A_log = p["A_log"].contiguous()
        self.w_out = p["out_weight"] * self.out_scale if self.out_scale != 1.0 else p["out_weight"]

    def reserve(self, workspace: Workspace, limits: StepLimits) -> None:
        n = limits.max_rows
        workspace.reserve("ssm.proj", n * 2 * self.inner, torch.float32)
        workspace.reserve("ssm.x", n * self.inner, torch.float32)
        workspace.reserve("ssm.x16", n * self.inner, torch.bfloat16)
        workspace.reserve("ssm.dt_low", n * self.rank_pad, self.dtype)
        workspace.reserve("ssm.bc", n * self.bc_cols, torch.float32)
        workspace.reserve("ssm.dt", n * self.inner, torch.float32)
        workspace.reserve("ssm.out", n * self.inner, self.dtype)

    def forward(self, xn: torch.Tensor, x: torch.Tensor, ctx: StepContext, cache: Optional[KVCacheView],
                state: Optional[torch.Tensor], writes_cache: bool = True) -> None:
        if state is None:
            raise ValueError("selective_scan needs a state slot tensor")
        if isinstance(xn, ops.NormInput):
            xn = xn.materialise(ctx.n_rows)
        T, p, ws, n = ctx.n_rows, self.params, ctx.workspace, ctx.max_rows
        proj = ws.get("ssm.proj", (n, 2 * self.inner), torch.float32)
        xc = ws.get("ssm.x", (n, self.inner), torch.float32)
        half = self.dtype == torch.bfloat16
        x16 = ws.get("ssm.x16", (n, self.inner), torch.bfloat16) if half else None
        dt_low = ws.get("ssm.dt_low", (n, self.rank_pad), self.dtype)
        bc = ws.get("ssm.bc", (n, self.bc_cols), torch.float32)
        dtp = ws.get("ssm.dt", (n, self.inner), torch.float32)
        out = ws.get("ssm.out", (n, self.inner), self.dtype)
        ops.trace_scope(ctx.layer, "scan_in")
        ops.linear(xn, p["in_weight"], None, proj, T)
        ops.short_conv(proj, 0, self.inner, self.taps, p["conv_weight"], p["conv_bias"], state, ctx, xc, ops.ACT_SILU,
                       out16=x16)
        xin = x16 if half else xc
        ops.trace_scope(ctx.layer, "scan_x")
        ops.linear(xin, self.w_x[:self.rank_pad], None, dt_low, T)
        ops.linear(xin, self.w_x[self.rank_pad:], None, bc, T)
        ops.trace_scope(ctx.layer, "scan_dt")
        ops.linear(dt_low, self.w_dt, p["dt_bias"], dtp, T)
        ops.selective_scan(dtp, xc, bc, 0, self.n_state, proj[:, self.inner:], self.A_log, p["D"], state, self.s_off,
                           ctx, self.inner, self.n_state, out)
        ops.trace_scope(ctx.layer, "scan_proj")
        ops.linear(out, self.w_out, None, x, T, residual=True)
