"""Recurrent mixers with a matrix state per head and ONE decay per head and token: the gated delta rule and the
state-space recurrence of Mamba-2 (state-space duality).  Both put a short causal convolution over time ahead of the
recurrence and a gated RMS norm behind it, and both run on the same kernels (``csrc/gated_scan.cu``).

Per head, with S an N x V matrix that starts at zero, a decay a_t in (0, 1] and a strength w_t:
    gated delta rule:   S <- a S;   u = w (v - S^T k);   S <- S + k u^T;   o = S^T q
    state space:        S <- a S + w k v^T;              o = S^T q + D v
(the read-out sees the current token's write).  What a request keeps between steps, in its state slot, 32-bit: the
convolution's last ``taps - 1`` inputs and the matrices.  Decays, strengths, unit vectors, the recurrence and the
norm behind it are computed in 32-bit whatever the engine's dtype: the projection that reads the mixer's input
leaves its product as 32-bit floats.  The work on the device is shaped by the step's shape alone, so steps are
captured in graphs like those of a mixer without state.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..kernels import ops
from .base import (INIT_ONE_PLUS_NORMAL, MATRIX, VECTOR, KVCacheView, Mixer, ParamSpec, StateSpec, StepContext,
                   StepLimits, Workspace, register_mixer)


def _round_up(n: int, m: int) -> int:
    return -(-n // m) * m


class _ScanMixer(Mixer):
    """What the two recurrences share: scratch, the state's layout, the run order of the kernels."""

    capture_safe = True
    #: set by the subclass: rows of the fused projection, channels of the convolution, its first column in the
    #: projection's output, key size N, value size V, heads, query/key heads (or groups)
    n_proj = channels = conv_off = n_key = n_val = n_head = n_kq = taps = 0

    def _state_layout(self) -> None:
        if ops._scan_padded_host(self.n_key) == 0:
            raise ValueError(f"{type(self).__name__}: a key size of {self.n_key} is not supported (at most 256: a "
                             "column of the state lives in the registers of four threads)")
        #: floats from the start of a request's row to its matrices (the convolution's inputs come first)
        self.s_off = _round_up(max(self.taps - 1, 0) * self.channels, 4)
        self.state_floats = ops.gated_scan_state_floats(self.taps, self.channels, self.n_head, self.n_key, self.n_val)
        self.cv_width = _round_up(self.channels, 4)

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((self.state_floats,), torch.float32)

    def reserve(self, workspace: Workspace, limits: StepLimits) -> None:
        n = limits.max_rows
        workspace.reserve("scan.proj", n * self.n_proj, torch.float32)
        workspace.reserve("scan.cv", n * self.cv_width, torch.float32)
        workspace.reserve("scan.coef", n * self.n_head * 2, torch.float32)
        workspace.reserve("scan.o", n * self.n_head * self.n_val, torch.float32)
        workspace.reserve("scan.out", n * self.n_head * self.n_val, self.dtype)

    def _fuse(self, keys, offsets) -> torch.Tensor:
        """The products that read the mixer's input become one; the parameters by name become views of it."""
        p = self.params
        first = p[keys[0]]
        w = torch.zeros(self.n_proj, self.width, dtype=first.dtype, device=first.device)
        for key, at in zip(keys, offsets):
            n = p[key].shape[0]
            w[at:at + n] = p[key]
            p[key] = w[at:at + n]
        return w

    def _buffers(self, ctx: StepContext):
        ws, n = ctx.workspace, ctx.max_rows
        return (ws.get("scan.proj", (n, self.n_proj), torch.float32),
                ws.get("scan.cv", (n, self.cv_width), torch.float32),
                ws.get("scan.coef", (n, self.n_head, 2), torch.float32),
                ws.get("scan.o", (n, self.n_head * self.n_val), torch.float32),
                ws.get("scan.out", (n, self.n_head * self.n_val), self.dtype))


@register_mixer("gated_delta")
class GatedDeltaRule(_ScanMixer):
    """The gated delta rule.  q = W_q h and k = W_k h (``n_kq_head`` heads of ``head_dim``), v = W_v h (``n_head``
    heads of ``v_dim``; head h reads query/key head h // (n_head / n_kq_head)); each passes a causal convolution
    over time per channel (``taps`` taps, the last the current token's, zeros before the start, no bias) and SiLU;
    q and k are then made unit vectors per head, x / sqrt(sum x^2 + 1e-6), q also times head_dim^(-1/2).
    beta = sigmoid(W_b h) and the decay a = exp(-exp(A_log) softplus(W_a h + dt_bias)), one per head.  After the
    recurrence each head's o is divided by its root mean square over ``v_dim``, multiplied by a weight of ``v_dim``
    values that the heads share and by silu(W_g h); then W_o."""

    def __init__(self, width: int, n_head: int, n_kq_head: int, head_dim: int, v_dim: int, taps: int, eps: float,
                 out_scale: float = 1.0):
        if min(width, n_head, n_kq_head, head_dim, v_dim, taps) <= 0 or n_head % n_kq_head:
            raise ValueError("gated_delta: sizes must be positive, n_head a multiple of n_kq_head")
        self.width, self.n_head, self.n_kq, self.n_key, self.n_val = int(width), int(n_head), int(n_kq_head), \
            int(head_dim), int(v_dim)
        self.taps, self.eps, self.out_scale = int(taps), float(eps), float(out_scale)
        self.n_qk, self.n_v = self.n_kq * self.n_key, self.n_head * self.n_val
        self.channels, self.conv_off = 2 * self.n_qk + self.n_v, 0
        #: columns of the fused projection's output: q | k | v | g | b | a, a multiple of 8 wide
        self.offsets = (0, self.n_qk, 2 * self.n_qk, 2 * self.n_qk + self.n_v, 2 * self.n_qk + 2 * self.n_v,
                        2 * self.n_qk + 2 * self.n_v + self.n_head)
        self.n_proj = _round_up(self.offsets[5] + self.n_head, 8)
        self._state_layout()

    def param_specs(self) -> List[ParamSpec]:
        c, t = self.width, self.taps
        return [ParamSpec("q_weight", (self.n_qk, c), MATRIX), ParamSpec("k_weight", (self.n_qk, c), MATRIX),
                ParamSpec("v_weight", (self.n_v, c), MATRIX), ParamSpec("g_weight", (self.n_v, c), MATRIX),
                ParamSpec("b_weight", (self.n_head, c), MATRIX), ParamSpec("a_weight", (self.n_head, c), MATRIX),
                ParamSpec("q_conv", (self.n_qk, t), VECTOR), ParamSpec("k_conv", (self.n_qk, t), VECTOR),
                ParamSpec("v_conv", (self.n_v, t), VECTOR),
                ParamSpec("A_log", (self.n_head,), VECTOR), ParamSpec("dt_bias", (self.n_head,), VECTOR),
                ParamSpec("out_norm", (self.n_val,), VECTOR, INIT_ONE_PLUS_NORMAL),
                ParamSpec("out_weight", (c, self.n_v), MATRIX)]

    def prepare(self, dtype, device) -> None:
        super().prepare(dtype, device)
        p = self.params
        self.w_in = self._fuse(("q_weight", "k_weight", "v_weight", "g_weight", "b_weight", "a_weight"), self.offsets)
        self.conv_w = torch.cat([p["q_conv"], p["k_conv"], p["v_conv"]], 0).contiguous()

    def forward(self, xn: torch.Tensor, x: torch.Tensor, ctx: StepContext, cache: Optional[KVCacheView],
                state: Optional[torch.Tensor], writes_cache: bool = True) -> None:
        if state is None:
            raise ValueError("gated_delta needs a state slot tensor")
        if isinstance(xn, ops.NormInput):
            xn = xn.materialise(ctx.n_rows)
        T, p = ctx.n_rows, self.params
        proj, cv, coef, o, out = self._buffers(ctx)
        ops.trace_scope(ctx.layer, "scan_in")
        ops.linear(xn, self.w_in, None, proj, T)
        ops.short_conv(proj, 0, self.channels, self.taps, self.conv_w, None, state, ctx, cv, ops.ACT_SILU)
        ops.scan_prepare(proj, self.offsets[5], self.offsets[4], p["A_log"], p["dt_bias"], cv, 0, self.n_qk, self.n_key,
                         self.n_head, self.n_kq, True, coef, T)
        ops.gated_scan(True, cv, 0, self.n_qk, 2 * self.n_qk, self.n_key, self.n_val, self.n_head,
                       self.n_head // self.n_kq, coef, None, state, self.s_off, ctx, o)
        ops.gated_norm(o, proj[:, self.offsets[3]:self.offsets[3] + self.n_v], p["out_norm"], self.n_head, self.n_val,
                       self.eps, False, self.out_scale, out, T)
        ops.trace_scope(ctx.layer, "scan_proj")
        ops.linear(out, p["out_weight"], None, x, T, residual=True)


@register_mixer("state_space")
class StateSpaceDuality(_ScanMixer):
    """Mamba-2.  With inner = n_head * v_dim, N = ``state`` and G = ``groups``, W_in h is laid out
    [z: inner | x: inner | B: G N | C: G N | dt: n_head]; x, B and C together pass a causal convolution over time per
    channel (``taps`` taps, the last the current token's, zeros before the start, a bias) and SiLU;
    dt <- softplus(dt + dt_bias) (no clamp); per head (head h reads group h // (n_head / G)):
        S <- exp(-exp(A_log) dt) S + dt B x^T;   y = S^T C + D x.
    Then y (heads concatenated) times silu(z), an RMS norm in ``norm_groups`` equal parts of the row (each by its own
    root mean square), times a weight of inner values; then W_o."""

    def __init__(self, width: int, n_head: int, v_dim: int, state: int, groups: int, norm_groups: int, taps: int,
                 eps: float, out_scale: float = 1.0):
        if min(width, n_head, v_dim, state, groups, norm_groups, taps) <= 0 or n_head % groups \
                or (n_head * v_dim) % norm_groups:
            raise ValueError("state_space: sizes must be positive, n_head a multiple of groups, the inner width a "
                             "multiple of norm_groups")
        self.width, self.n_head, self.n_val, self.n_key, self.n_kq = int(width), int(n_head), int(v_dim), int(state), \
            int(groups)
        self.norm_groups, self.taps, self.eps, self.out_scale = int(norm_groups), int(taps), float(eps), float(out_scale)
        self.inner, self.n_bc = self.n_head * self.n_val, self.n_kq * self.n_key
        self.channels, self.conv_off = self.inner + 2 * self.n_bc, self.inner
        self.n_in = 2 * self.inner + 2 * self.n_bc + self.n_head
        self.n_proj = _round_up(self.n_in, 8)
        self._state_layout()

    def param_specs(self) -> List[ParamSpec]:
        c = self.width
        return [ParamSpec("in_weight", (self.n_in, c), MATRIX),
                ParamSpec("conv_weight", (self.channels, self.taps), VECTOR),
                ParamSpec("conv_bias", (self.channels,), VECTOR),
                ParamSpec("dt_bias", (self.n_head,), VECTOR), ParamSpec("A_log", (self.n_head,), VECTOR),
                ParamSpec("D", (self.n_head,), VECTOR, INIT_ONE_PLUS_NORMAL),
                ParamSpec("out_norm", (self.inner,), VECTOR, INIT_ONE_PLUS_NORMAL),
                ParamSpec("out_weight", (c, self.inner), MATRIX)]

    def prepare(self, dtype, device) -> None:
        super().prepare(dtype, device)
        self.w_in = self._fuse(("in_weight",), (0,))

    def forward(self, xn: torch.Tensor, x: torch.Tensor, ctx: StepContext, cache: Optional[KVCacheView],
                state: Optional[torch.Tensor], writes_cache: bool = True) -> None:
        if state is None:
            raise ValueError("state_space needs a state slot tensor")
        if isinstance(xn, ops.NormInput):
            xn = xn.materialise(ctx.n_rows)
        T, p = ctx.n_rows, self.params
        proj, cv, coef, o, out = self._buffers(ctx)
        ops.trace_scope(ctx.layer, "scan_in")
        ops.linear(xn, self.w_in, None, proj, T)
        ops.short_conv(proj, self.inner, self.channels, self.taps, p["conv_weight"], p["conv_bias"], state, ctx, cv,
                       ops.ACT_SILU)
        dt_off = 2 * self.inner + 2 * self.n_bc
        ops.scan_prepare(proj, dt_off, dt_off, p["A_log"], p["dt_bias"], cv, 0, 0, self.n_key, self.n_head, self.n_kq,
                         False, coef, T)
        # cv: x | B | C;  the recurrence's k is B, its q is C, its v is x
        ops.gated_scan(False, cv, self.inner + self.n_bc, self.inner, 0, self.n_key, self.n_val, self.n_head,
                       self.n_head // self.n_kq, coef, p["D"], state, self.s_off, ctx, o)
        ops.gated_norm(o, proj[:, :self.inner], p["out_norm"], self.norm_groups, self.inner // self.norm_groups,
                       self.eps, True, self.out_scale, out, T)
        ops.trace_scope(ctx.layer, "scan_proj")
        ops.linear(out, p["out_weight"], None, x, T, residual=True)


@register_mixer("parallel")
class ParallelMixers(Mixer):
    """Two mixers side by side that read the same input.  The result is left_scale * left + right_scale * right or,
    with ``out_norm_eps`` given, left_scale * norm(left) + right_scale * norm(right), each an RMS norm over the model
    width with a weight of its own (``left.out_norm``, ``right.out_norm``).
    ``left`` and ``right`` are {"kind": registered name, "args": constructor arguments}; both kinds must take an
    ``out_scale`` argument (without the norms the scale is applied inside each, ahead of its output projection, whose
    epilogue then adds into the same buffer; with them each adds into a 32-bit buffer of its own that it finds zero,
    and one kernel per side norms it, scales it, adds it to the result and zeroes it again).  At most one of the two
    may want paged keys and values: the cache manager gives a run of a layer one set of pages.  Both may keep
    per-request state: the layer's state row is the two side by side, each a multiple of four floats.  Parameters are
    named ``left.<key>`` and ``right.<key>``."""

    def __init__(self, width: int, left: dict, right: dict, left_scale: float = 1.0, right_scale: float = 1.0,
                 out_norm_eps: Optional[float] = None):
        from .base import MIXERS

        self.width = int(width)
        self.left_scale, self.right_scale = float(left_scale), float(right_scale)
        self.out_norm_eps = None if out_norm_eps is None else float(out_norm_eps)
        inner = (1.0, 1.0) if self.out_norm_eps is not None else (self.left_scale, self.right_scale)
        self.children = {
            "left": MIXERS.build(left["kind"], **{**left["args"], "out_scale": inner[0]}),
            "right": MIXERS.build(right["kind"], **{**right["args"], "out_scale": inner[1]}),
        }
        if sum(c.kv_spec() is not None for c in self.children.values()) > 1:
            raise ValueError("parallel: at most one of the two mixers may want a paged cache")
        #: where each side's state lies in the layer's state row: side -> (first float, floats)
        self.state_at, at = {}, 0
        for side, c in self.children.items():
            spec = c.state_spec()
            if spec is not None:
                if len(spec.shape) != 1 or spec.dtype != torch.float32:
                    raise ValueError("parallel: a side's state must be one row of 32-bit floats")
                self.state_at[side] = (at, int(spec.shape[0]))
                at += _round_up(int(spec.shape[0]), 4)
        self.state_floats = at

    def param_specs(self) -> List[ParamSpec]:
        specs = [ParamSpec(f"{side}.{s.key}", s.shape, s.kind, s.init) for side, c in self.children.items()
                 for s in c.param_specs()]
        if self.out_norm_eps is not None:
            specs += [ParamSpec(f"{side}.out_norm", (self.width,), VECTOR, INIT_ONE_PLUS_NORMAL) for side in self.children]
        return specs

    def bind(self, params) -> None:
        self.params = params
        for side, c in self.children.items():
            c.bind({k[len(side) + 1:]: v for k, v in params.items() if k.startswith(side + ".") and
                    not (self.out_norm_eps is not None and k == side + ".out_norm")})

    def prepare(self, dtype, device) -> None:
        super().prepare(dtype, device)
        for c in self.children.values():
            c.prepare(dtype, device)
        if self.out_norm_eps is not None:
            # (the side's share of the sum rides in its norm's weight)
            self.norm_w = {side: (self.params[f"{side}.out_norm"] * scale).contiguous()
                           for side, scale in (("left", self.left_scale), ("right", self.right_scale))}

    def reserve(self, workspace: Workspace, limits: StepLimits) -> None:
        for c in self.children.values():
            c.reserve(workspace, limits)
        if self.out_norm_eps is not None:
            for side in self.children:
                workspace.reserve(f"parallel.{side}", limits.max_rows * self.width, torch.float32, zeroed=True)

    def kv_spec(self):
        return next((c.kv_spec() for c in self.children.values() if c.kv_spec() is not None), None)

    def state_spec(self):
        return StateSpec((self.state_floats,), torch.float32) if self.state_floats else None

    def step_planner(self):
        return next((c.step_planner() for c in self.children.values() if c.step_planner() is not None), None)

    def flops_per_key(self) -> float:
        return sum(c.flops_per_key() for c in self.children.values())

    def matrix_flops_per_row(self) -> float:
        return sum(c.matrix_flops_per_row() for c in self.children.values())

    @property
    def capture_safe(self) -> bool:
        return all(c.capture_safe for c in self.children.values())

    def forward(self, xn: torch.Tensor, x: torch.Tensor, ctx: StepContext, cache: Optional[KVCacheView],
                state: Optional[torch.Tensor], writes_cache: bool = True) -> None:
        if isinstance(xn, ops.NormInput):
            xn = xn.materialise(ctx.n_rows)
        for side, c in self.children.items():
            own = None
            if side in self.state_at:
                at, n = self.state_at[side]
                own = state[:, at:at + n]
            into = x
            if self.out_norm_eps is not None:
                # zero when first handed out, and zeroed again by the kernel that reads it
                into = ctx.workspace.get_zeroed(f"parallel.{side}", (ctx.max_rows, self.width), torch.float32)
            c.forward(xn, into, ctx, cache if c.kv_spec() is not None else None, own, writes_cache)
            if self.out_norm_eps is not None:
                ops.add_norm(x, into, self.norm_w[side], self.out_norm_eps, ctx.n_rows)
