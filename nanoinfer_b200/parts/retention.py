"""Retention: linear attention with ONE fixed decay per head and neither softmax nor denominator.

q = W_q h and k = W_k h (``n_head`` heads of ``head_dim``), v = W_v h (``n_head`` heads of ``v_dim``), no biases;
rotary positions in the halves layout on the first ``rot_dims`` values of every query and key head; k times
head_dim^(-1/2) after the rotation.  Per head, with S a head_dim x v_dim matrix that starts at zero:
    S <- decay_h S + k v^T;    o = S^T q
(the read-out sees the current token's write).  Each head's o is divided by its root mean square over ``v_dim``
(``eps`` inside the root, no weight); the heads side by side are multiplied by silu(W_g h) and projected by W_o.

The recurrence runs on the kernel that the other matrix-state mixers use (``csrc/gated_scan.cu``, the form without
the delta correction), its per-row decay and strength being the head's constant and 1.  The matrices live in the
request's state slot as 32-bit floats; rotation, scaling, recurrence and norm are 32-bit whatever the engine's dtype.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..kernels import ops
from .base import MATRIX, POSITIONS, KVCacheView, ParamSpec, StepContext, register_mixer
from .gated_scan import _ScanMixer, _round_up


@register_mixer("retention")
class Retention(_ScanMixer):
    def __init__(self, width: int, n_head: int, head_dim: int, v_dim: int, decay: Sequence[float], eps: float,
                 rot_dims: int = 0, rot_base: float = 10000.0, out_scale: float = 1.0):
        if min(width, n_head, head_dim, v_dim) <= 0 or len(decay) != n_head:
            raise ValueError("retention: sizes must be positive, one decay per head")
        if any(not 0.0 < float(d) <= 1.0 for d in decay):
            raise ValueError("retention: a decay lies in (0, 1]")
        if rot_dims < 0 or rot_dims % 2 or rot_dims > head_dim:
            raise ValueError("retention: rot_dims must be even and at most head_dim")
        self.width, self.n_head, self.n_kq, self.n_key, self.n_val = int(width), int(n_head), int(n_head), \
            int(head_dim), int(v_dim)
        self.decay, self.eps, self.out_scale = [float(d) for d in decay], float(eps), float(out_scale)
        self.taps, self.channels = 0, 0
        self.rotary = POSITIONS.build("rotary_halves", base=rot_base, dims=rot_dims)
        self.n_qk, self.n_v = self.n_head * self.n_key, self.n_head * self.n_val
        #: columns of the fused projection's output: q | k | v | g, a multiple of 8 wide
        self.offsets = (0, self.n_qk, 2 * self.n_qk, 2 * self.n_qk + self.n_v)
        self.n_proj = _round_up(2 * self.n_qk + 2 * self.n_v, 8)
        self._state_layout()

    def param_specs(self) -> List[ParamSpec]:
        c = self.width
        return [ParamSpec("q_weight", (self.n_qk, c), MATRIX), ParamSpec("k_weight", (self.n_qk, c), MATRIX),
                ParamSpec("v_weight", (self.n_v, c), MATRIX), ParamSpec("g_weight", (self.n_v, c), MATRIX),
                ParamSpec("out_weight", (c, self.n_v), MATRIX)]

    def prepare(self, dtype, device) -> None:
        super().prepare(dtype, device)
        self.rotary.prepare(dtype, device)
        self.w_in = self._fuse(("q_weight", "k_weight", "v_weight", "g_weight"), self.offsets)
        self.decays = torch.tensor(self.decay, dtype=torch.float32, device=device)
        self.ones = torch.ones(self.n_val, dtype=torch.float32, device=device)

    def forward(self, xn: torch.Tensor, x: torch.Tensor, ctx: StepContext, cache: Optional[KVCacheView],
                state: Optional[torch.Tensor], writes_cache: bool = True) -> None:
        if state is None:
            raise ValueError("retention needs a state slot tensor")
        if isinstance(xn, ops.NormInput):
            xn = xn.materialise(ctx.n_rows)
        T, p = ctx.n_rows, self.params
        proj, _, coef, o, out = self._buffers(ctx)
        ops.trace_scope(ctx.layer, "scan_in")
        ops.linear(xn, self.w_in, None, proj, T)
        ops.rope_halves(proj, 0, self.n_qk, self.n_head, self.n_key, self.rotary.dims, self.rotary.freqs, ctx.positions,
                        self.n_key ** -0.5, T, self.decays, coef)
        ops.gated_scan(False, proj, 0, self.n_qk, 2 * self.n_qk, self.n_key, self.n_val, self.n_head, 1, coef, None,
                       state, self.s_off, ctx, o)
        ops.gated_norm(o, proj[:, self.offsets[3]:self.offsets[3] + self.n_v], self.ones, self.n_head, self.n_val,
                       self.eps, False, self.out_scale, out, T)
        ops.trace_scope(ctx.layer, "scan_proj")
        ops.linear(out, p["out_weight"], None, x, T, residual=True)
