"""Learned absolute positions: a table row per position, added to the token embedding
(reference: crates/core/src/kernels/reference.rs:86-94).  The table's length bounds the
context (crates/core/src/stages/mod.rs:516-519)."""
from __future__ import annotations

from typing import List, Optional

import torch

from ..kernels import ops
from .base import TABLE, ParamSpec, PositionEncoding, register_position


@register_position("learned_absolute")
class LearnedAbsolutePositions(PositionEncoding):
    def __init__(self, n_positions: int, width: int):
        self.n_positions, self.width = int(n_positions), int(width)

    def param_specs(self) -> List[ParamSpec]:
        return [ParamSpec("table", (self.n_positions, self.width), TABLE)]

    def additive_table(self) -> Optional[torch.Tensor]:
        return self.params["table"]

    def max_positions(self) -> Optional[int]:
        return self.n_positions


@register_position("rotary_pairs")
class RotaryPairs(PositionEncoding):
    """Rotary positions inside a mixer: of every query and key head the first ``dims`` values turn in pairs
    (2i, 2i + 1) (the interleaved layout) by the angle position * base^(-2i / dims); the other values pass.
    It has no parameters.  The frequencies are made in double precision on the host; the rotation itself is
    done by the mixer's own kernel between the projection and the cache (``kernels.ops.rope_append``), which asks
    this part for ``dims`` and ``freqs``."""

    def __init__(self, base: float, dims: int):
        if dims < 0 or dims % 2:
            raise ValueError(f"rotary_pairs: dims {dims} must be even and not negative")
        if dims and not base > 0.0:
            raise ValueError(f"rotary_pairs: base {base} must be positive")
        self.base, self.dims = float(base), int(dims)
        self.freqs: Optional[torch.Tensor] = None

    def prepare(self, dtype, device) -> None:
        super().prepare(dtype, device)
        if self.dims:
            i = torch.arange(self.dims // 2, dtype=torch.float64)
            self.freqs = (self.base ** (-2.0 * i / self.dims)).to(device)

    def on_qk(self, q, k, ctx) -> None:
        raise NotImplementedError("rotary_pairs turns queries and keys inside ops.rope_append, on the projection's "
                                  "32-bit output; a mixer that holds it calls that")


@register_position("sinusoidal")
class SinusoidalPositions(PositionEncoding):
    """Fixed sinusoidal positions added to the embedding: entry 2i of a row at position p gets
    sin(p * base^(-2i / width)), entry 2i + 1 the cosine of the same angle.  No parameters and no table: the
    frequencies are made in double precision on the host, and one kernel makes angle, sine and cosine in double
    precision from the row's position, so no length bounds the context."""

    def __init__(self, width: int, base: float = 10000.0):
        if width <= 0 or not base > 0.0:
            raise ValueError("sinusoidal: width and base must be positive")
        self.width, self.base = int(width), float(base)
        self.freqs: Optional[torch.Tensor] = None

    def prepare(self, dtype, device) -> None:
        super().prepare(dtype, device)
        i = torch.arange((self.width + 1) // 2, dtype=torch.float64)
        self.freqs = (self.base ** (-2.0 * i / self.width)).to(device)

    def on_embedding(self, x, ctx) -> None:
        ops.add_sinusoid(x, ctx.positions, self.freqs, ctx.n_rows)


@register_position("rotary_halves")
class RotaryHalves(RotaryPairs):
    """Rotary positions in the halves layout: of every query and key head the first ``dims`` values turn, value i
    paired with value i + dims / 2, by the angle position * base^(-2i / dims); the other values pass.  The rotation is
    done by the mixer's own kernel (``kernels.ops.wide_norm_rope_append``, ``kernels.ops.rope_halves``)."""

    layout = "halves"
