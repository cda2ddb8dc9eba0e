"""Hyper-connections with an optional gate on the sublayer's result.

Instead of one residual stream a model keeps ``streams`` copies x_0 .. x_{S-1}, all equal to the embedding's output
at the start.  A sublayer reads u = sum_s in[s] x_s (through the layer's norm); its result y goes back into all copies
at once, from the old ones:   x_t <- sum_s mix[s, t] x_s + out[t] y   (``mix`` indexed [from, to]).  What leaves the
last layer is the sum of the copies.  ``gated``: y is first multiplied element by element by sigmoid(W h + b), h being
the sublayer's own input (the normed u).

The part owns the parameters of ONE sublayer's connection (in [S], out [S], mix [S, S], and the gate's W [C, C] and
b [C]); the ``hyper_connections`` block arrangement holds one per sublayer and runs the kernels
(``csrc/hyper.cu``).  With ``streams`` 1, in = out = mix = 1 and no gate this is the plain residual sum."""
from __future__ import annotations

from typing import List

from .base import INIT_ONE_PLUS_NORMAL, MATRIX, VECTOR, Connector, ParamSpec, register_connector

#: the most copies the kernels hold in a thread's registers
MAX_STREAMS = 8


@register_connector("hyper_connection")
class HyperConnection(Connector):
    def __init__(self, width: int, streams: int, gated: bool = False):
        if not 1 <= streams <= MAX_STREAMS:
            raise ValueError(f"hyper_connection: streams must lie between 1 and {MAX_STREAMS}, got {streams}")
        self.width, self.streams, self.gated = int(width), int(streams), bool(gated)

    def param_specs(self) -> List[ParamSpec]:
        s, c = self.streams, self.width
        specs = [ParamSpec("in", (s,), VECTOR, INIT_ONE_PLUS_NORMAL), ParamSpec("out", (s,), VECTOR, INIT_ONE_PLUS_NORMAL),
                 ParamSpec("mix", (s, s), VECTOR, INIT_ONE_PLUS_NORMAL)]
        if self.gated:
            specs += [ParamSpec("gate_weight", (c, c), MATRIX), ParamSpec("gate_bias", (c,), VECTOR)]
        return specs

    def matrix_flops_per_row(self) -> float:
        return 2.0 * self.width * self.width if self.gated else 0.0
