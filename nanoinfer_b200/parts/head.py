"""The LM head: logits = h . W^T without bias, as 32-bit floats, for the rows that were
asked for only (reference: crates/core/src/stages/blocks.rs:143-158).  Whether W is the token
embedding's table (tied) or a tensor of its own is the checkpoint mapping's business."""
from __future__ import annotations

from typing import List

import torch

from ..kernels import ops
from .base import TABLE, Head, ParamSpec, StepContext, register_head


@register_head("linear_head")
class LinearHead(Head):
    takes_norm_input = True

    def __init__(self, vocab_size: int, width: int, softcap: float = 0.0, scale: float = 1.0):
        """``scale`` != 1: logits <- scale * logits; ``softcap`` > 0: logits <- softcap * tanh(logits / softcap)
        (after the scale); both in 32-bit, in place."""
        if softcap < 0.0:
            raise ValueError("linear_head: softcap must not be negative")
        self._vocab, self.width, self.softcap, self.scale = int(vocab_size), int(width), float(softcap), float(scale)
        self._cap = self._scale = None

    def prepare(self, dtype, device) -> None:
        super().prepare(dtype, device)
        if self.softcap > 0.0:
            self._cap = torch.tensor([self.softcap], dtype=torch.float32, device=device)
        if self.scale != 1.0:
            self._scale = torch.tensor([self.scale], dtype=torch.float32, device=device)

    @property
    def vocab_size(self) -> int:
        return self._vocab

    def param_specs(self) -> List[ParamSpec]:
        return [ParamSpec("weight", (self._vocab, self.width), TABLE)]

    def forward(self, h, out: torch.Tensor, n_rows: int, ctx: StepContext) -> None:
        """``h``: the normed rows, or a foldable norm input (``Norm.as_input``) of the rows wanted."""
        ops.trace_scope(-1, "lm_head")
        if isinstance(h, ops.NormInput):
            ops.linear(None, self.params["weight"], None, out, n_rows, norm=h)
        else:
            ops.linear(h, self.params["weight"], None, out, n_rows)
        if self._scale is not None:
            ops.unary(out, out, n_rows, ops.UNARY_SCALE, self._scale)
        if self._cap is not None:
            ops.unary(out, out, n_rows, ops.UNARY_SOFTCAP, self._cap)
