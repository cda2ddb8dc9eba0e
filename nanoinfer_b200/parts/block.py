"""How the parts of a layer are arranged.  The pre-norm block is the reference's
(crates/core/src/stages/blocks.rs:4-8):
    x = x + mixer(norm_1(x));   x = x + feed_forward(norm_2(x))
Another arrangement is another class registered under another name.  An arrangement names the
parts it is made of and the registry each comes from (``slots``); a layer's specification gives a
part for each of these names, and the model builds them."""
from __future__ import annotations

from typing import Callable, ClassVar, Dict, Optional, Type

import torch

from ..kernels import ops
from .base import (CONNECTORS, DEPTH_MIXES, FEED_FORWARDS, MIXERS, NORMS, KVCacheView, Mixer, Part, Registry, StepContext,
                   StepLimits, Workspace)

BLOCKS: Dict[str, Type["Block"]] = {}


def register_block(name: str) -> Callable[[Type["Block"]], Type["Block"]]:
    def deco(cls):
        BLOCKS[name] = cls
        return cls
    return deco


class Block:
    #: part name -> the registry it is built from.  At most one of them may be a mixer: the cache
    #: manager gives a run of the layer one set of pages or one state slot tensor.
    slots: ClassVar[Dict[str, Registry]] = {}
    #: names of ``slots`` that a layer may leave out
    optional: ClassVar[tuple] = ()

    def __init__(self, width: int, parts: Dict[str, Part]):
        missing, unknown = set(self.slots) - set(parts) - set(self.optional), set(parts) - set(self.slots)
        if missing or unknown:
            raise ValueError(f"{type(self).__name__} is made of {sorted(self.slots)}: missing {sorted(missing)}, "
                             f"unknown {sorted(unknown)}")
        self.width = int(width)
        self._parts = dict(parts)
        for name, part in parts.items():
            setattr(self, name, part)
        mixers = [p for p in parts.values() if isinstance(p, Mixer)]
        if len(mixers) > 1:
            raise ValueError("a block holds at most one mixer")
        #: the part that mixes across positions (None: the layer has none)
        self.mixer: Optional[Mixer] = mixers[0] if mixers else None

    def parts(self) -> Dict[str, Part]:
        return dict(self._parts)

    def reserve(self, workspace: Workspace, limits: StepLimits) -> None:
        """Size the arrangement's own scratch (the parts size theirs themselves)."""

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Optional[KVCacheView],
                state: Optional[torch.Tensor], writes_cache: bool, dtype: torch.dtype) -> None:
        raise NotImplementedError


@register_block("pre_norm")
class PreNormBlock(Block):
    slots = {"norm_1": NORMS, "mixer": MIXERS, "norm_2": NORMS, "feed_forward": FEED_FORWARDS}

    def reserve(self, workspace, limits) -> None:
        workspace.reserve("block.normed", limits.max_rows * self.width, limits.dtype)

    def _normed(self, norm, part, x, ctx, dtype):
        """The part's input: a foldable norm input where both the norm and the part can do that,
        else the norm's output in scratch."""
        if part.takes_norm_input:
            folded = norm.as_input(x, ctx, dtype)
            if folded is not None:
                return folded
        xn = ctx.workspace.get("block.normed", (ctx.max_rows, self.width), dtype)
        norm.forward(x, xn, ctx.n_rows)
        return xn

    def forward(self, x, ctx, cache, state, writes_cache, dtype) -> None:
        self.mixer.forward(self._normed(self.norm_1, self.mixer, x, ctx, dtype), x, ctx, cache, state, writes_cache)
        self.feed_forward.forward(self._normed(self.norm_2, self.feed_forward, x, ctx, dtype), x, ctx)


@register_block("post_norm_depth_mix")
class PostNormDepthMixBlock(Block):
    """Norm AFTER the sum, the sublayers reading the stream itself:
        x <- norm_1(alpha * x + mixer(x));   x <- norm_2(alpha * x + feed_forward(x))
    (a layer without a feed-forward has the first line only), and then, with a ``depth_mix``, what goes on
    is a weighted sum of the embedding's output and ALL layers' results so far, this one's among them.

    On the device the stream is kept pre-scaled: one kernel leaves the sublayer's input (the stream in the
    engine's dtype) and alpha times the stream, into which the sublayer's last product adds; the norm that
    follows does the same for the next sublayer in its own kernel, and the layer's last kernel (norm, the
    level's store, the sum over levels) does it for the next layer where that is one of this arrangement."""

    slots = {"norm_1": NORMS, "mixer": MIXERS, "norm_2": NORMS, "feed_forward": FEED_FORWARDS,
             "depth_mix": DEPTH_MIXES}
    optional = ("norm_2", "feed_forward", "depth_mix")

    def __init__(self, width: int, parts: Dict[str, Part], alpha: float = 1.0):
        super().__init__(width, parts)
        if ("norm_2" in parts) != ("feed_forward" in parts):
            raise ValueError("post_norm_depth_mix: norm_2 and feed_forward come together or not at all")
        for name in ("norm_1", "norm_2"):
            if name in parts and not hasattr(parts[name], "eps"):
                raise ValueError(f"post_norm_depth_mix: {name} must be an RMS norm")
        self.alpha = float(alpha)
        self.norm_2 = parts.get("norm_2")
        self.feed_forward = parts.get("feed_forward")
        self.depth_mix = parts.get("depth_mix")

    def reserve(self, workspace, limits) -> None:
        workspace.reserve("block.stream_in", limits.max_rows * self.width, limits.dtype)
        if self.depth_mix is not None:
            workspace.reserve("block.levels", self.depth_mix.n_levels * limits.max_rows * self.width, torch.float32)

    def forward(self, x, ctx, cache, state, writes_cache, dtype) -> None:
        T, ws = ctx.n_rows, ctx.workspace
        xn = ws.get("block.stream_in", (ctx.max_rows, self.width), dtype)
        levels = None
        if self.depth_mix is not None:
            levels = ws.get("block.levels", (self.depth_mix.n_levels, ctx.max_rows, self.width), torch.float32)
        if ctx.stream_entered:
            ctx.stream_entered = False      # the arrangement before this one left xn and alpha * x behind
        else:
            first = levels is not None and self.depth_mix.n_levels == 2   # level 0 is what this layer was given
            ops.stream_enter(x, xn, self.alpha, T, levels[0] if first else None)
        self.mixer.forward(xn, x, ctx, cache, state, writes_cache)
        last = self.norm_1
        if self.feed_forward is not None:
            ops.post_norm(x, self.norm_1.params["weight"], self.norm_1.eps, T, xn=xn, alpha_next=self.alpha)
            self.feed_forward.forward(xn, x, ctx)
            last = self.norm_2
        nxt = ctx.next_block
        fuse = isinstance(nxt, PostNormDepthMixBlock) and nxt.width == self.width
        if fuse:
            ctx.stream_entered = True
        ops.post_norm(x, last.params["weight"], last.eps, T, xn=xn if fuse else None,
                      alpha_next=nxt.alpha if fuse else 1.0, levels=levels,
                      n_levels=self.depth_mix.n_levels if levels is not None else 0,
                      mix=self.depth_mix.params["weights"] if levels is not None else None)


@register_block("sandwich_norm")
class SandwichNormBlock(Block):
    """A norm before AND after each sublayer, the second one ahead of the sum:
        x <- x + norm_1b(mixer(norm_1(x)));   x <- x + norm_2b(feed_forward(norm_2(x)))
    (a layer without a feed-forward has the first line only).  All four are RMS norms with one eps.

    A sublayer adds its products into a 32-bit buffer of its own that it finds zero.  Between two sublayers runs
    ONE kernel: the norm of that buffer, the sum into the stream, the buffer zeroed again, and the norm that the
    next sublayer reads, also the first norm of the next layer where that is of this arrangement
    (``ctx.stream_entered`` then tells it that its input is ready)."""

    slots = {"norm_1": NORMS, "mixer": MIXERS, "norm_1b": NORMS, "norm_2": NORMS, "feed_forward": FEED_FORWARDS,
             "norm_2b": NORMS}
    optional = ("norm_2", "feed_forward", "norm_2b")

    def __init__(self, width: int, parts: Dict[str, Part]):
        super().__init__(width, parts)
        have = [name in parts for name in ("norm_2", "feed_forward", "norm_2b")]
        if any(have) and not all(have):
            raise ValueError("sandwich_norm: norm_2, feed_forward and norm_2b come together or not at all")
        norms = [parts[n] for n in ("norm_1", "norm_1b", "norm_2", "norm_2b") if n in parts]
        if any(not hasattr(n, "eps") or "bias" in {s.key for s in n.param_specs()} for n in norms):
            raise ValueError("sandwich_norm: its norms must be RMS norms")
        if len({n.eps for n in norms}) != 1:
            raise ValueError("sandwich_norm: its norms share one eps")
        self.eps = norms[0].eps
        self.norm_2, self.feed_forward, self.norm_2b = parts.get("norm_2"), parts.get("feed_forward"), parts.get("norm_2b")

    def reserve(self, workspace, limits) -> None:
        workspace.reserve("block.normed", limits.max_rows * self.width, limits.dtype)
        workspace.reserve("block.sublayer", limits.max_rows * self.width, torch.float32, zeroed=True)

    def forward(self, x, ctx, cache, state, writes_cache, dtype) -> None:
        T, ws = ctx.n_rows, ctx.workspace
        xn = ws.get("block.normed", (ctx.max_rows, self.width), dtype)
        # zero when first handed out, and zeroed again by every kernel that reads it
        y = ws.get_zeroed("block.sublayer", (ctx.max_rows, self.width), torch.float32)
        if ctx.stream_entered:
            ctx.stream_entered = False      # the arrangement before this one left norm_1(x) behind
        else:
            self.norm_1.forward(x, xn, T)
        self.mixer.forward(xn, y, ctx, cache, state, writes_cache)
        last = self.norm_1b
        if self.feed_forward is not None:
            ops.add_norm(x, y, self.norm_1b.params["weight"], self.eps, T, self.norm_2.params["weight"], xn)
            self.feed_forward.forward(xn, y, ctx)
            last = self.norm_2b
        nxt = ctx.next_block
        fuse = isinstance(nxt, SandwichNormBlock) and nxt.width == self.width and nxt.eps == self.eps
        if fuse:
            ctx.stream_entered = True
        ops.add_norm(x, y, last.params["weight"], self.eps, T, nxt.norm_1.params["weight"] if fuse else None,
                     xn if fuse else None)


@register_block("output_norm")
class OutputNormBlock(Block):
    """A norm on each sublayer's OUTPUT only, ahead of the sum; the sublayers read the stream itself:
        x <- x + norm_1(mixer(x));   x <- x + norm_2(feed_forward(x));   x <- x + norm_3(token_input(x))
    (the second and the third line only where the layer has that part; ``token_input`` is any row-wise part that
    also reads the rows' tokens).  All are RMS norms with one eps.

    A sublayer reads the stream cast to the engine's dtype and adds its products into a 32-bit buffer of its own
    that it finds zero.  Between two sublayers runs ONE kernel: the norm of that buffer, the sum into the stream,
    the buffer zeroed again, and the cast of the new stream that the next sublayer reads, also for the next layer
    where that is of this arrangement (``ctx.stream_entered`` then tells it that its input is ready)."""

    slots = {"mixer": MIXERS, "norm_1": NORMS, "feed_forward": FEED_FORWARDS, "norm_2": NORMS,
             "token_input": FEED_FORWARDS, "norm_3": NORMS}
    optional = ("feed_forward", "norm_2", "token_input", "norm_3")

    def __init__(self, width: int, parts: Dict[str, Part]):
        super().__init__(width, parts)
        for a, b in (("feed_forward", "norm_2"), ("token_input", "norm_3")):
            if (a in parts) != (b in parts):
                raise ValueError(f"output_norm: {a} and {b} come together or not at all")
        norms = [parts[n] for n in ("norm_1", "norm_2", "norm_3") if n in parts]
        if any(not hasattr(n, "eps") or "bias" in {s.key for s in n.param_specs()} for n in norms):
            raise ValueError("output_norm: its norms must be RMS norms")
        if len({n.eps for n in norms}) != 1:
            raise ValueError("output_norm: its norms share one eps")
        self.eps = norms[0].eps
        #: (sublayer, the norm of its output), in run order
        self.sublayers = [(parts["mixer"], parts["norm_1"])]
        self.sublayers += [(parts[a], parts[b]) for a, b in (("feed_forward", "norm_2"), ("token_input", "norm_3"))
                           if a in parts]

    def reserve(self, workspace, limits) -> None:
        workspace.reserve("block.normed", limits.max_rows * self.width, limits.dtype)
        workspace.reserve("block.sublayer", limits.max_rows * self.width, torch.float32, zeroed=True)

    def forward(self, x, ctx, cache, state, writes_cache, dtype) -> None:
        T, ws = ctx.n_rows, ctx.workspace
        xn = ws.get("block.normed", (ctx.max_rows, self.width), dtype)
        # zero when first handed out, and zeroed again by every kernel that reads it
        y = ws.get_zeroed("block.sublayer", (ctx.max_rows, self.width), torch.float32)
        if ctx.stream_entered:
            ctx.stream_entered = False      # the arrangement before this one left the cast stream behind
        else:
            ops.stream_enter(x, xn, 1.0, T)
        nxt = ctx.next_block
        fuse = isinstance(nxt, OutputNormBlock) and nxt.width == self.width
        for i, (part, norm) in enumerate(self.sublayers):
            if i == 0:
                part.forward(xn, y, ctx, cache, state, writes_cache)
            else:
                part.forward(xn, y, ctx)
            last = i + 1 == len(self.sublayers)
            ops.add_norm(x, y, norm.params["weight"], self.eps, T, None, None if last and not fuse else xn)
        if fuse:
            ctx.stream_entered = True


@register_block("hyper_connections")
class HyperConnectionBlock(Block):
    """Pre-norm sublayers on several copies of the residual stream (hyper-connections):
        u = sum_s in[s] x_s;   y = sublayer(norm(u));   x_t <- sum_s mix[s, t] x_s + out[t] y   for all copies t at once
    for the mixer (``norm_1``, ``connect_1``) and then for the feed-forward (``norm_2``, ``connect_2``; a layer may have
    none).  A connector that is ``gated`` multiplies y by sigmoid(W norm(u) + b) first.  The norms are RMS norms.  The
    copies are all equal to the stream the first such layer is given; behind the last one the stream is their sum.

    The copies live in a 32-bit buffer of the arrangement's own.  A sublayer adds its products into a 32-bit buffer
    that it finds zero; the gate's logits are one more product of the sublayer's input.  Between two sublayers runs ONE
    kernel: the gate, all copies' update, the buffer zeroed again, and the next sublayer's normed input, also the next
    layer's where that is of this arrangement (``ctx.stream_entered`` tells it that its input is ready); behind the
    last layer of the arrangement the same kernel leaves the copies' sum in the stream."""

    slots = {"norm_1": NORMS, "mixer": MIXERS, "connect_1": CONNECTORS, "norm_2": NORMS, "feed_forward": FEED_FORWARDS,
             "connect_2": CONNECTORS}
    optional = ("norm_2", "feed_forward", "connect_2")
    #: True: every layer also leaves the copies' sum in the stream (for looking at a model layer by layer)
    always_sum = False

    def __init__(self, width: int, parts: Dict[str, Part]):
        super().__init__(width, parts)
        have = [name in parts for name in ("norm_2", "feed_forward", "connect_2")]
        if any(have) and not all(have):
            raise ValueError("hyper_connections: norm_2, feed_forward and connect_2 come together or not at all")
        norms = [parts[n] for n in ("norm_1", "norm_2") if n in parts]
        if any(not hasattr(n, "eps") or "bias" in {s.key for s in n.param_specs()} for n in norms):
            raise ValueError("hyper_connections: its norms must be RMS norms")
        self.norm_2, self.feed_forward, self.connect_2 = parts.get("norm_2"), parts.get("feed_forward"), parts.get("connect_2")
        connectors = [parts[n] for n in ("connect_1", "connect_2") if n in parts]
        if len({c.streams for c in connectors}) != 1 or any(c.width != self.width for c in connectors):
            raise ValueError("hyper_connections: the connectors of a layer share the number of copies and the width")
        self.streams = connectors[0].streams

    def reserve(self, workspace, limits) -> None:
        workspace.reserve("block.normed", limits.max_rows * self.width, limits.dtype)
        workspace.reserve("block.sublayer", limits.max_rows * self.width, torch.float32, zeroed=True)
        workspace.reserve("block.copies", self.streams * limits.max_rows * self.width, torch.float32)
        workspace.reserve("block.gate", limits.max_rows * self.width, torch.float32)

    def _back(self, connect, xn, y, copies, gate, ctx, T, nxt_norm, nxt_connect, total) -> None:
        """The sublayer's result back into the copies, and the next sublayer's input (``nxt_norm`` None: none)."""
        p = connect.params
        if connect.gated:
            ops.trace_scope(ctx.layer, "gate")
            ops.linear(xn, p["gate_weight"], p["gate_bias"], gate, T)
        ops.hyper_update(copies, y, gate if connect.gated else None, p["mix"], p["out"],
                         nxt_norm.eps if nxt_norm is not None else 0.0, T,
                         in_next=nxt_connect.params["in"] if nxt_norm is not None else None,
                         w_next=nxt_norm.params["weight"] if nxt_norm is not None else None,
                         xn=xn if nxt_norm is not None else None, total=total)

    def forward(self, x, ctx, cache, state, writes_cache, dtype) -> None:
        T, ws = ctx.n_rows, ctx.workspace
        xn = ws.get("block.normed", (ctx.max_rows, self.width), dtype)
        # zero when first handed out, and zeroed again by every kernel that reads it
        y = ws.get_zeroed("block.sublayer", (ctx.max_rows, self.width), torch.float32)
        copies = ws.get("block.copies", (self.streams, ctx.max_rows, self.width), torch.float32)
        gate = ws.get("block.gate", (ctx.max_rows, self.width), torch.float32)
        if ctx.stream_entered:
            ctx.stream_entered = False      # the arrangement before this one left the copies and norm_1's output behind
        else:
            ops.hyper_enter(x, copies, self.connect_1.params["in"], self.norm_1.params["weight"], self.norm_1.eps, xn, T)
        nxt = ctx.next_block
        fuse = isinstance(nxt, HyperConnectionBlock) and nxt.width == self.width and nxt.streams == self.streams
        total = x if (not fuse or self.always_sum) else None
        last = (nxt.norm_1, nxt.connect_1) if fuse else (None, None)
        self.mixer.forward(xn, y, ctx, cache, state, writes_cache)
        if self.feed_forward is None:
            self._back(self.connect_1, xn, y, copies, gate, ctx, T, last[0], last[1], total)
        else:
            self._back(self.connect_1, xn, y, copies, gate, ctx, T, self.norm_2, self.connect_2, None)
            self.feed_forward.forward(xn, y, ctx)
            self._back(self.connect_2, xn, y, copies, gate, ctx, T, last[0], last[1], total)
        if fuse:
            ctx.stream_entered = True
