"""Causal multi-head attention over the paged cache, with a fused query/key/value projection
and an output projection whose epilogue adds into the residual stream.

Reference: qkv = ln_1(x) . W^T + b with the row laid out [q | k | v] and head h owning
columns h*hd..(h+1)*hd of each third (crates/core/src/stages/blocks.rs:31-50); keys and values
appended to the cache after the bias (crates/core/src/stages/kv_cache.rs:44-57); scores
(q . k) * scale over the keys j <= pos, softmax, weighted sum of values
(crates/core/src/kernels/reference.rs:109-142); x += att . W_proj^T + b (blocks.rs:103-112).
The reference fixes scale = 1/sqrt(hd) and one key/value head per query head; here the
scale, the number of key/value heads, the head size and a window are parameters.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..kernels import ops
from .base import (INIT_ONE_PLUS_NORMAL, MATRIX, VECTOR, KVCacheSpec, KVCacheView, Mixer, ParamSpec, PositionEncoding, StepContext,
                   StepLimits, StepPlan, Workspace, register_mixer)

#: a plan made for a graph rounds the longest key range of the decoded rows up to this many positions:
#: the split of the keys then stays the same from step to step while the requests grow
GRAPH_KEY_BUCKET = 256


class AttentionPlan(StepPlan):
    """Which rows of a step are single decoded tokens and which belong to prompt portions, and the
    portions cut into tiles of 64 and of 128 query rows, longest key range first; the same for
    every attention layer of the step.  Words: [decoded rows | portion rows (only beside decoded rows) |
    (entry, first row) per 64-row tile | the same per 128-row tile]."""

    def __init__(self, entry_start, entry_pos0, for_graph: bool = False, device=None):
        dec, pre, tiles = [], [], []
        self.max_decode_keys = 0
        #: for the trace's counts: keys seen by the decoded rows, keys seen by the portions' rows, and the
        #: key/value rows the portions' requests hold (each is read once)
        self.decode_keys = self.prefill_keys = self.prefill_kv_rows = 0
        for e in range(len(entry_start) - 1):
            a, b = entry_start[e], entry_start[e + 1]
            if b - a == 1:
                dec.append(a)
                self.max_decode_keys = max(self.max_decode_keys, entry_pos0[e] + 1)
                self.decode_keys += entry_pos0[e] + 1
            else:
                pre.extend(range(a, b))
                tiles.extend((e, off) for off in range(0, b - a, 64))
                n = b - a
                self.prefill_keys += n * entry_pos0[e] + n * (n + 1) // 2
                self.prefill_kv_rows += entry_pos0[e] + n
        # the same portions in tiles of 128 rows, for the tcgen05 kernel
        wide = [(e, off) for e in range(len(entry_start) - 1) if entry_start[e + 1] - entry_start[e] > 1
                for off in range(0, entry_start[e + 1] - entry_start[e], 128)]
        # the tiles that reach furthest back have the most keys to go through: they are launched first,
        # so that the short ones fill the gaps at the end
        tiles.sort(key=lambda t: -(entry_pos0[t[0]] + t[1]))
        wide.sort(key=lambda t: -(entry_pos0[t[0]] + t[1]))
        self.n_decode, self.n_prefill_rows, self.n_tiles = len(dec), len(pre), len(tiles)
        self.n_wide_tiles = len(wide)
        if for_graph:
            self.max_decode_keys = -(-self.max_decode_keys // GRAPH_KEY_BUCKET) * GRAPH_KEY_BUCKET
        # (the portions' rows are listed only beside decoded rows: alone they are the rows 0..n-1, and two
        # steps of portions that differ in a few tokens then have the same words' layout and one graph)
        self.n_listed_rows = len(pre) if dec else 0
        self.words = dec + (pre if dec else []) + [v for t in tiles for v in t] + [v for t in wide for v in t]
        if device is not None:
            self.bind(torch.tensor(self.words, dtype=torch.int32, device=device) if self.words else None)

    def graph_key(self) -> tuple:
        return (self.n_decode, self.n_listed_rows, self.n_tiles, self.n_wide_tiles, self.max_decode_keys)

    def bind(self, buf) -> None:
        """``buf``: a device int32 tensor holding ``self.words``."""
        nd, npre = self.n_decode, self.n_listed_rows
        all_decode = self.n_prefill_rows == 0
        # rows 0..n-1 in order need no index list
        self.decode_rows = None if all_decode or nd == 0 else buf[:nd]
        self.prefill_rows = None if nd == 0 or npre == 0 else buf[nd:nd + npre]
        self.tiles = buf[nd + npre:nd + npre + 2 * self.n_tiles] if self.n_tiles else None
        at = nd + npre + 2 * self.n_tiles
        self.wide_tiles = buf[at:at + 2 * self.n_wide_tiles] if self.n_wide_tiles else None


def _split(xn):
    """(tensor, norm input): a part's input is either the normed rows or a foldable norm input."""
    return (None, xn) if isinstance(xn, ops.NormInput) else (xn, None)


@register_mixer("causal_attention")
class CausalSelfAttention(Mixer):
    takes_norm_input = True

    def __init__(self, width: int, n_head: int, n_kv_head: int, head_dim: int, scale: float,
                 window: int = 0, bias: bool = True, position: Optional[PositionEncoding] = None):
        if n_head <= 0 or n_kv_head <= 0 or n_head % n_kv_head != 0:
            raise ValueError(f"n_head {n_head} must be a positive multiple of n_kv_head {n_kv_head}")
        if head_dim <= 0 or head_dim % 8 != 0 or head_dim > 256:
            raise ValueError(f"head_dim {head_dim} is not supported: it must be a multiple of 8, at most 256")
        if window < 0:
            raise ValueError("window must be >= 0")
        self.width, self.n_head, self.n_kv_head, self.head_dim = int(width), int(n_head), int(n_kv_head), int(head_dim)
        self.scale, self.window, self.bias, self.position = float(scale), int(window), bool(bias), position
        self.q_dim = self.n_head * self.head_dim
        self.kv_dim = self.n_kv_head * self.head_dim

    def param_specs(self) -> List[ParamSpec]:
        specs = [ParamSpec("qkv_weight", (self.q_dim + 2 * self.kv_dim, self.width), MATRIX),
                 ParamSpec("out_weight", (self.width, self.q_dim), MATRIX)]
        if self.bias:
            specs += [ParamSpec("qkv_bias", (self.q_dim + 2 * self.kv_dim,), VECTOR),
                      ParamSpec("out_bias", (self.width,), VECTOR)]
        return specs

    def kv_spec(self) -> Optional[KVCacheSpec]:
        return KVCacheSpec(self.n_kv_head, self.head_dim, self.window)

    def step_planner(self):
        return "causal_attention", AttentionPlan

    def flops_per_key(self) -> float:
        return 4.0 * self.q_dim

    def reserve(self, workspace: Workspace, limits: StepLimits) -> None:
        n = limits.max_rows
        workspace.reserve("attention.qkv", n * (self.q_dim + 2 * self.kv_dim), self.dtype)
        workspace.reserve("attention.out", n * self.q_dim, self.dtype)
        ops.attention_decode_reserve(workspace, self.n_head, self.head_dim)

    def forward(self, xn: torch.Tensor, x: torch.Tensor, ctx: StepContext, cache: Optional[KVCacheView],
                state: Optional[torch.Tensor], writes_cache: bool = True) -> None:
        if cache is None:
            raise ValueError("causal_attention needs a paged cache")
        T, p = ctx.n_rows, self.params
        ws = ctx.workspace
        xn, norm = _split(xn)
        if writes_cache:
            qkv = ws.get("attention.qkv", (ctx.max_rows, self.q_dim + 2 * self.kv_dim), self.dtype)
            # small steps: keys and values go to the cache from the projection's epilogue
            ops.trace_scope(ctx.layer, "qkv")
            fused = self.position is None and ops.linear_qkv(
                xn, p["qkv_weight"], p.get("qkv_bias"), qkv, T, self.q_dim, cache.layer, cache.block_table,
                ctx.row_entry, ctx.positions, ctx.status, norm=norm)
            if not fused:
                ops.linear(xn, p["qkv_weight"], p.get("qkv_bias"), qkv, T, norm=norm)
                if self.position is not None:
                    self.position.on_qk(qkv[:T, :self.q_dim], qkv[:T, self.q_dim:self.q_dim + self.kv_dim], ctx)
                ops.kv_append(qkv, self.q_dim, self.q_dim + self.kv_dim, cache.layer, cache.block_table,
                              ctx.row_entry, ctx.positions, T, ctx.status)
            q = qkv[:, :self.q_dim]
        else:
            # this layer reads another layer's keys and values: only the queries are projected
            q = ws.get("attention.q", (ctx.max_rows, self.q_dim), self.dtype)
            qb = p.get("qkv_bias")
            ops.trace_scope(ctx.layer, "qkv")
            ops.linear(xn, p["qkv_weight"][:self.q_dim], None if qb is None else qb[:self.q_dim], q, T, norm=norm)
            if self.position is not None:
                self.position.on_qk(q[:T], None, ctx)
        att = ws.get("attention.out", (ctx.max_rows, self.q_dim), self.dtype)
        plan = ctx.plans.get("causal_attention")
        if plan is None:    # a caller that drives the part without the step function
            plan = ctx.plans["causal_attention"] = AttentionPlan(ctx.host_entry_start, ctx.host_entry_pos0,
                                                                 device=x.device)
        ops.attention(q, cache.layer, att, cache.block_table, ctx, self.n_head, self.scale, self.window, plan)
        ops.trace_scope(ctx.layer, "attn_proj")
        ops.linear(att, p["out_weight"], p.get("out_bias"), x, T, residual=True)


def _round_up(n: int, m: int) -> int:
    return -(-n // m) * m


@register_mixer("general_attention")
class GeneralAttention(CausalSelfAttention):
    """Causal attention with the projections as separate tensors and without biases, key and value heads of sizes of
    their own (``head_dim`` for queries and keys, ``v_dim`` for values), grouped key/value heads (query head h reads
    key/value head h // (n_head / n_kv_head)), an optional rotary position encoding on queries and keys (``position``:
    a ``rotary_pairs`` part) and an optional **sink**: the softmax's denominator has one more term, exp(0), as if
    every row also saw a key of score 0 that has no value:  p_j = exp(s_j) / (1 + sum_j exp(s_j)).

    One product makes q, k and v as 32-bit floats; one kernel turns queries and keys by their positions (in 32-bit,
    angles in double precision), casts, and writes keys and values into the cache.  The cache and the attention
    kernels know one head size: the larger of the two, rounded up to 16; keys or values of the smaller size are
    padded with zeros there (a zero adds nothing to a score and a zero value gives a zero output, which the output
    projection, its matrix padded with zero columns at load, ignores)."""

    def __init__(self, width: int, n_head: int, n_kv_head: int, head_dim: int, v_dim: int, scale: float,
                 window: int = 0, sink: bool = False, position: Optional[PositionEncoding] = None):
        if head_dim <= 0 or v_dim <= 0 or head_dim % 2 or v_dim % 2:
            raise ValueError(f"general_attention: head_dim {head_dim} and v_dim {v_dim} must be positive and even")
        self.cache_dim = _round_up(max(head_dim, v_dim), 16)
        super().__init__(width, n_head, n_kv_head, self.cache_dim, scale, window, bias=False, position=position)
        self.key_dim, self.v_dim, self.sink = int(head_dim), int(v_dim), bool(sink)
        rot = getattr(position, "dims", 0)
        if position is not None and (not hasattr(position, "freqs") or rot > self.key_dim):
            raise ValueError("general_attention: the position encoding must be rotary_pairs with dims <= head_dim")
        self.n_q, self.n_k, self.n_v = self.n_head * self.key_dim, self.n_kv_head * self.key_dim, self.n_kv_head * self.v_dim
        #: columns of the fused projection's output (rows of 32-bit floats, a multiple of 8 wide)
        self.n_proj = _round_up(self.n_q + self.n_k + self.n_v, 8)

    def param_specs(self) -> List[ParamSpec]:
        return [ParamSpec("q_weight", (self.n_q, self.width), MATRIX), ParamSpec("k_weight", (self.n_k, self.width), MATRIX),
                ParamSpec("v_weight", (self.n_v, self.width), MATRIX),
                ParamSpec("out_weight", (self.width, self.n_head * self.v_dim), MATRIX)]

    def kv_spec(self) -> Optional[KVCacheSpec]:
        return KVCacheSpec(self.n_kv_head, self.cache_dim, self.window)

    def flops_per_key(self) -> float:
        return 2.0 * self.n_head * (self.key_dim + self.v_dim)

    def prepare(self, dtype, device) -> None:
        super().prepare(dtype, device)
        p = self.params
        # the three products that read the mixer's input are one; the parameters by name become views of it
        w = torch.zeros(self.n_proj, self.width, dtype=p["q_weight"].dtype, device=p["q_weight"].device)
        at = 0
        for key in ("q_weight", "k_weight", "v_weight"):
            n = p[key].shape[0]
            w[at:at + n] = p[key]
            p[key] = w[at:at + n]
            at += n
        self.w_qkv = w
        self._pad_out_weight()

    def _pad_out_weight(self) -> None:
        """The output projection reads heads of the cache's size: zero columns where a value head is shorter."""
        p = self.params
        w = p["out_weight"]
        if self.v_dim == self.cache_dim:
            self.w_out = p["out_weight"]
        else:
            wo = torch.zeros(self.width, self.n_head, self.cache_dim, dtype=w.dtype, device=w.device)
            wo[:, :, :self.v_dim] = p["out_weight"].view(self.width, self.n_head, self.v_dim)
            self.w_out = wo.view(self.width, self.n_head * self.cache_dim)
            p["out_weight"] = self.w_out.view(self.width, self.n_head, self.cache_dim)[:, :, :self.v_dim]

    def reserve(self, workspace: Workspace, limits: StepLimits) -> None:
        n = limits.max_rows
        workspace.reserve("attention.proj32", n * self.n_proj, torch.float32)
        workspace.reserve("attention.q", n * self.q_dim, self.dtype)
        workspace.reserve("attention.out", n * self.q_dim, self.dtype)
        ops.attention_decode_reserve(workspace, self.n_head, self.head_dim)

    def forward(self, xn: torch.Tensor, x: torch.Tensor, ctx: StepContext, cache: Optional[KVCacheView],
                state: Optional[torch.Tensor], writes_cache: bool = True) -> None:
        if cache is None:
            raise ValueError("general_attention needs a paged cache")
        if isinstance(xn, ops.NormInput):
            xn = xn.materialise(ctx.n_rows)
        T, ws = ctx.n_rows, ctx.workspace
        proj = ws.get("attention.proj32", (ctx.max_rows, self.n_proj), torch.float32)
        ops.trace_scope(ctx.layer, "qkv")
        # (a run that reads another run's keys and values projects its queries only)
        ops.linear(xn, self.w_qkv if writes_cache else self.w_qkv[:self.n_q], None,
                   proj if writes_cache else proj[:, :self.n_q], T)
        q = ws.get("attention.q", (ctx.max_rows, self.q_dim), self.dtype)
        pos = self.position
        ops.rope_append(proj, (0, self.n_q, self.n_q + self.n_k), self.n_head, self.n_kv_head, self.key_dim, self.v_dim,
                        pos.dims if pos is not None else 0, pos.freqs if pos is not None else None, ctx, q,
                        cache.layer if writes_cache else None, cache.block_table if writes_cache else None)
        att = ws.get("attention.out", (ctx.max_rows, self.q_dim), self.dtype)
        plan = ctx.plans.get("causal_attention")
        if plan is None:
            plan = ctx.plans["causal_attention"] = AttentionPlan(ctx.host_entry_start, ctx.host_entry_pos0,
                                                                 device=x.device)
        ops.attention(q, cache.layer, att, cache.block_table, ctx, self.n_head, self.scale, self.window, plan,
                      sink=self.sink)
        ops.trace_scope(ctx.layer, "attn_proj")
        ops.linear(att, self.w_out, None, x, T, residual=True)


@register_mixer("normed_attention")
class NormedAttention(GeneralAttention):
    """``general_attention`` with what some designs put around the scores, each an option of its own:

    * ``bias``: q, k, v and the output projection have biases;
    * ``qk_norm``: every query and key head is divided by its root mean square over ``head_dim`` (``eps`` inside the
      root) and multiplied by a weight of ``head_dim`` values that all heads share (one for queries, one for keys),
      ahead of the rotation (if any) and of the cache, so the cache holds normed keys;
    * ``softcap`` > 0: s <- softcap * tanh(s / softcap) after the scale;
    * ``distance_bias`` = b: s <- s - slope_h * (i - j) with slope_h = 2^(-b (h + 1) / n_head) for query head h;
    * ``window`` with ``keep_first``: position i sees j <= i with i - j < window or j < keep_first;
    * ``head_gate``: head h's output is multiplied by sigmoid(W_g x)_h, one number per row and head;
    * ``out_scale``: the mixer's whole output times a constant (applied to the heads' outputs, and to the bias);
    * ``own_kv`` False: the layer has no key and value tensors (projections, biases, key norm) at all: it only ever
      runs on another run's cache.

    One product makes [q | gate | k | v] (+ biases) as 32-bit floats; one kernel norms, turns, casts and writes
    queries to the attention's input and keys and values into the cache.  The attention kernels that take the
    options on the scores are the general one (prompt portions) and the streaming split-KV one (single tokens)."""

    def __init__(self, width: int, n_head: int, n_kv_head: int, head_dim: int, v_dim: int, scale: float, eps: float,
                 window: int = 0, keep_first: int = 0, sink: bool = False, bias: bool = False, qk_norm: bool = True,
                 softcap: float = 0.0, distance_bias: Optional[float] = None, head_gate: bool = False,
                 out_scale: float = 1.0, own_kv: bool = True, position: Optional[PositionEncoding] = None):
        super().__init__(width, n_head, n_kv_head, head_dim, v_dim, scale, window, sink, position)
        if keep_first < 0 or softcap < 0.0:
            raise ValueError("normed_attention: keep_first and softcap must not be negative")
        self.bias = bool(bias)
        self.eps, self.keep_first, self.qk_norm, self.softcap = float(eps), int(keep_first), bool(qk_norm), float(softcap)
        self.distance_bias = None if distance_bias is None else float(distance_bias)
        self.head_gate, self.out_scale, self.own_kv = bool(head_gate), float(out_scale), bool(own_kv)
        self.n_g = self.n_head if self.head_gate else 0
        #: columns of the fused projection's output: q | gate | k | v; the first two (a multiple of 8 wide) are all
        #: that a run on another run's cache needs
        self.n_qg = _round_up(self.n_q + self.n_g, 8)
        self.k_off, self.v_off = self.n_qg, self.n_qg + self.n_k
        self.n_proj = _round_up(self.n_qg + self.n_k + self.n_v, 8) if self.own_kv else self.n_qg
        self.slopes: Optional[torch.Tensor] = None

    def param_specs(self) -> List[ParamSpec]:
        c = self.width
        specs = [ParamSpec("q_weight", (self.n_q, c), MATRIX),
                 ParamSpec("out_weight", (c, self.n_head * self.v_dim), MATRIX)]
        if self.own_kv:
            specs += [ParamSpec("k_weight", (self.n_k, c), MATRIX), ParamSpec("v_weight", (self.n_v, c), MATRIX)]
        if self.bias:
            specs += [ParamSpec("q_bias", (self.n_q,), VECTOR), ParamSpec("out_bias", (c,), VECTOR)]
            if self.own_kv:
                specs += [ParamSpec("k_bias", (self.n_k,), VECTOR), ParamSpec("v_bias", (self.n_v,), VECTOR)]
        if self.qk_norm:
            specs.append(ParamSpec("q_norm", (self.key_dim,), VECTOR, INIT_ONE_PLUS_NORMAL))
            if self.own_kv:
                specs.append(ParamSpec("k_norm", (self.key_dim,), VECTOR, INIT_ONE_PLUS_NORMAL))
        if self.head_gate:
            specs.append(ParamSpec("gate_weight", (self.n_head, c), MATRIX))
        return specs

    def kv_spec(self) -> Optional[KVCacheSpec]:
        return KVCacheSpec(self.n_kv_head, self.cache_dim, self.window,
                           keep_first=self.keep_first if self.window > 0 else 0)

    def prepare(self, dtype, device) -> None:
        Mixer.prepare(self, dtype, device)
        p = self.params
        q = p["q_weight"]
        w = torch.zeros(self.n_proj, self.width, dtype=q.dtype, device=q.device)
        b = torch.zeros(self.n_proj, dtype=torch.float32, device=q.device) if self.bias else None
        places = [("q", 0), ("gate", self.n_q)] + ([("k", self.k_off), ("v", self.v_off)] if self.own_kv else [])
        for name, at in places:
            if name + "_weight" not in p:
                continue
            n = p[name + "_weight"].shape[0]
            w[at:at + n] = p[name + "_weight"]
            p[name + "_weight"] = w[at:at + n]
            if b is not None and name + "_bias" in p:
                b[at:at + n] = p[name + "_bias"]
                p[name + "_bias"] = b[at:at + n]
        self.w_qkv, self.b_qkv = w, b
        self._pad_out_weight()
        self.out_bias = p["out_bias"] * self.out_scale if self.bias else None
        if self.distance_bias is not None:
            h = torch.arange(1, self.n_head + 1, dtype=torch.float64)
            self.slopes = (2.0 ** (-self.distance_bias * h / self.n_head)).to(torch.float32).to(device)

    def reserve(self, workspace: Workspace, limits: StepLimits) -> None:
        super().reserve(workspace, limits)
        workspace.reserve("attention.proj32", limits.max_rows * max(self.n_proj, self.n_qg), torch.float32)

    def forward(self, xn: torch.Tensor, x: torch.Tensor, ctx: StepContext, cache: Optional[KVCacheView],
                state: Optional[torch.Tensor], writes_cache: bool = True) -> None:
        if cache is None:
            raise ValueError("normed_attention needs a paged cache")
        if writes_cache and not self.own_kv:
            raise ValueError("normed_attention: a layer without key and value tensors can only read another run's cache")
        if isinstance(xn, ops.NormInput):
            xn = xn.materialise(ctx.n_rows)
        T, ws, p = ctx.n_rows, ctx.workspace, self.params
        n = self.n_proj if writes_cache else self.n_qg
        proj = ws.get("attention.proj32", (ctx.max_rows, n), torch.float32)
        ops.trace_scope(ctx.layer, "qkv")
        ops.linear(xn, self.w_qkv[:n], None if self.b_qkv is None else self.b_qkv[:n], proj, T)
        q = ws.get("attention.q", (ctx.max_rows, self.q_dim), self.dtype)
        pos = self.position
        ops.norm_rope_append(proj, (0, self.k_off, self.v_off), self.n_head, self.n_kv_head, self.key_dim, self.v_dim,
                             p.get("q_norm"), p.get("k_norm") if writes_cache else None, self.eps,
                             pos.dims if pos is not None else 0, pos.freqs if pos is not None else None, ctx, q,
                             cache.layer if writes_cache else None, cache.block_table if writes_cache else None)
        att = ws.get("attention.out", (ctx.max_rows, self.q_dim), self.dtype)
        plan = ctx.plans.get("causal_attention")
        if plan is None:
            plan = ctx.plans["causal_attention"] = AttentionPlan(ctx.host_entry_start, ctx.host_entry_pos0,
                                                                 device=x.device)
        extras = ops.AttnExtras(self.softcap, self.keep_first if self.window > 0 else 0, self.slopes,
                                proj[:, self.n_q:self.n_q + self.n_g] if self.head_gate else None, self.out_scale)
        ops.attention(q, cache.layer, att, cache.block_table, ctx, self.n_head, self.scale, self.window, plan,
                      sink=self.sink, extras=extras)
        ops.trace_scope(ctx.layer, "attn_proj")
        ops.linear(att, self.w_out, self.out_bias, x, T, residual=True)


@register_mixer("span_attention")
class SpanAttention(GeneralAttention):
    """Attention whose queries see only the keys of their own span of ``span`` positions (position i sees j <= i with
    i // span == j // span; spans count from position 0 of the sequence, however a prompt is cut into steps; 0: all
    keys), with what this kind of layer puts around it, each an option:

    * ``taps`` > 0: a short causal convolution over time on every channel of q and of k (weights [channels, taps],
      the last tap the current token's, zeros before the sequence, no bias), right behind the projection; the last
      ``taps - 1`` projected rows of a request are its state;
    * ``wide_norm``: q and k are each divided by the root mean square of the WHOLE projection (all heads at once)
      and multiplied by a weight of that size, ahead of the rotation;
    * ``rot_dims``/``rot_base``: rotary positions in the halves layout on the first ``rot_dims`` values of a head;
    * ``values_are_keys``: there is no value projection; a key head as it leaves the convolution (ahead of norm and
      rotation) is the value head (so ``v_dim`` equals ``head_dim``);
    * ``head_temperature``: a learned number per query head that multiplies the scale;
    * ``learned_sink``: a learned number per query head whose exponential joins the softmax's denominator (a key
      without a value, neither scaled nor multiplied by the temperature).

    One product makes [q | k (| v)] as 32-bit floats, one kernel the convolution (and its state), one the norm, the
    rotation, the cast and the cache write; then the attention kernels with the span, the heads' scales and the sinks
    as options, and the output projection."""

    def __init__(self, width: int, n_head: int, n_kv_head: int, head_dim: int, v_dim: int, scale: float, eps: float,
                 span: int = 0, taps: int = 0, wide_norm: bool = True, rot_dims: int = 0, rot_base: float = 10000.0,
                 values_are_keys: bool = False, head_temperature: bool = False, learned_sink: bool = False,
                 out_scale: float = 1.0):
        from .base import POSITIONS

        if values_are_keys and v_dim != head_dim:
            raise ValueError("span_attention: values that are the keys have the keys' size")
        if span < 0 or taps < 0 or rot_dims < 0 or rot_dims % 2 or rot_dims > head_dim:
            raise ValueError("span_attention: span and taps must not be negative, rot_dims even and at most head_dim")
        super().__init__(width, n_head, n_kv_head, head_dim, v_dim, scale, window=0, sink=learned_sink, position=None)
        self.eps, self.span, self.taps, self.wide_norm = float(eps), int(span), int(taps), bool(wide_norm)
        self.values_are_keys, self.head_temperature = bool(values_are_keys), bool(head_temperature)
        self.learned_sink, self.out_scale = bool(learned_sink), float(out_scale)
        self.rotary = POSITIONS.build("rotary_halves", base=rot_base, dims=rot_dims)
        if self.values_are_keys:
            self.n_v = 0
        self.n_proj = _round_up(self.n_q + self.n_k + self.n_v, 8)
        #: channels that pass the convolution (q and k), and the floats of state that keeps per request
        self.channels = self.n_q + self.n_k
        self.state_floats = _round_up(max(self.taps - 1, 0) * self.channels, 4)

    capture_safe = True

    def param_specs(self) -> List[ParamSpec]:
        c = self.width
        specs = [ParamSpec("q_weight", (self.n_q, c), MATRIX), ParamSpec("k_weight", (self.n_k, c), MATRIX),
                 ParamSpec("out_weight", (c, self.n_head * self.v_dim), MATRIX)]
        if not self.values_are_keys:
            specs.append(ParamSpec("v_weight", (self.n_v, c), MATRIX))
        if self.taps > 0:
            specs += [ParamSpec("q_conv", (self.n_q, self.taps), VECTOR), ParamSpec("k_conv", (self.n_k, self.taps), VECTOR)]
        if self.wide_norm:
            specs += [ParamSpec("q_norm", (self.n_q,), VECTOR, INIT_ONE_PLUS_NORMAL),
                      ParamSpec("k_norm", (self.n_k,), VECTOR, INIT_ONE_PLUS_NORMAL)]
        if self.head_temperature:
            specs.append(ParamSpec("temperature", (self.n_head,), VECTOR, INIT_ONE_PLUS_NORMAL))
        if self.learned_sink:
            specs.append(ParamSpec("sink", (self.n_head,), VECTOR))
        return specs

    def state_spec(self):
        from .base import StateSpec

        return StateSpec((self.state_floats,), torch.float32) if self.state_floats else None

    def prepare(self, dtype, device) -> None:
        Mixer.prepare(self, dtype, device)
        self.rotary.prepare(dtype, device)
        p = self.params
        q = p["q_weight"]
        w = torch.zeros(self.n_proj, self.width, dtype=q.dtype, device=q.device)
        at = 0
        for key in ("q_weight", "k_weight") + (() if self.values_are_keys else ("v_weight",)):
            n = p[key].shape[0]
            w[at:at + n] = p[key]
            p[key] = w[at:at + n]
            at += n
        self.w_qkv = w
        self._pad_out_weight()
        if self.out_scale != 1.0:
            self.w_out = self.w_out * self.out_scale
        self.conv_w = torch.cat([p["q_conv"], p["k_conv"]], 0).contiguous() if self.taps > 0 else None

    def reserve(self, workspace: Workspace, limits: StepLimits) -> None:
        super().reserve(workspace, limits)
        workspace.reserve("attention.conv32", limits.max_rows * _round_up(self.channels, 4), torch.float32)

    def forward(self, xn: torch.Tensor, x: torch.Tensor, ctx: StepContext, cache: Optional[KVCacheView],
                state: Optional[torch.Tensor], writes_cache: bool = True) -> None:
        if cache is None or not writes_cache:
            raise ValueError("span_attention needs a paged cache of its own")
        if self.state_floats and state is None:
            raise ValueError("span_attention: the convolution needs a state slot tensor")
        if isinstance(xn, ops.NormInput):
            xn = xn.materialise(ctx.n_rows)
        T, ws, p = ctx.n_rows, ctx.workspace, self.params
        proj = ws.get("attention.proj32", (ctx.max_rows, self.n_proj), torch.float32)
        ops.trace_scope(ctx.layer, "qkv")
        ops.linear(xn, self.w_qkv, None, proj, T)
        src, k_off = proj, self.n_q
        if self.taps > 0:
            src = ws.get("attention.conv32", (ctx.max_rows, _round_up(self.channels, 4)), torch.float32)
            ops.short_conv(proj, 0, self.channels, self.taps, self.conv_w, None, state, ctx, src, ops.ACT_NONE)
        # the values: the keys' own columns as they stand here, or the value projection's (which no convolution touches)
        v_src_off = k_off if self.values_are_keys else None
        q = ws.get("attention.q", (ctx.max_rows, self.q_dim), self.dtype)
        if v_src_off is None:
            if src is not proj:   # the value columns did not pass the convolution: they are read from the projection
                raise NotImplementedError("span_attention: a value projection beside a convolution on q and k")
            v_src_off = self.n_q + self.n_k
        ops.wide_norm_rope_append(src, (0, k_off, v_src_off), self.n_head, self.n_kv_head, self.key_dim, self.v_dim,
                                  p["q_norm"] if self.wide_norm else None, p["k_norm"] if self.wide_norm else None,
                                  self.eps, self.rotary.dims, self.rotary.freqs, ctx, q, cache.layer, cache.block_table)
        att = ws.get("attention.out", (ctx.max_rows, self.q_dim), self.dtype)
        plan = ctx.plans.get("causal_attention")
        if plan is None:
            plan = ctx.plans["causal_attention"] = AttentionPlan(ctx.host_entry_start, ctx.host_entry_pos0,
                                                                 device=x.device)
        extras = ops.AttnExtras(span=self.span, head_scale=p.get("temperature"), sinks=p.get("sink"))
        ops.attention(q, cache.layer, att, cache.block_table, ctx, self.n_head, self.scale, 0, plan,
                      sink=self.learned_sink, extras=extras)
        ops.trace_scope(ctx.layer, "attn_proj")
        ops.linear(att, self.w_out, None, x, T, residual=True)
