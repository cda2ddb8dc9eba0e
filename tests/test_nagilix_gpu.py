"""Nagilix on the GPU: every new kernel and every kernel option alone against plain torch in float64, every
mechanism alone as a one-layer model, and whole models through the step function, cut into steps every way, against
the plain implementation (tests/plain_nagilix.py).  Test weights are made so that faults show
(nagilix_util.write_model); where random values would still hide one (a key at the edge of a span, a token far
back), the test builds queries and keys, or the prompts, by hand."""
import json
import math
import random

import pytest
import torch

from nagilix_util import TOL, assert_close, config, moe, pair_layer, rel_err, row_errs, scan_layer, write_model
from test_mulavik_gpu import _paged, step_ctx, toks

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
DEV = "cuda"


# =============================================================================== kernels alone
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("S,C,gated", [(1, 40, False), (2, 264, True), (3, 100, True), (8, 48, False)])
def test_stream_copies_kernels_against_torch(S, C, gated, dtype):
    from nanoinfer_b200.kernels import ops

    torch.manual_seed(S * C)
    dt, T, R, eps = DT[dtype], 7, 9, 2e-5
    x = torch.randn(R, C, device=DEV) * 3
    in_w, out_w, mix = torch.rand(S, device=DEV) + 0.2, torch.randn(S, device=DEV), torch.randn(S, S, device=DEV)
    in2, w1, w2 = torch.rand(S, device=DEV) + 0.2, torch.rand(C, device=DEV) + 0.5, torch.rand(C, device=DEV) + 0.5
    rms = lambda v, w: v / torch.sqrt((v ** 2).mean(-1, keepdim=True) + eps) * w.double()
    copies = torch.full((S, R, C), 9.0, device=DEV)
    xn = torch.zeros(R, C, device=DEV, dtype=dt)
    ops.hyper_enter(x, copies, in_w, w1, eps, xn, T)
    tol = 2e-6 if dtype == "float32" else 1e-2
    want_n = rms(in_w.double().sum() * x[:T].double(), w1)
    assert float(((xn[:T].double() - want_n) / (want_n.abs() + 1)).abs().max()) < tol
    assert all(torch.equal(copies[s, :T], x[:T]) for s in range(S)) and float(copies[:, T:].min()) == 9.0
    # a sublayer's result back into the copies, with the next sublayer's input and the copies' sum
    copies[:, :T] = torch.randn(S, T, C, device=DEV)
    old = copies.clone()
    y0 = torch.randn(R, C, device=DEV) * 2
    y, gate = y0.clone(), torch.randn(R, C + 3, device=DEV) * 2
    total = torch.zeros(R, C, device=DEV)
    ops.hyper_update(copies, y, gate[:, :C] if gated else None, mix, out_w, eps, T, in_next=in2, w_next=w2, xn=xn, total=total)
    r = y0[:T].double() * (torch.sigmoid(gate[:T, :C].double()) if gated else 1.0)
    want = torch.stack([sum(mix[s, t].double() * old[s, :T].double() for s in range(S)) + out_w[t].double() * r
                        for t in range(S)])
    assert float((copies[:, :T].double() - want).abs().max()) < 1e-5
    assert torch.equal(copies[:, T:], old[:, T:]) and not y[:T].any() and torch.equal(y[T:], y0[T:])
    assert float((total[:T].double() - want.sum(0)).abs().max()) < 1e-5
    want_n = rms(sum(in2[s].double() * want[s] for s in range(S)), w2)
    assert float(((xn[:T].double() - want_n) / (want_n.abs() + 1)).abs().max()) < tol
    # without a next sublayer nothing else is written
    before = xn.clone()
    ops.hyper_update(copies, y, None, mix, out_w, eps, T)
    assert torch.equal(xn, before)


def _scan_reference(dtp, x, B, C, z, A_log, D, S):
    """One request's rows through Mamba's recurrence in float64; S [inner, N] is updated in place."""
    out = torch.zeros_like(x)
    A = -torch.exp(A_log)
    for t in range(x.shape[0]):
        dt = torch.nn.functional.softplus(dtp[t])
        S.copy_(torch.exp(dt[:, None] * A) * S + (dt * x[t])[:, None] * B[t][None, :])
        out[t] = (S @ C[t] + D * x[t]) * z[t] * torch.sigmoid(z[t])
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("inner,N", [(40, 1), (33, 5), (64, 16), (100, 24), (20, 70), (48, 130), (7, 256)])
def test_selective_scan_kernel_carries_its_state_in_the_slot(inner, N, dtype):
    from nanoinfer_b200.kernels import ops

    g = torch.Generator().manual_seed(inner + N)
    NP, s_off, n_slots = ops.selective_scan_padded(N), 8, 5
    state = torch.zeros(n_slots, s_off + inner * NP + 4, device=DEV)
    state[:, :s_off] = 3.0
    A_log, D = torch.rand(inner, N, generator=g) * 4 - 3, torch.randn(inner, generator=g)
    ref = {s: torch.zeros(inner, N, dtype=torch.float64) for s in range(n_slots)}
    tol = 3e-5 if dtype == "float32" else 1e-2
    for step, (rows, slots) in enumerate([([5, 1, 19], [3, 0, 4]), ([1, 1, 1], [4, 3, 0]), ([2, 30], [0, 1])]):
        T = sum(rows)
        mk = lambda c, s=1.0: torch.randn(T + 2, c, generator=g) * s
        dtp, x, z, bc = mk(inner + 4, 2.0), mk(inner), mk(inner + 1), mk(2 * N + 8)
        positions = [p for n in rows for p in range(n)]
        ctx = step_ctx(rows, positions, slots=slots, n_pad=2)
        out = torch.full((T + 2, inner + 2), 7.0, device=DEV, dtype=DT[dtype])
        ops.selective_scan(dtp.to(DEV), x.to(DEV), bc.to(DEV), 4, 4 + N, z.to(DEV), A_log.to(DEV).contiguous(), D.to(DEV),
                           state, s_off, ctx, inner, N, out)
        at = 0
        for n, s in zip(rows, slots):
            sl = slice(at, at + n)
            want = _scan_reference(dtp[sl, :inner].double(), x[sl].double(), bc[sl, 4:4 + N].double(),
                                   bc[sl, 4 + N:4 + 2 * N].double(), z[sl, :inner].double(), A_log.double(), D.double(), ref[s])
            got = out[sl, :inner].double().cpu()
            assert float(((got - want) / (want.abs() + 1)).abs().max()) < tol, (step, s)
            at += n
        assert float(out[T:].float().min()) == 7.0 and float(out[:, inner:].float().min()) == 7.0
        for s in range(n_slots):
            got = state[s, s_off:s_off + inner * NP].view(inner, NP).double().cpu()
            assert float((got[:, :N] - ref[s]).abs().max()) < 3e-5 * (1 + float(ref[s].abs().max()))
            assert not got[:, N:].any() and float(state[s, :s_off].min()) == 3.0


def _turn_halves(x, pos, dims, base):
    """x [n, heads, dim] float64."""
    if not dims:
        return x
    half = dims // 2
    ang = pos.double()[:, None] * base ** (-2.0 * torch.arange(half, dtype=torch.float64) / dims)
    c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], -1)


@pytest.mark.parametrize("H,dim,rot", [(3, 16, 16), (2, 24, 8), (1, 10, 0), (5, 64, 2)])
def test_halves_rotation_in_place_with_fixed_decays_against_torch(H, dim, rot):
    from nanoinfer_b200.kernels import ops

    torch.manual_seed(H * dim)
    T, base, ld = 9, 30000.0, 2 * H * dim + 12
    pos = torch.tensor([0, 1, 2, 77, 1023, 50001, 5, 6, 7], dtype=torch.int32, device=DEV)
    rows0 = torch.randn(T + 1, ld, device=DEV)
    rows, coef = rows0.clone(), torch.full((T + 1, H, 2), 5.0, device=DEV)
    freqs = (base ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)).to(DEV) if rot else None
    decay = torch.rand(H, device=DEV)
    q_off, k_off = 4, 4 + H * dim + 4
    ops.rope_halves(rows, q_off, k_off, H, dim, rot, freqs, pos, 0.37, T, decay, coef)
    want = rows0.double().cpu().clone()
    for off, mul in ((q_off, 1.0), (k_off, 0.37)):
        x = rows0[:T, off:off + H * dim].double().cpu().view(T, H, dim)
        want[:T, off:off + H * dim] = (_turn_halves(x, pos.cpu(), rot, base) * mul).reshape(T, H * dim)
    assert float((rows.double().cpu() - want).abs().max()) < 2e-6
    assert torch.equal(coef[:T, :, 0], decay.expand(T, H)) and float(coef[:T, :, 1].min()) == 1.0 and float(coef[T:].min()) == 5.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,dim,hd,rot,norm,own_values", [(4, 2, 16, 16, 8, True, False), (3, 1, 24, 32, 24, True, False),
                                                             (2, 2, 12, 16, 0, False, False), (5, 5, 64, 64, 32, True, True)])
def test_wide_norm_rotation_cast_and_cache_write_against_torch(H, G, dim, hd, rot, norm, own_values, dtype):
    from nanoinfer_b200.kernels import ops

    torch.manual_seed(H + dim)
    dt, page, eps, base = DT[dtype], 16, 3e-5, 9000.0
    rows, positions = [5, 1, 3], [0, 1, 2, 3, 4, 40, 14, 15, 16]
    ctx = step_ctx(rows, positions, n_pad=2)
    T = ctx.n_rows
    nq, nk = H * dim, G * dim
    v_off = nq + nk if own_values else nq
    src = torch.randn(T, nq + 2 * nk + 4, device=DEV) * 2
    wq, wk = (torch.rand(nq, device=DEV) + 0.5, torch.rand(nk, device=DEV) + 0.5) if norm else (None, None)
    table = torch.tensor([[3, -1, -1], [5, 0, 4], [2, 1, -1]], dtype=torch.int32, device=DEV)
    cache = torch.full((6, 2, G, page, hd), 9.0, device=DEV, dtype=dt)
    q_out = torch.full((T, H * hd + 8), 7.0, device=DEV, dtype=dt)
    freqs = (base ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)).to(DEV) if rot else None
    ops.wide_norm_rope_append(src, (0, nq, v_off), H, G, dim, dim, wq, wk, eps, rot, freqs, ctx, q_out[:, :H * hd], cache, table)
    assert int(ctx.status.item()) == 0
    s = src.double().cpu()
    rms = lambda v, w: v / torch.sqrt((v ** 2).mean(-1, keepdim=True) + eps) * w.double().cpu() if w is not None else v
    pos = torch.tensor(positions + [0, 0])
    q = _turn_halves(rms(s[:, :nq], wq).view(T, H, dim), pos, rot, base)
    k = _turn_halves(rms(s[:, nq:nq + nk], wk).view(T, G, dim), pos, rot, base)
    v = s[:, v_off:v_off + nk].view(T, G, dim)
    tol = 3e-6 if dtype == "float32" else 1e-2
    close = lambda a, b: float(((a.double().cpu() - b) / (b.abs() + 1)).abs().max()) < tol
    got_q = q_out[:, :H * hd].view(T, H, hd)
    assert close(got_q[..., :dim], q) and not got_q[..., dim:].any() and float(q_out[:, H * hd:].float().min()) == 7.0
    entry = [e for e, n in enumerate(rows) for _ in range(n)]
    written = set()
    for t, (e, p) in enumerate(zip(entry, positions)):
        pg, slot = int(table[e, p // page]), p % page
        written.add((pg, slot))
        assert close(cache[pg, 0, :, slot, :dim], k[t]) and close(cache[pg, 1, :, slot, :dim], v[t])
        assert not cache[pg, :, :, slot, dim:].any()
    for pg in range(6):
        for slot in range(page):
            if (pg, slot) not in written:
                assert float(cache[pg, :, :, slot].float().min()) == 9.0


def _span_attention(q, k, v, scale, pos0, span=0, temps=None, sinks=None):
    """q [n, H, d], k, v [m, G, d]: row i stands at position pos0 + i and sees key j <= its position of its own span
    of positions; the denominator has exp(sinks[h]) more.  float64."""
    H, G = q.shape[1], k.shape[1]
    out = torch.zeros(q.shape[0], H, v.shape[2], dtype=torch.float64)
    j = torch.arange(k.shape[0])
    for h in range(H):
        s = (q[:, h].double() @ k[:, h // (H // G)].double().T) * scale * (float(temps[h]) if temps is not None else 1.0)
        for i in range(q.shape[0]):
            p = pos0 + i
            see = (j <= p) & ((j // span == p // span) if span else torch.ones_like(j, dtype=torch.bool))
            e = torch.exp(s[i][see] - s[i][see].max())
            den = e.sum() + (math.exp(float(sinks[h]) - float(s[i][see].max())) if sinks is not None else 0.0)
            out[i, h] = (e / den) @ v[see, h // (H // G)].double()
    return out


SPAN_SETS = {
    "spans of 64": dict(span=64),
    "spans of 24, a temperature and a sink": dict(span=24, temps=True, sinks=True),
    "spans of 100 and a sink": dict(span=100, sinks=True),
    "spans of one position": dict(span=1, sinks=True, temps=True),
    "all keys, a temperature and a sink": dict(temps=True, sinks=True),
    "spans longer than any request": dict(span=4096, temps=True),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hd,n_head,n_kv_head", [(64, 4, 1), (32, 3, 1), (48, 4, 2), (128, 2, 2), (144, 2, 1)])
@pytest.mark.parametrize("name", list(SPAN_SETS))
def test_attention_kernels_with_spans_temperatures_and_sinks(name, hd, n_head, n_kv_head, dtype):
    """Portions and single tokens side by side through the dispatcher (the tcgen05, the warp-MMA or the general kernel
    for portions, the streaming one for single tokens), then the streaming kernel with the keys split every way."""
    from nanoinfer_b200.kernels import ops
    from nanoinfer_b200.parts.attention import AttentionPlan

    o = dict(SPAN_SETS[name])
    dt, page, scale = DT[dtype], 16, 1.2 / math.sqrt(hd)
    span = o.get("span", 0)
    temps = torch.tensor([0.5 + 0.6 * h for h in range(n_head)]) if o.get("temps") else None
    sinks = torch.tensor([2.0 - 1.5 * h for h in range(n_head)]) if o.get("sinks") else None
    tol = 3e-5 if dtype == "float32" else 2e-2

    def run(lengths, q_rows, seed, direct_splits=None):
        cache, table, ks, vs, qs = _paged(dt, n_head, n_kv_head, hd, page, lengths, q_rows, seed=seed)
        positions = [p for n, r in zip(lengths, q_rows) for p in range(n - r, n)]
        ctx = step_ctx(q_rows, positions)
        T = ctx.n_rows
        want = torch.cat([_span_attention(qq, k, v, scale, n - r, span, temps, sinks)
                          for qq, k, v, n, r in zip(qs, ks, vs, lengths, q_rows)])
        q = torch.cat(qs).view(-1, n_head * hd).to(dt).to(DEV)
        ex = ops.AttnExtras(span=span, head_scale=temps.to(DEV) if temps is not None else None,
                            sinks=sinks.to(DEV) if sinks is not None else None)
        cache_d, table_d = cache.to(dt).to(DEV), table.to(DEV)
        out = torch.full_like(q, 7.0)
        if direct_splits is None:
            plan = AttentionPlan(ctx.host_entry_start, ctx.host_entry_pos0, device=torch.device(DEV))
            ops.attention(q, cache_d, out, table_d, ctx, n_head, scale, 0, plan, sink=sinks is not None, extras=ex)
        else:
            keys = min(max(lengths), span) if span else max(lengths)
            chunk = max(16, -(-(-(-keys // direct_splits)) // 16) * 16)
            n_splits = -(-keys // chunk)
            scratch = torch.zeros(ops.DECODE_RESIDENT_BLOCKS * (hd + 2), device=DEV)
            counters = torch.zeros(ops.DECODE_RESIDENT_BLOCKS, dtype=torch.int32, device=DEV)
            code = ops.library().nib_attention_decode(
                0 if dtype == "float32" else 1, q.data_ptr(), q.stride(0), cache_d.data_ptr(), scratch.data_ptr(),
                out.data_ptr(), out.stride(0), table_d.data_ptr(), table_d.shape[1], None, ctx.row_entry.data_ptr(),
                ctx.positions.data_ptr(), T, n_head, n_kv_head, hd, page, cache_d.shape[0], scale, 0,
                int(sinks is not None), *ex.args(), chunk, n_splits, counters.data_ptr(), ctx.status.data_ptr(),
                torch.cuda.current_stream().cuda_stream)
            assert code == 0
        assert int(ctx.status.item()) == 0
        diff = float((out.double().cpu().view(want.shape) - want).abs().max())
        assert diff < tol, f"{name}, splits {direct_splits}: {diff:.3e}"
        return want

    lengths, q_rows = [200, 77, 450, 130, 16, 3, 333], [130, 1, 1, 40, 16, 1, 290]
    with_options = run(lengths, q_rows, seed=hd)
    if hd <= 128:
        for ns in (1, 2, 3, 5, 16):
            run([450, 77, 300, 2, 40, 65, 64], [1] * 7, seed=hd + 1, direct_splits=ns)
    if name != "spans longer than any request":
        cache, table, ks, vs, qs = _paged(dt, n_head, n_kv_head, hd, page, lengths, q_rows, seed=hd)
        plain = torch.cat([_span_attention(qq, k, v, scale, n - r) for qq, k, v, n, r in zip(qs, ks, vs, lengths, q_rows)])
        assert float((plain - with_options).abs().max()) > 20 * tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows", [1, 2, 40, 150])
@pytest.mark.parametrize("span", [16, 24, 64, 100])
def test_one_matching_key_just_inside_and_just_outside_a_span(span, rows, dtype):
    """All keys but one are orthogonal to the query; the one that matches carries a value of its own.  It shows in a
    row's output exactly when it lies in the row's span, for the last row of a portion and for single tokens, with
    the span's edge anywhere in a page or a tile."""
    from nanoinfer_b200.kernels import ops
    from nanoinfer_b200.parts.attention import AttentionPlan

    dt, hd, page, n = DT[dtype], 64, 16, 3 * span + 7 + rows
    for far in (n - 1, n - 2, (n - 1) // span * span, (n - 1) // span * span - 1, (n - 1) // span * span + 1, 0, span - 1, span):
        if far < 0 or far > n - 1:
            continue
        k = torch.zeros(n, 1, hd)
        k[:, 0, 1] = 1.0
        k[far, 0, 0] = 30.0
        v = torch.zeros(n, 1, hd)
        v[:, 0, 1] = 1.0
        v[far, 0, :] = 0.0
        v[far, 0, 2] = 1.0
        q = torch.zeros(rows, 2, hd)
        q[:, :, 0] = 1.0
        nb = -(-n // page)
        perm = torch.randperm(nb, generator=torch.Generator().manual_seed(far)).tolist()
        cache = torch.zeros(nb, 2, 1, page, hd)
        for b in range(nb):
            m = min(page, n - b * page)
            cache[perm[b], 0, 0, :m] = k[b * page:b * page + m, 0]
            cache[perm[b], 1, 0, :m] = v[b * page:b * page + m, 0]
        table = torch.tensor([perm], dtype=torch.int32, device=DEV)
        ctx = step_ctx([rows], list(range(n - rows, n)))
        out = torch.zeros(rows, 2 * hd, device=DEV, dtype=dt)
        plan = AttentionPlan(ctx.host_entry_start, ctx.host_entry_pos0, device=torch.device(DEV))
        ops.attention(q.view(rows, -1).to(dt).to(DEV), cache.to(dt).to(DEV), out, table, ctx, 2, 1.0, 0, plan,
                      extras=ops.AttnExtras(span=span))
        for i in (0, rows - 1):
            p = n - rows + i
            visible = far <= p and far // span == p // span
            found = float(out[i, 2]) > 0.9
            assert found == visible, f"key {far}, row at {p}: visible {visible}, found {found}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,J,top,bias", [(6, 2, 3, True), (4, 0, 1, True), (5, 3, 8, False), (1, 1, 1, True), (9, 1, 2, True)])
def test_routing_with_a_correction_and_experts_that_hand_their_input_on(E, J, top, bias, dtype):
    from nanoinfer_b200.kernels import ops

    torch.manual_seed(E * 10 + J)
    dt, T, C = DT[dtype], 23, 40
    h = torch.randn(T + 1, C, device=DEV).to(dt)
    wr = (torch.randn(E + J, C, device=DEV) * 0.5).to(dt)
    corr = torch.randn(E + J, device=DEV) * 0.3 if bias else None
    ids = torch.full((T + 1, top), 77, dtype=torch.int32, device=DEV)
    w = torch.full((T + 1, top), 7.0, device=DEV)
    x0 = torch.randn(T + 1, C, device=DEV)
    x = x0.clone()
    ops.moe_route(h, wr, T, top, False, ids, w, choice_bias=corr, n_real=E, x=x)
    s = torch.softmax(h[:T].double() @ wr.double().T, -1)
    pick = torch.topk(s + (corr.double() if bias else 0.0), top, -1).indices
    want_ids = torch.where(pick < E, pick, torch.full_like(pick, -1))
    assert torch.equal(ids[:T].long().cpu(), want_ids.cpu()) and int(ids[T, 0]) == 77
    assert float((w[:T].double() - s.gather(1, pick)).abs().max()) < 2e-6
    handed = (s.gather(1, pick) * (pick >= E)).sum(-1, keepdim=True)
    assert float((x[:T].double() - (x0[:T].double() + handed * h[:T].double())).abs().max()) < 1e-5
    assert torch.equal(x[T], x0[T])
    if bias and E >= 6:
        assert not torch.equal(pick, torch.topk(s, top, -1).indices)       # (the correction moves choices here)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,E,top", [(3, 5, 2), (70, 4, 3), (300, 20, 2), (90, 3, 2)])
def test_capped_gated_experts_every_way_with_choices_that_are_skipped(T, E, top, dtype):
    """Row by row (few rows), expert by expert (many rows, many experts) and all experts at once (many rows, few
    experts): the capped gated unit, and choices without matrices (id -1) left out."""
    from nanoinfer_b200.kernels import ops
    from nanoinfer_b200.parts.base import Workspace

    torch.manual_seed(T + E)
    dt, C, F, limit = DT[dtype], 48, 24, 0.7
    h = (torch.randn(T, C, device=DEV)).to(dt)
    w_gate, w_val = torch.randn(E, F, C, device=DEV) * 0.3, torch.randn(E, F, C, device=DEV) * 0.3
    w_up = torch.stack([w_gate, w_val], 2).reshape(E, 2 * F, C).to(dt).contiguous()
    w_down = (torch.randn(E, C, F, device=DEV) * 0.3).to(dt).contiguous()
    ids = torch.stack([torch.randperm(E + 2, device=DEV)[:top] for _ in range(T)]).int()
    ids = torch.where(ids < E, ids, torch.full_like(ids, -1)).contiguous()
    ids[0, 0] = -1
    weights = torch.rand(T, top, device=DEV)
    x0 = torch.randn(T, C, device=DEV)
    x, ws = x0.clone(), Workspace(torch.device(DEV))
    inner = torch.zeros(T * top, F, device=DEV, dtype=dt)
    ops.moe_experts(h, w_up, w_down, ids, weights, inner, x, T, top, ops.ACT_SWIGLU_CAPPED, ws, gated=True, act_prm=limit)
    want = x0.double().clone()
    hd_ = h.double()
    for t in range(T):
        for k in range(top):
            e = int(ids[t, k])
            if e < 0:
                continue
            g = torch.clamp(w_up[e, 0::2].double() @ hd_[t], max=limit)
            u = torch.clamp(w_up[e, 1::2].double() @ hd_[t], -limit, limit)
            y = g * torch.sigmoid(1.702 * g) * (u + 1.0)
            if dtype == "bfloat16":
                y = y.to(torch.bfloat16).double()        # the first product's result is stored in the engine's dtype
            want[t] += float(weights[t, k]) * (w_down[e].double() @ y)
    tol = 1e-4 if dtype == "float32" else 3e-2
    assert float(((x.double() - want) / (want.abs() + 1)).abs().max()) < tol
    assert int((ids < 0).sum()) > 0


# =============================================================================== models through the step function
class Harness:
    def __init__(self, cfg, tmp_path, dtype, max_tokens=512, slots=4, page=16, max_rows=256, seed=1, sharpen=3.0,
                 long_memory=False):
        from nanoinfer_b200 import load_model
        from nanoinfer_b200.cache import CacheManager
        from nanoinfer_b200.engine import ModelRunner
        from plain_nagilix import PlainNagilix

        self.dir = write_model(cfg, str(tmp_path), DT[dtype], seed=seed, sharpen=sharpen, long_memory=long_memory)
        self.plain = PlainNagilix(self.dir)
        self.model = load_model(self.dir, DT[dtype], DEV)
        self.cache = CacheManager(self.model.kv_needs(), self.model.state_needs(), max_tokens=max_tokens,
                                  max_requests=slots, page_size=page, dtype=DT[dtype], device=torch.device(DEV),
                                  max_positions=self.model.max_positions, padding=True)
        self.runner = ModelRunner(self.model, self.cache, max_rows=max_rows, max_entries=slots, check_status=True)
        self.dtype, self.vocab = dtype, cfg["vocab"]

    def alone(self, tokens, cuts):
        """One request cut into portions of the sizes in ``cuts`` (cycled), all logits back."""
        from nanoinfer_b200.engine import StepItem

        r, at, k, rows = self.cache.open_request(), 0, 0, []
        while at < len(tokens):
            n = min(cuts[k % len(cuts)], len(tokens) - at)
            rows.append(self.runner.step([StepItem(r, tokens[at:at + n], list(range(n)))]).clone())
            at, k = at + n, k + 1
        self.cache.close_request(r)
        return torch.cat(rows)

    def check(self, got, tokens, what=""):
        assert_close(row_errs(got, self.plain.logits(tokens)), self.dtype, what)


ONE_LAYER = {
    "selective scan": [scan_layer()],
    "selective scan, a state of one value, two taps": [scan_layer(inner=24, state=1, dt_rank=1, conv=2)],
    "selective scan, a state of 70 values, one tap": [scan_layer(inner=33, state=70, dt_rank=9, conv=1)],
    "selective scan, a wide step-size product": [scan_layer(inner=64, state=16, dt_rank=40, conv=5)],
    "spans beside retention": [pair_layer()],
    "spans beside retention, one key head, spans of 7, all of a head turned": [pair_layer(heads=3, kv_heads=1, dim=12, span=7, rot=12,
                                                                                        r_heads=1, r_dim=32, r_vdim=8, r_rot=32)],
    "spans beside retention, every head its own keys, no convolution": [pair_layer(heads=2, kv_heads=2, dim=64, conv=0, span=33,
                                                                                  rot=2, r_heads=4, r_dim=16, r_vdim=16, r_rot=0)],
    "all keys beside retention, nothing turned, two taps": [pair_layer(heads=4, kv_heads=1, dim=32, conv=2, span=0, rot=0,
                                                                      r_heads=2, r_dim=20, r_vdim=36, r_rot=4, decay=[1.0, 0.5])],
    "spans of one position": [pair_layer(span=1, conv=5)],
    "routed experts": [scan_layer(mlp=moe())],
    "routed experts, one of one and one that hands its input on": [scan_layer(mlp=moe(experts=1, identity=1, top=1, ff=8))],
    "routed experts, all with matrices, all chosen": [pair_layer(mlp=moe(experts=3, identity=0, top=3, ff=40, limit=0.3))],
    "routed experts, more handed on than computed": [scan_layer(mlp=moe(experts=2, identity=4, top=4, ff=16, limit=5.0))],
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(ONE_LAYER))
def test_each_mechanism_alone_as_a_one_layer_model(name, dtype, tmp_path):
    h = Harness(config(ONE_LAYER[name], vocab=150, width=48), tmp_path, dtype)
    t = toks(150, 75, 3)
    h.check(h.alone(t, [1000]), t, name)
    h.check(h.alone(t, [40, 1, 1, 2, 3, 1]), t, name + " in portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("what", ["one copy of the stream", "eight copies", "an odd vocabulary and width, no constant on the logits"])
def test_the_parts_around_the_layers(what, dtype, tmp_path):
    layers = [scan_layer(mlp=moe()), pair_layer(mlp=None), scan_layer(mlp=None)]
    cfg = {"one copy of the stream": config(layers, vocab=90, width=40, streams=1),
           "eight copies": config(layers, vocab=90, width=40, streams=8, logit_scale=0.3),
           "an odd vocabulary and width, no constant on the logits": config(layers, vocab=131, width=36, eps=3e-4, logit_scale=1.0)}[what]
    if "odd" in what:
        del cfg["logit_scale"], cfg["streams"]
    h = Harness(cfg, tmp_path, dtype)
    t = toks(cfg["vocab"], 50, 6)
    h.check(h.alone(t, [1000]), t, what)
    h.check(h.alone(t, [30, 1, 2]), t, what + " in portions")


FULL = [scan_layer(inner=56, state=16, dt_rank=6, conv=4, mlp=moe(experts=6, identity=2, top=3, ff=32)),
        pair_layer(mlp=moe(experts=4, identity=1, top=2, ff=24)),
        pair_layer(heads=2, kv_heads=1, dim=32, conv=2, span=40, rot=16, r_heads=4, r_dim=16, r_vdim=8, mlp=None),
        scan_layer(inner=40, state=24, dt_rank=3, conv=2, mlp=None),
        pair_layer(heads=4, kv_heads=4, dim=16, conv=4, span=17, rot=16, r_heads=2, r_dim=24, r_vdim=24, r_rot=24,
                   mlp=moe(experts=3, identity=0, top=1, ff=48))]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_token_by_token_and_portions_agree(dtype, tmp_path):
    h = Harness(config(FULL, vocab=190, width=64, eps=1e-6), tmp_path, dtype)
    t = toks(190, 97, 5)
    whole = h.alone(t, [1000])
    h.check(whole, t, "whole")
    ways = {"one by one": [1], "portions of two": [2], "3 and 5": [3, 5], "17, 16, 1, 31": [17, 16, 1, 31],
            "most of it, then single tokens": [60] + [1] * 40}
    for what, cuts in ways.items():
        got = h.alone(t, cuts)
        h.check(got, t, what)
        if dtype == "float32":     # how the prompt was cut shows in rounding only
            assert rel_err(got, whole) < 2e-5, what
    assert h.runner.graph_replays > 50            # single tokens ran as replayed graphs, states and all
    assert h.cache.pages_used() == [0] * len(h.cache.groups)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_requests_together_equal_each_alone_and_pages_and_slots_come_back(dtype, tmp_path):
    from nanoinfer_b200.engine import StepItem

    h = Harness(config(FULL, vocab=170, width=64), tmp_path, dtype, max_tokens=4 * 64, slots=3)
    lens = [3, 120, 41, 64, 17, 88, 1]
    prompts = [toks(170, n, 20 + i) for i, n in enumerate(lens)]
    cuts = [[3], [50, 1, 1, 30, 2], [1, 40], [16, 16, 1], [17], [2, 2, 2, 80, 1], [1]]
    waiting, live, got = list(range(len(lens))), {}, {i: [] for i in range(len(lens))}
    slot_users, page_users, tick = {}, {}, 0
    while waiting or live:
        while waiting and len(live) < 3:
            i = waiting.pop(0)
            live[i] = [h.cache.open_request(), 0, 0]
            slot_users.setdefault(live[i][0].slot, set()).add(i)
        items, meta = [], []
        for j, (i, (req, at, k)) in enumerate(list(live.items())):
            if (tick + j) % 4 == 3 and len(live) > 1:
                continue                                   # sits this step out and goes on later
            n = min(cuts[i][k % len(cuts[i])], lens[i] - at)
            if not h.cache.can_append([(it.request, len(it.tokens)) for it in items] + [(req, n)]):
                continue
            items.append(StepItem(req, prompts[i][at:at + n], list(range(n))))
            meta.append((i, n))
        tick += 1
        if not items:
            continue
        out = h.runner.step(items)
        row = 0
        for i, n in meta:
            got[i].append(out[row:row + n].clone())
            row += n
            live[i][1] += n
            live[i][2] += 1
            for g, blocks in enumerate(live[i][0].blocks):
                for p in blocks:
                    if p >= 0:
                        page_users.setdefault((g, p), set()).add(i)
            if live[i][1] == lens[i]:
                h.cache.close_request(live[i][0])
                del live[i]
        h.cache.check()
    for i, t in enumerate(prompts):
        h.check(torch.cat(got[i]), t, f"request {i}")
    assert max(len(u) for u in slot_users.values()) >= 2 and max(len(u) for u in page_users.values()) >= 2
    assert h.cache.pages_used() == [0] * len(h.cache.groups) and h.cache.slots.n_free == 3


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_lengths_around_page_and_span_edges_and_the_first_tokens(dtype, tmp_path):
    layers = [pair_layer(span=16, mlp=None), scan_layer(mlp=None), pair_layer(heads=2, kv_heads=1, dim=16, span=17, mlp=None)]
    h = Harness(config(layers, vocab=120, width=40), tmp_path, dtype, sharpen=4.0)
    for n in (1, 2, 3, 15, 16, 17, 18, 31, 32, 33, 34, 47, 48, 49, 51):
        t = toks(120, n + 3, n)
        h.check(h.alone(t, [n, 1, 1, 1]), t, f"{n} tokens, then three alone")
        h.check(h.alone(t, [1, 1, 1, n]), t, f"three alone, then {n}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_spans_and_states(dtype, tmp_path):
    from nanoinfer_b200.engine import StepItem

    layers = [scan_layer(mlp=moe()), pair_layer(span=40, mlp=moe(top=2)), pair_layer(span=64, conv=4, mlp=None)]
    h = Harness(config(layers, vocab=100, width=48), tmp_path, dtype, max_tokens=384, slots=2)
    t = toks(100, 330, 9)
    r = h.cache.open_request()
    rows = [h.runner.step([StepItem(r, t[:5], list(range(5)))]).clone()]
    for p in range(5, len(t)):
        rows.append(h.runner.step([StepItem(r, t[p:p + 1], [0])]).clone())
    h.cache.close_request(r)
    h.check(torch.cat(rows), t, "330 positions")
    assert h.runner.graph_replays > 300


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_long_prompts_through_the_tiled_prompt_kernels(dtype, tmp_path):
    """Heads of 64 (the tcgen05 prompt kernel in bfloat16) and of 128 and 32 (the warp-MMA one) over prompts of
    several tiles of keys: spans that end in the middle of a tile and of a page, spans longer than the prompt; whole, in
    portions that start anywhere, and with the last tokens one by one."""
    layers = [pair_layer(heads=4, kv_heads=2, dim=64, span=150, rot=32, mlp=moe()),
              pair_layer(heads=2, kv_heads=1, dim=64, span=64, rot=64, r_heads=2, r_dim=16, r_vdim=16, mlp=None),
              pair_layer(heads=2, kv_heads=1, dim=128, span=129, rot=16, mlp=None),
              pair_layer(heads=3, kv_heads=3, dim=32, span=2000, rot=8, r_heads=1, r_dim=8, r_vdim=8, conv=2, mlp=None),
              scan_layer(mlp=None)]
    # (16-bit rounding at a sequence's first positions, where a retention head's output is a single term over its own
    # root mean square, is amplified from layer to layer: in bfloat16 the stack is run as two shorter ones)
    stacks = [layers] if dtype == "float32" else [layers[:2], layers[2:]]
    tokens = toks(150, 590, 77)
    for k, stack in enumerate(stacks):
        h = Harness(config(stack, vocab=150, width=64, max_positions=700), tmp_path / str(k), dtype, max_tokens=1216,
                    slots=2, max_rows=640, seed=5)
        h.check(h.alone(tokens, [590]), tokens, "whole")
        h.check(h.alone(tokens, [333, 2, 131, 100] + [1] * 24), tokens, "in portions")
        assert h.cache.pages_used() == [0] * len(h.cache.groups)


def test_a_token_far_back_shows_through_the_states(tmp_path):
    """A scan whose rates let it remember for hundreds of tokens, and retention with decays next to 1 beside an
    attention that sees a few positions only: two prompts that differ in their first twelve tokens only still differ 150
    tokens on, and the engine follows the plain model in both."""
    for layers in ([scan_layer(inner=48, state=16)], [pair_layer(span=4, decay=[0.999, 1.0, 0.99])]):
        cfg = config(layers, vocab=90, width=64, max_positions=200)
        h = Harness(cfg, tmp_path, "float32", long_memory=True, sharpen=6.0)
        a = toks(90, 150, 4)
        b = [(v + 1) % 90 for v in a[:12]] + a[12:]
        la, lb = h.plain.logits(a)[-1], h.plain.logits(b)[-1]
        assert rel_err(la[None], lb[None]) > 5 * TOL["float32"], layers[0]["type"]
        for t in (a, b):
            h.check(h.alone(t, [120, 7, 1]), t)


def random_config(rnd):
    width = rnd.choice([32, 40, 64, 72, 96, 100])
    layers = []
    for _ in range(rnd.randint(1, 5)):
        mlp = None
        if rnd.random() < 0.6:
            e, j = rnd.randint(1, 7), rnd.randint(0, 3)
            mlp = moe(experts=e, identity=j, top=rnd.randint(1, e + j), ff=rnd.choice([8, 20, 32, 56]),
                      limit=rnd.choice([0.3, 1.0, 7.0]))
        if rnd.random() < 0.45:
            layers.append(scan_layer(inner=rnd.choice([16, 24, 50, 96]), state=rnd.choice([1, 4, 9, 16, 24, 40]),
                                     dt_rank=rnd.choice([1, 4, 8, 13]), conv=rnd.randint(1, 5), mlp=mlp))
        else:
            g = rnd.choice([1, 2, 3])
            dim = rnd.choice([8, 16, 24, 32, 64])
            r_dim, r_heads = rnd.choice([8, 12, 16, 40]), rnd.randint(1, 4)
            layers.append(pair_layer(heads=g * rnd.choice([1, 2]), kv_heads=g, dim=dim, scale=rnd.choice([None, 0.2, 0.05]),
                                     conv=rnd.choice([0, 1, 2, 4]), span=rnd.choice([0, 1, 5, 16, 31, 64, 300]),
                                     rot=rnd.choice([0, 2, dim // 2, dim]), base=rnd.choice([100.0, 10000.0, 1e6]),
                                     r_heads=r_heads, r_dim=r_dim, r_vdim=rnd.choice([4, 16, 33]),
                                     decay=[rnd.choice([0.5, 0.9, 0.96875, 0.999, 1.0]) for _ in range(r_heads)],
                                     r_rot=rnd.choice([0, 2, r_dim]), r_base=rnd.choice([50.0, 1e5]), mlp=mlp))
    return config(layers, vocab=rnd.choice([50, 131, 256]), width=width, streams=rnd.randint(1, 4),
                  eps=rnd.choice([1e-6, 1e-5, 1e-3]), logit_scale=rnd.choice([0.5, 1.0, 2.0]), max_positions=200)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", range(12))
def test_random_configuration_cut_at_random(case, dtype, tmp_path):
    from nanoinfer_b200.engine import StepItem

    rnd = random.Random(9100 + case)
    cfg = random_config(rnd)
    page = rnd.choice([16, 32, 48])
    lens = [rnd.randint(1, 150) for _ in range(rnd.randint(2, 6))]
    pages_of = lambda n: -(-n // page)
    pages = max(max(pages_of(n) for n in lens) + 2, int(0.6 * sum(pages_of(n) for n in lens)))
    h = Harness(cfg, tmp_path, dtype, max_tokens=pages * page, slots=3, page=page, max_rows=rnd.choice([64, 160]),
                seed=case + 1, sharpen=rnd.choice([2.0, 4.0]))
    prompts = [[rnd.randrange(cfg["vocab"]) for _ in range(n)] for n in lens]
    pending, live, got = list(range(len(lens))), {}, {}
    while pending or live:
        while pending and len(live) < 3:
            live[pending.pop(0)] = [h.cache.open_request(), 0]
        items, meta, rows = [], [], 0
        for i, (req, at) in list(live.items()):
            if rnd.random() < 0.2 and len(live) > 1:
                continue
            n = min(lens[i] - at, rnd.choice([1, 1, 2, 3, 7, 16, 17, 33, 64, 100]), h.runner.max_rows - rows)
            if n <= 0 or not h.cache.can_append([(it.request, len(it.tokens)) for it in items] + [(req, n)]):
                continue
            places = sorted(rnd.sample(range(n), min(n, rnd.randint(0, 3))))
            items.append(StepItem(req, prompts[i][at:at + n], places))
            meta.append((i, at, n, places))
            rows += n
        if not items:
            # nothing fits beside what is held: the newest request gives way and starts again later
            i = max(live)
            h.cache.close_request(live.pop(i)[0])
            pending.insert(0, i)
            got = {k: v for k, v in got.items() if k[0] != i}
            continue
        out = h.runner.step(items)
        k = 0
        for i, at, n, places in meta:
            for j in places:
                got[(i, at + j)] = out[k].clone()
                k += 1
            live[i][1] = at + n
            if at + n == lens[i]:
                h.cache.close_request(live.pop(i)[0])
    h.cache.check()
    assert got and h.cache.pages_used() == [0] * len(h.cache.groups)
    want = [h.plain.logits(t) for t in prompts]
    keys = sorted(got)
    errs = row_errs(torch.stack([got[k] for k in keys]), torch.stack([want[i][p] for i, p in keys]))
    assert_close(errs, dtype, f"case {case} {json.dumps(cfg)} at (request, position) {keys}")


def test_greedy_generation_through_the_engine_and_its_scheduler(tmp_path):
    import nanoinfer_b200 as nb
    from plain_nagilix import PlainNagilix

    cfg = config(FULL, vocab=130, width=64)
    d = write_model(cfg, str(tmp_path), torch.float32, seed=3)
    plain = PlainNagilix(d)
    prompts = [toks(130, n, 40 + n) for n in (1, 9, 30, 55, 17)]
    eng = nb.Engine(d, dtype="float32", max_tokens=3 * 128, max_batch=3, max_rows=64)
    outs = eng.generate(prompts, nb.SamplingParams(max_new_tokens=20))
    for p, o in zip(prompts, outs):
        assert o == plain.greedy(p, 20)
    assert eng.runner.graph_replays > 0 and eng.cache.pages_used() == [0] * len(eng.cache.groups)


def test_trace_replay_of_a_model_folder(tmp_path):
    from plain_nagilix import PlainNagilix
    from trace_util import TraceSession

    cfg = config(FULL[:4], vocab=110, width=48)
    d = write_model(cfg, str(tmp_path / "m"), torch.float32, seed=8)
    plain = PlainNagilix(d)
    reqs = {f"r{i}": toks(110, n, 60 + i) for i, n in enumerate((50, 3, 64, 20, 33, 9))}
    s = TraceSession(d, "float32", tmp_path / "out", 4 * 64, 110)
    order, live, at = list(reqs), [], {r: 0 for r in reqs}
    k = 0
    while order or live:
        while order and len(live) < 4:
            live.append(order.pop(0))
        entries, ended = [], []
        for r in list(live):
            n = min([7, 1, 20, 2][k % 4], len(reqs[r]) - at[r])
            k += 1
            entries.append((r, reqs[r][at[r]:at[r] + n], range(n)))
            at[r] += n
            if at[r] == len(reqs[r]):
                ended.append(r)
                live.remove(r)
        s.step(entries, end=ended)
    s.close()
    for r, t in reqs.items():
        assert rel_err(s.stacked(r, len(t)), plain.logits(t)) <= TOL["float32"], r


def test_command_line_writes_a_folder_generates_from_it_and_profiles(tmp_path, capsys):
    from nanoinfer_b200 import cli
    from plain_nagilix import PlainNagilix

    d = str(tmp_path / "m")
    assert cli.main(["random-weights", "--config", "nagilix-tiny", "--seed", "6", "--out", d, "--dtype", "float32"]) == 0
    capsys.readouterr()
    prompt = toks(512, 12, 77)
    assert cli.main(["--weights", d, "generate", "--dtype", "float32", "--prompt-ids", ",".join(map(str, prompt)),
                     "--tokens", "10", "--temperature", "0.0", "--profile"]) == 0
    captured = capsys.readouterr()
    printed = [int(t) for t in captured.out.split()]
    assert printed == PlainNagilix(d).greedy(prompt, 10)
    assert "scan" in captured.err and "attn" in captured.err
