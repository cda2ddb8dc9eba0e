"""Kemuzen on the GPU: every new kernel and every kernel option alone against plain torch in float64, every
mechanism alone as a one-layer model, and whole models through the step function, cut into steps every way, against
the plain implementation (tests/plain_kemuzen.py).  Test weights are made so that faults show
(kemuzen_util.write_model); where random values would still hide one (a far key, the edge of a window, the kept
first tokens), the kernel test builds queries and keys by hand."""
import json
import math
import random

import pytest
import torch

from kemuzen_util import (TOL, assert_close, attention_layer, config, delta_layer, dense, parallel_layer, rel_err,
                          row_errs, write_model)
from test_mulavik_gpu import _paged, step_ctx, toks

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
DEV = "cuda"


def _cut(n, sizes):
    """n rows cut into portions of the sizes given (cycled)."""
    out, k = [], 0
    while n > 0:
        out.append(min(sizes[k % len(sizes)], n))
        n -= out[-1]
        k += 1
    return out


# =============================================================================== kernels alone
@pytest.mark.parametrize("C", [10, 64, 200])
def test_sinusoidal_positions_against_torch(C):
    from nanoinfer_b200.kernels import ops

    pos = torch.tensor([0, 1, 2, 17, 4095, 70001, 3], dtype=torch.int32, device=DEV)
    i = torch.arange((C + 1) // 2, dtype=torch.float64)
    freqs = 10000.0 ** (-2.0 * i / C)
    x0 = torch.randn(9, C, device=DEV)
    x = x0.clone()
    ops.add_sinusoid(x, pos, freqs.to(DEV), 7)
    ang = pos.cpu().double()[:, None] * freqs[None, :]
    want = x0[:7].double().cpu()
    want[:, 0::2] += torch.sin(ang)[:, :want[:, 0::2].shape[1]]
    want[:, 1::2] += torch.cos(ang)[:, :want[:, 1::2].shape[1]]
    assert float((x[:7].double().cpu() - want).abs().max()) < 1e-6 and torch.equal(x[7:], x0[7:])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_token_gate_kernel_against_torch(dtype):
    from nanoinfer_b200.kernels import ops

    torch.manual_seed(3)
    dt, T, D, off = DT[dtype], 11, 6, 12
    table = torch.randn(30, 24, device=DEV).to(dt)
    pre = torch.randn(T + 2, D + 2, device=DEV) * 2
    tok = torch.randint(0, 30, (T,), dtype=torch.int32, device=DEV)
    tok[4] = -3                                       # stands for feedback[2]
    feedback = torch.tensor([0, 0, 21], dtype=torch.int32, device=DEV)
    real = tok.clone()
    real[4] = 21
    z = pre[:T, :D].double()
    gelu = 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))
    want = gelu * table[real.long(), off:off + D].double()
    out = torch.zeros(T + 2, D + 1, device=DEV, dtype=dt)
    ops.gate_by_table(pre, tok, feedback, table, off, D, ops.ACT_GELU_TANH, out, T)
    tol = 1e-5 if dtype == "float32" else 0.02
    assert float(((out[:T, :D].double() - want) / (want.abs() + 1)).abs().max()) < tol
    assert not out[T:].any() and not out[:, D:].any()


def test_soft_cap_and_sum_with_cast_kernels_against_torch():
    from nanoinfer_b200.kernels import ops

    torch.manual_seed(5)
    z = torch.randn(7, 33, device=DEV) * 40
    cap = torch.tensor([13.0], device=DEV)
    out = z.clone()
    ops.unary(out, out, 5, ops.UNARY_SOFTCAP, cap)
    assert float((out[:5].double() - 13.0 * torch.tanh(z[:5].double() / 13.0)).abs().max()) < 1e-5
    assert torch.equal(out[5:], z[5:])
    # the norm of a sublayer's output summed into the stream, and the stream itself cast for the next sublayer
    for C in (40, 264):
        x0, y0, w = torch.randn(9, C, device=DEV) * 3, torch.randn(9, C, device=DEV) * 40, torch.rand(C, device=DEV) + 0.5
        want = x0.double() + y0.double() / torch.sqrt((y0.double() ** 2).mean(-1, keepdim=True) + 1e-5) * w.double()
        for dt in (torch.float32, torch.bfloat16):
            x, y, xn = x0.clone(), y0.clone(), torch.zeros(9, C, device=DEV, dtype=dt)
            ops.add_norm(x, y, w, 1e-5, 6, None, xn)
            assert float((x[:6] - want[:6]).abs().max()) < 1e-5 and torch.equal(x[6:], x0[6:]) and not y[:6].any()
            assert torch.equal(xn[:6], x[:6].to(dt)) and not xn[6:].any()


@pytest.mark.parametrize("taps,bias", [(1, False), (2, True), (4, False), (4, True), (5, True)])
def test_short_convolution_carries_its_inputs_in_the_slot(taps, bias):
    """Three requests of unequal lengths in shuffled slots, cut into portions down to single rows (where one kernel
    also moves the state on), against the convolution of each whole sequence."""
    from nanoinfer_b200.kernels import ops

    torch.manual_seed(taps)
    Cn, ld, c_off, lens, slots = 37, 64, 9, [23, 9, 41], [4, 0, 2]
    w = torch.randn(Cn, taps, device=DEV)
    b = torch.randn(Cn, device=DEV) if bias else None
    xs = [torch.randn(n, ld, device=DEV) for n in lens]
    state = torch.zeros(6, (taps - 1) * Cn + 12, device=DEV)
    state[:, (taps - 1) * Cn:] = 7.0                  # (what lies behind the convolution's part of a slot stays)
    cuts = [_cut(lens[0], [5, 1, 1, 2, 9]), _cut(lens[1], [1, 1, 3]), _cut(lens[2], [17, 1, 2, 1])]
    at, got = [0, 0, 0], [[], [], []]
    while any(a < n for a, n in zip(at, lens)):
        live = [e for e in range(3) if at[e] < lens[e]]
        rows = [cuts[e].pop(0) for e in live]
        n_pad = 0 if all(r == 1 for r in rows) else 2      # (single rows only: one kernel also moves the state on)
        proj = torch.cat([xs[e][at[e]:at[e] + r] for e, r in zip(live, rows)] + [torch.randn(n_pad, ld, device=DEV)])
        ctx = step_ctx(rows, [0] * sum(rows), slots=[slots[e] for e in live], n_pad=n_pad)
        out = torch.full((sum(rows) + 2, Cn + 3), 9.0, device=DEV)
        ops.short_conv(proj, c_off, Cn, taps, w, b, state, ctx, out, ops.ACT_SILU)
        assert torch.all(out[sum(rows):] == 9.0) and torch.all(out[:, Cn:] == 9.0)
        r0 = 0
        for e, r in zip(live, rows):
            got[e].append(out[r0:r0 + r, :Cn].clone())
            at[e] += r
            r0 += r
    for e in range(3):
        x = xs[e][:, c_off:c_off + Cn].double()
        xx = torch.cat([torch.zeros(taps - 1, Cn, device=DEV, dtype=torch.float64), x])
        want = sum(w[:, j].double() * xx[j:j + lens[e]] for j in range(taps))
        if bias:
            want = want + b.double()
        want = want * torch.sigmoid(want)
        assert float((torch.cat(got[e]).double() - want).abs().max()) < 1e-5, e
        if taps > 1:      # the slot holds the last taps - 1 inputs, oldest first
            assert torch.equal(state[slots[e], :(taps - 1) * Cn].view(taps - 1, Cn), xs[e][lens[e] - taps + 1:, c_off:c_off + Cn])
    assert torch.all(state[:, (taps - 1) * Cn:] == 7.0) and not state[[1, 3, 5], :(taps - 1) * Cn].any()


def _scan_reference(delta, q, k, v, a, w, skip, kq_ratio):
    """q, k [n, G, N], v [n, H, V], a, w [n, H]: outputs [n, H, V] and the final matrices [H, N, V], in float64."""
    n, H, V = v.shape
    N = q.shape[2]
    out, S = torch.zeros(n, H, V, dtype=torch.float64), torch.zeros(H, N, V, dtype=torch.float64)
    for h in range(H):
        g = h // kq_ratio
        for t in range(n):
            if delta:
                S[h] = a[t, h] * S[h]
                u = w[t, h] * (v[t, h] - S[h].T @ k[t, g])
                S[h] = S[h] + torch.outer(k[t, g], u)
                out[t, h] = S[h].T @ q[t, g]
            else:
                S[h] = a[t, h] * S[h] + w[t, h] * torch.outer(k[t, g], v[t, h])
                out[t, h] = S[h].T @ q[t, g] + skip[h] * v[t, h]
    return out, S


@pytest.mark.parametrize("delta", [True, False])
@pytest.mark.parametrize("H,G,N,V", [(2, 2, 16, 24), (4, 2, 20, 10), (1, 1, 64, 64), (3, 1, 50, 33), (2, 1, 256, 16),
                                     (6, 3, 48, 48), (2, 2, 128, 70)])
def test_recurrence_kernel_carries_its_matrices_in_the_slot(H, G, N, V, delta):
    """Two requests in shuffled slots, cut into portions and single rows, against the recurrence in float64; the
    slot's layout [head][value channel][key channel, padded] checked at the end."""
    from nanoinfer_b200.kernels import ops

    torch.manual_seed(N + V)
    lens, slots, s_off = [37, 12], [3, 1], 8
    NP = ops.gated_scan_padded(N)
    assert NP >= N and NP % 16 == 0
    ldc = 2 * G * N + H * V + 4
    q_off, k_off, v_off = G * N, 0, 2 * G * N                 # (any order of the three)
    state = torch.zeros(5, s_off + H * V * NP, device=DEV)
    seqs = []
    for n in lens:
        cv = torch.randn(n, ldc, device=DEV)
        kk = cv[:, k_off:k_off + G * N].view(n, G, N)
        kk /= kk.norm(dim=-1, keepdim=True)                   # unit keys, as the delta rule has them
        coef = torch.stack([torch.rand(n, H, device=DEV) * 0.5 + 0.5, torch.rand(n, H, device=DEV)], -1).contiguous()
        seqs.append((cv, coef))
    skip = torch.randn(H, device=DEV)
    cuts = [_cut(lens[0], [9, 1, 1, 8, 2]), _cut(lens[1], [1, 1, 10])]
    at, got = [0, 0], [[], []]
    while any(a < n for a, n in zip(at, lens)):
        live = [e for e in range(2) if at[e] < lens[e]]
        rows = [cuts[e].pop(0) for e in live]
        cv = torch.cat([seqs[e][0][at[e]:at[e] + r] for e, r in zip(live, rows)])
        coef = torch.cat([seqs[e][1][at[e]:at[e] + r] for e, r in zip(live, rows)])
        ctx = step_ctx(rows, [0] * sum(rows), slots=[slots[e] for e in live])
        out = torch.full((sum(rows), H * V + 2), 9.0, device=DEV)
        ops.gated_scan(delta, cv, q_off, k_off, v_off, N, V, H, H // G, coef, None if delta else skip, state, s_off, ctx, out)
        assert torch.all(out[:, H * V:] == 9.0)
        r0 = 0
        for e, r in zip(live, rows):
            got[e].append(out[r0:r0 + r, :H * V].clone())
            at[e] += r
            r0 += r
    for e, n in enumerate(lens):
        cv, coef = seqs[e][0].double().cpu(), seqs[e][1].double().cpu()
        want, S = _scan_reference(delta, cv[:, q_off:q_off + G * N].view(n, G, N), cv[:, k_off:k_off + G * N].view(n, G, N),
                                  cv[:, v_off:v_off + H * V].view(n, H, V), coef[..., 0], coef[..., 1], skip.double().cpu(), H // G)
        diff = float((torch.cat(got[e]).double().cpu().view(n, H, V) - want).abs().max())
        assert diff < 2e-4 * max(1.0, float(want.abs().max())), (e, diff)
        held = state[slots[e], s_off:].view(H, V, NP).double().cpu()
        assert float((held[:, :, :N] - S.transpose(1, 2)).abs().max()) < 2e-4 * max(1.0, float(S.abs().max()))
        assert not held[:, :, N:].any()
    assert not state[[0, 2, 4]].any() and not state[:, :s_off].any()


@pytest.mark.parametrize("delta", [True, False])
def test_decays_strengths_and_unit_vectors_against_torch(delta):
    from nanoinfer_b200.kernels import ops

    torch.manual_seed(8)
    T, H, G, N, ld = 13, 6, 2, 20, 64
    proj = torch.randn(T + 1, ld, device=DEV) * 3
    proj[2, 40] = 60.0                                # a softplus that is its argument
    A_log, dt_bias = torch.randn(H, device=DEV), torch.randn(H, device=DEV)
    cv0 = torch.randn(T + 1, 2 * G * N + 5, device=DEV)
    cv, coef = cv0.clone(), torch.zeros(T + 1, H, 2, device=DEV)
    a_off, w_off, q_off, k_off = 40, 50, G * N, 0
    ops.scan_prepare(proj, a_off, w_off, A_log, dt_bias, cv, q_off, k_off, N, H, G, delta, coef, T)
    p = proj[:T].double()
    sp = torch.nn.functional.softplus
    if delta:
        a = torch.exp(-torch.exp(A_log.double()) * sp(p[:, a_off:a_off + H] + dt_bias.double()))
        w = torch.sigmoid(p[:, w_off:w_off + H])
        for off, mul in ((q_off, N ** -0.5), (k_off, 1.0)):
            x = cv0[:T, off:off + G * N].double().view(T, G, N)
            want = x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6) * mul
            assert float((cv[:T, off:off + G * N].double().view(T, G, N) - want).abs().max()) < 1e-6
        assert torch.equal(cv[:, 2 * G * N:], cv0[:, 2 * G * N:]) and torch.equal(cv[T:], cv0[T:])
    else:
        w = sp(p[:, w_off:w_off + H] + dt_bias.double())
        a = torch.exp(-torch.exp(A_log.double()) * w)
        assert torch.equal(cv, cv0)
    assert float((coef[:T, :, 0].double() - a).abs().max()) < 1e-6
    assert float(((coef[:T, :, 1].double() - w) / (w.abs() + 1)).abs().max()) < 1e-6 and not coef[T:].any()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("groups,gs,wlen,gate_first", [(3, 24, 24, False), (1, 72, 72, True), (4, 18, 72, True),
                                                       (2, 130, 130, False)])
def test_gated_norm_kernel_against_torch(groups, gs, wlen, gate_first, dtype):
    from nanoinfer_b200.kernels import ops

    torch.manual_seed(gs)
    T, n, eps = 9, groups * gs, 1e-5
    o, gate_buf = torch.randn(T + 1, n, device=DEV) * 4, torch.randn(T + 1, n + 8, device=DEV) * 2
    gate, weight = gate_buf[:, 8:], torch.rand(wlen, device=DEV) + 0.5
    out = torch.zeros(T + 1, n, device=DEV, dtype=DT[dtype])
    ops.gated_norm(o, gate, weight, groups, gs, eps, gate_first, 0.7, out, T)
    g = gate[:T].double()
    silu = g * torch.sigmoid(g)
    y = o[:T].double() * (silu if gate_first else 1.0)
    y = y.view(T, groups, gs)
    y = (y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)).view(T, n) * weight.double().repeat(n // wlen)
    want = y * (1.0 if gate_first else silu) * 0.7
    tol = 1e-5 if dtype == "float32" else 0.02
    assert float(((out[:T].double() - want) / (want.abs() + 1)).abs().max()) < tol and not out[T:].any()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,dim,vdim,norms", [(4, 2, 16, 16, "qk"), (3, 1, 24, 8, "qk"), (2, 2, 12, 40, "q"),
                                                (2, 1, 96, 96, "qk"), (5, 5, 20, 20, "")])
def test_head_norm_cast_and_cache_write_against_torch(H, G, dim, vdim, norms, dtype):
    from nanoinfer_b200.kernels import ops

    torch.manual_seed(dim)
    dt, page, eps = DT[dtype], 16, 1e-5
    hd = -(-max(dim, vdim) // 16) * 16
    rows, pos0 = [5, 1, 20], [30, 47, 0]
    positions = [p0 + i for p0, r in zip(pos0, rows) for i in range(r)]
    ctx = step_ctx(rows, positions, n_pad=2)
    T = ctx.n_rows
    k_off = H * dim + 2
    v_off = k_off + G * dim
    proj = torch.randn(T, v_off + G * vdim + 2, device=DEV) * 3
    wq = torch.rand(dim, device=DEV) + 0.5 if "q" in norms else None
    wk = torch.rand(dim, device=DEV) + 0.5 if "k" in norms else None
    table = torch.full((3, 4), -1, dtype=torch.int32)
    table[0, :3], table[1, :3], table[2, :2] = torch.tensor([5, 1, 7]), torch.tensor([0, 2, 6]), torch.tensor([3, 4])
    cache = torch.full((8, 2, G, page, hd), 9.0, device=DEV, dtype=dt)
    q_out = torch.full((T, H * hd), 9.0, device=DEV, dtype=dt)
    ops.norm_rope_append(proj, (0, k_off, v_off), H, G, dim, vdim, wq, wk, eps, 0, None, ctx, q_out, cache, table.to(DEV))
    assert int(ctx.status.item()) == 0

    def normed(x, w):
        x = x.double()
        return x if w is None else x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w.double()
    tol = 1e-5 if dtype == "float32" else 0.04
    q = normed(proj[:, :H * dim].view(T, H, dim), wq)
    got = q_out.double().view(T, H, hd)
    assert float((got[:, :, :dim] - q).abs().max()) < tol and not got[:, :, dim:].any()
    k, v = normed(proj[:, k_off:k_off + G * dim].view(T, G, dim), wk), proj[:, v_off:v_off + G * vdim].view(T, G, vdim).double()
    written = torch.zeros(8, page, dtype=torch.bool)
    t = 0
    for e, (p0, r) in enumerate(zip(pos0, rows)):
        for i in range(r):
            pg, sl = int(table[e, (p0 + i) // page]), (p0 + i) % page
            written[pg, sl] = True
            assert float((cache[pg, 0, :, sl, :dim].double() - k[t]).abs().max()) < tol
            assert float((cache[pg, 1, :, sl, :vdim].double() - v[t]).abs().max()) < tol
            assert not cache[pg, 0, :, sl, dim:].any() and not cache[pg, 1, :, sl, vdim:].any()
            t += 1
    assert torch.all(cache.cpu().permute(0, 3, 1, 2, 4)[~written] == 9.0)      # rows of no request wrote nothing


# =============================================================================== attention with options
def _option_attention(q, k, v, scale, pos0, window=0, keep_first=0, softcap=0.0, slopes=None, gate=None, out_scale=1.0):
    """q [n, H, d], k, v [m, G, d]: row i stands at position pos0 + i and sees key j <= its position if
    position - j < window (any, without one) or j < keep_first.  float64."""
    H, G = q.shape[1], k.shape[1]
    out = torch.zeros(q.shape[0], H, v.shape[2], dtype=torch.float64)
    j = torch.arange(k.shape[0])
    for h in range(H):
        s = (q[:, h].double() @ k[:, h // (H // G)].double().T) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        for i in range(q.shape[0]):
            p = pos0 + i
            see = (j <= p) & (((p - j) < window) | (j < keep_first) if window else torch.ones_like(j, dtype=torch.bool))
            si = s[i] - (float(slopes[h]) * (p - j).double() if slopes is not None else 0.0)
            w = torch.softmax(si.masked_fill(~see, -math.inf), -1)
            o = w @ v[:, h // (H // G)].double() * out_scale
            out[i, h] = o * (torch.sigmoid(gate[i, h].double()) if gate is not None else 1.0)
    return out


OPTION_SETS = {
    "a cap": dict(softcap=5.0),
    "a window that keeps the first tokens": dict(window=70, keep_first=5),
    "a window that keeps more than a page": dict(window=33, keep_first=21, softcap=9.0),
    "a distance bias, a gate and a constant": dict(window=50, slopes=True, gate=True, out_scale=1.7),
    "a distance bias over all keys": dict(slopes=True),
    "kept tokens that the window still covers": dict(window=500, keep_first=4, softcap=4.0),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hd,n_head,n_kv_head", [(48, 4, 1), (96, 4, 2), (64, 2, 2), (32, 3, 1), (144, 2, 1)])
@pytest.mark.parametrize("name", list(OPTION_SETS))
def test_attention_kernels_with_options_on_scores_and_output(name, hd, n_head, n_kv_head, dtype):
    """Portions and single tokens side by side through the dispatcher, then the streaming kernel of single tokens
    with the keys split every way."""
    from nanoinfer_b200.kernels import ops
    from nanoinfer_b200.parts.attention import AttentionPlan

    o = dict(OPTION_SETS[name])
    dt, page, scale = DT[dtype], 16, 1.2 / math.sqrt(hd)
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / n_head) for h in range(n_head)]) if o.pop("slopes", False) else None
    want_gate = o.pop("gate", False)
    window = o.get("window", 0)
    tol = 3e-5 if dtype == "float32" else 2e-2

    def run(lengths, q_rows, seed, direct_splits=None):
        cache, table, ks, vs, qs = _paged(dt, n_head, n_kv_head, hd, page, lengths, q_rows, seed=seed)
        positions = [p for n, r in zip(lengths, q_rows) for p in range(n - r, n)]
        ctx = step_ctx(q_rows, positions)
        T = ctx.n_rows
        gate = torch.randn(T, n_head + 3) * 2 if want_gate else None
        want, r0 = [], 0
        for qq, k, v, n, r in zip(qs, ks, vs, lengths, q_rows):
            want.append(_option_attention(qq, k, v, scale, n - r, slopes=slopes, gate=gate[r0:r0 + r] if want_gate else None, **o))
            r0 += r
        want = torch.cat(want)
        q = torch.cat(qs).view(-1, n_head * hd).to(dt).to(DEV)
        ex = ops.AttnExtras(o.get("softcap", 0.0), o.get("keep_first", 0), slopes.to(DEV) if slopes is not None else None,
                            gate.to(DEV)[:, :n_head] if want_gate else None, o.get("out_scale", 1.0))
        cache_d, table_d = cache.to(dt).to(DEV), table.to(DEV)
        out = torch.full_like(q, 7.0)
        if direct_splits is None:
            plan = AttentionPlan(ctx.host_entry_start, ctx.host_entry_pos0, device=torch.device(DEV))
            ops.attention(q, cache_d, out, table_d, ctx, n_head, scale, window, plan, extras=ex)
        else:
            keys = min(max(lengths), window) if window else max(lengths)
            chunk = max(16, -(-(-(-keys // direct_splits)) // 16) * 16)
            n_splits = -(-keys // chunk)
            scratch = torch.zeros(ops.DECODE_RESIDENT_BLOCKS * (hd + 2), device=DEV)
            counters = torch.zeros(ops.DECODE_RESIDENT_BLOCKS, dtype=torch.int32, device=DEV)
            code = ops.library().nib_attention_decode(
                0 if dtype == "float32" else 1, q.data_ptr(), q.stride(0), cache_d.data_ptr(), scratch.data_ptr(),
                out.data_ptr(), out.stride(0), table_d.data_ptr(), table_d.shape[1], None, ctx.row_entry.data_ptr(),
                ctx.positions.data_ptr(), T, n_head, n_kv_head, hd, page, cache_d.shape[0], scale, window, 0, *ex.args(),
                chunk, n_splits, counters.data_ptr(), ctx.status.data_ptr(), torch.cuda.current_stream().cuda_stream)
            assert code == 0
        assert int(ctx.status.item()) == 0
        diff = float((out.double().cpu().view(want.shape) - want).abs().max())
        assert diff < tol, f"{name}, splits {direct_splits}: {diff:.3e}"
        return want

    with_options = run([200, 77, 450, 130, 16, 3], [130, 1, 1, 40, 16, 1], seed=hd)
    if hd <= 128:
        for ns in (1, 2, 3, 5, 16):
            run([450, 77, 300, 2, 40], [1, 1, 1, 1, 1], seed=hd + 1, direct_splits=ns)
    # the options show: without them the same inputs give something else
    cache, table, ks, vs, qs = _paged(dt, n_head, n_kv_head, hd, page, [200, 77, 450, 130, 16, 3], [130, 1, 1, 40, 16, 1], seed=hd)
    plain = torch.cat([_option_attention(qq, k, v, scale, n - r) for qq, k, v, n, r in
                       zip(qs, ks, vs, [200, 77, 450, 130, 16, 3], [130, 1, 1, 40, 16, 1])])
    assert float((plain - with_options).abs().max()) > 20 * tol


LONG_OPTION_SETS = {
    "kept tokens a tile or more behind the window": dict(window=70, keep_first=5, softcap=6.0),
    "more kept tokens than a tile holds": dict(window=40, keep_first=150),
    "kept tokens that end in the window's first tile": dict(window=200, keep_first=140, softcap=11.0),
    "a distance bias, a gate and a constant behind a window": dict(window=260, slopes=True, gate=True, out_scale=0.6),
    "a cap and a distance bias over all keys": dict(softcap=3.0, slopes=True),
}


@pytest.mark.parametrize("hd,n_head,n_kv_head", [(64, 4, 2), (64, 3, 1), (32, 2, 2), (128, 2, 1), (48, 4, 4)])
@pytest.mark.parametrize("name", list(LONG_OPTION_SETS))
def test_prompt_kernels_with_options_over_many_tiles(name, hd, n_head, n_kv_head):
    """Long portions in bfloat16, so that the tiled tensor-core kernels of prompts (the tcgen05 one at head size 64,
    the warp-MMA one elsewhere) walk several tiles of keys, those of the kept tokens ahead of the window's, with rows
    that start anywhere in a tile and pages in any order."""
    from nanoinfer_b200.kernels import ops
    from nanoinfer_b200.parts.attention import AttentionPlan

    o = dict(LONG_OPTION_SETS[name])
    dt, page, scale = torch.bfloat16, 16, 1.3 / math.sqrt(hd)
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / n_head) for h in range(n_head)]) if o.pop("slopes", False) else None
    want_gate = o.pop("gate", False)
    window = o.get("window", 0)
    lengths, q_rows = [700, 333, 390, 131], [300, 290, 3, 130]
    cache, table, ks, vs, qs = _paged(dt, n_head, n_kv_head, hd, page, lengths, q_rows, seed=hd + n_head)
    positions = [p for n, r in zip(lengths, q_rows) for p in range(n - r, n)]
    ctx = step_ctx(q_rows, positions)
    T = ctx.n_rows
    gate = torch.randn(T, n_head + 1) * 2 if want_gate else None
    want, r0 = [], 0
    for qq, k, v, n, r in zip(qs, ks, vs, lengths, q_rows):
        want.append(_option_attention(qq, k, v, scale, n - r, slopes=slopes, gate=gate[r0:r0 + r] if want_gate else None, **o))
        r0 += r
    want = torch.cat(want)
    q = torch.cat(qs).view(-1, n_head * hd).to(dt).to(DEV)
    ex = ops.AttnExtras(o.get("softcap", 0.0), o.get("keep_first", 0), slopes.to(DEV) if slopes is not None else None,
                        gate.to(DEV)[:, :n_head] if want_gate else None, o.get("out_scale", 1.0))
    cache_d = cache.to(dt).to(DEV)
    if window:
        # pages that hold nothing visible to any row of the step are gone: the kernels must not need them
        for e, (n, r) in enumerate(zip(lengths, q_rows)):
            for b in range(-(-n // page)):
                if (b + 1) * page <= n - r - window + 1 and b * page >= o.get("keep_first", 0):
                    cache_d[int(table[e, b])] = float("nan")
                    table[e, b] = -1
    out = torch.full_like(q, 7.0)
    plan = AttentionPlan(ctx.host_entry_start, ctx.host_entry_pos0, device=torch.device(DEV))
    ops.attention(q, cache_d, out, table.to(DEV), ctx, n_head, scale, window, plan, extras=ex)
    assert int(ctx.status.item()) == 0
    diff = (out.double().cpu().view(want.shape) - want).abs()
    assert float(diff.max()) < 2e-2, f"{name}: {float(diff.max()):.3e} at row {int(diff.amax((1, 2)).argmax())}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows", [1, 40])
def test_one_matching_key_at_the_edges_of_the_window_and_of_the_kept_tokens(rows, dtype):
    """Every key is at right angles to every query but one, which matches: the last row's output is that key's value
    exactly when the key is visible (the last of the window, the last kept token, either side of a page border) and
    an average that has nothing of it when it is just outside."""
    from nanoinfer_b200.kernels import ops
    from nanoinfer_b200.parts.attention import AttentionPlan

    dt, hd, page, n, window, keep = DT[dtype], 80, 16, 600, 150, 20
    last = n - 1
    places = {0: True, keep - 1: True, keep: False, 15: True, 16: True, 31: False, last - window: False,
              last - window + 1: True, last - window + 2: True, 463: True, 464: True, 479: True, 480: True, last: True}
    for far, visible in places.items():
        cache, table, ks, vs, qs = _paged(dt, 2, 1, hd, page, [n], [rows], seed=11)
        u = torch.zeros(hd)
        u[5] = 1.0
        ks[0][:, 0] = ks[0][:, 0] - ks[0][:, 0, 5:6] * u            # at right angles to u
        ks[0][far, 0] = 8.0 * u
        qs[0] = 6.0 * u.expand(rows, 2, hd).clone()
        for b in range(-(-n // page)):
            m = min(page, n - b * page)
            cache[int(table[0, b]), 0, :, :m] = ks[0][b * page:b * page + m].transpose(0, 1)
        want = _option_attention(qs[0], ks[0], vs[0], 1.0, n - rows, window=window, keep_first=keep, softcap=30.0)
        ctx = step_ctx([rows], list(range(n - rows, n)))
        q = qs[0].reshape(rows, -1).to(dt).to(DEV)
        out = torch.full_like(q, 7.0)
        plan = AttentionPlan(ctx.host_entry_start, ctx.host_entry_pos0, device=torch.device(DEV))
        ops.attention(q, cache.to(dt).to(DEV), out, table.to(DEV), ctx, 2, 1.0, window, plan,
                      extras=ops.AttnExtras(softcap=30.0, keep_first=keep))
        got = out.double().cpu().view(want.shape)
        assert float((got - want).abs().max()) < (1e-4 if dtype == "float32" else 3e-2), (rows, far)
        found = float((got[-1] - vs[0][far].double()).abs().max()) < 3e-2
        assert found == visible, f"key {far}: visible {visible}, found {found}"


# =============================================================================== models through the step function
class Harness:
    def __init__(self, cfg, tmp_path, dtype, max_tokens=512, slots=4, page=16, max_rows=256, seed=1, sharpen=3.0,
                 long_memory=False):
        from nanoinfer_b200 import load_model
        from nanoinfer_b200.cache import CacheManager
        from nanoinfer_b200.engine import ModelRunner
        from plain_kemuzen import PlainKemuzen

        self.dir = write_model(cfg, str(tmp_path), DT[dtype], seed=seed, sharpen=sharpen, long_memory=long_memory)
        self.plain = PlainKemuzen(self.dir)
        self.model = load_model(self.dir, DT[dtype], DEV)
        self.cache = CacheManager(self.model.kv_needs(), self.model.state_needs(), max_tokens=max_tokens,
                                  max_requests=slots, page_size=page, dtype=DT[dtype], device=torch.device(DEV),
                                  max_positions=None, padding=True)
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
    "capped attention": [attention_layer()],
    "capped attention, one head, values longer than keys, no cap": [attention_layer(heads=1, kv_heads=1, dim=8, vdim=24, softcap=None)],
    "capped attention, every head its own keys, nothing kept": [attention_layer(heads=3, kv_heads=3, dim=12, vdim=6, keep_first=None)],
    "capped attention over all keys": [attention_layer(heads=5, kv_heads=1, dim=20, vdim=10, window=None, scale=0.4)],
    "capped attention, a window of one token and two kept": [attention_layer(window=1, keep_first=2)],
    "capped attention, more kept than a page holds": [attention_layer(heads=2, kv_heads=1, dim=64, vdim=16, window=17, keep_first=19)],
    "gated delta rule": [delta_layer()],
    "gated delta rule, one head of 40 by 72, two taps": [delta_layer(heads=1, kv_heads=1, dim=40, vdim=72, conv=2)],
    "gated delta rule, four heads on two keys, sizes no multiple of four": [delta_layer(heads=4, kv_heads=2, dim=18, vdim=10, conv=3)],
    "gated delta rule without a convolution to speak of": [delta_layer(heads=2, kv_heads=1, dim=32, vdim=8, conv=1)],
    "attention beside a state space": [parallel_layer()],
    "attention beside a state space, groups and norm parts": [parallel_layer(heads=2, kv_heads=2, dim=24, vdim=8, window=7, r_heads=4,
                                                                             r_vdim=12, state=20, groups=2, norm_groups=3, conv=2,
                                                                             left_scale=0.4, right_scale=2.0)],
    "attention beside a state space, over all keys, one head each": [parallel_layer(heads=1, kv_heads=1, dim=16, vdim=32, window=None,
                                                                                    r_heads=1, r_vdim=40, state=64, conv=5)],
    "gated feed-forward": [delta_layer(mlp=dense(72))],
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(ONE_LAYER))
def test_each_mechanism_alone_as_a_one_layer_model(name, dtype, tmp_path):
    h = Harness(config(ONE_LAYER[name], vocab=150, width=48), tmp_path, dtype)
    t = toks(150, 75, 3)
    h.check(h.alone(t, [1000]), t, name)
    h.check(h.alone(t, [40, 1, 1, 2, 3, 1]), t, name + " in portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("what", ["no token input, no cap on the logits", "a token input of one value", "an odd vocabulary and width"])
def test_the_parts_around_the_layers(what, dtype, tmp_path):
    layers = [delta_layer(mlp=dense(40)), attention_layer(mlp=None)]
    cfg = {"no token input, no cap on the logits": config(layers, vocab=90, width=40, side=0, logit_softcap=None),
           "a token input of one value": config(layers, vocab=90, width=40, side=1, logit_softcap=3.0, scale=1.0),
           "an odd vocabulary and width": config(layers, vocab=131, width=36, side=5, eps=3e-4)}[what]
    h = Harness(cfg, tmp_path, dtype)
    t = toks(cfg["vocab"], 50, 6)
    h.check(h.alone(t, [1000]), t, what)
    h.check(h.alone(t, [30, 1, 2]), t, what + " in portions")


FULL = [delta_layer(heads=2, kv_heads=1, dim=24, vdim=40, mlp=dense(80)),
        parallel_layer(mlp=dense(56)),
        attention_layer(heads=4, kv_heads=2, dim=32, vdim=32, window=40, keep_first=5, mlp=dense(64)),
        attention_layer(heads=4, kv_heads=2, dim=32, vdim=32, window=24, keep_first=2, softcap=6.0, kv_from=2, mlp=None),
        delta_layer(heads=4, kv_heads=4, dim=16, vdim=16, conv=3, mlp=None),
        attention_layer(heads=4, kv_heads=2, dim=32, vdim=32, window=None, kv_from=2, mlp=dense(40)),
        parallel_layer(heads=2, kv_heads=1, dim=32, vdim=16, window=33, r_heads=4, r_vdim=8, state=32, groups=2,
                       norm_groups=2, conv=4, mlp=None)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_token_by_token_and_portions_agree(dtype, tmp_path):
    h = Harness(config(FULL, vocab=190, width=64, scale=5.0, eps=1e-6), tmp_path, dtype)
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
    assert h.runner.graph_replays > 50            # single tokens ran as replayed graphs, state and all
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
def test_lengths_around_page_and_window_edges_and_the_first_tokens(dtype, tmp_path):
    layers = [attention_layer(window=16, keep_first=1, mlp=None), delta_layer(mlp=None),
              parallel_layer(heads=2, kv_heads=1, dim=16, vdim=32, window=17, mlp=None)]
    h = Harness(config(layers, vocab=120, width=40), tmp_path, dtype, sharpen=4.0)
    for n in (1, 2, 3, 15, 16, 17, 18, 31, 32, 33, 47, 48, 49):
        t = toks(120, n + 3, n)
        h.check(h.alone(t, [n, 1, 1, 1]), t, f"{n} tokens, then three alone")
        h.check(h.alone(t, [1, 1, 1, n]), t, f"three alone, then {n}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_behind_windows_gives_pages_back_but_not_the_first(dtype, tmp_path):
    from nanoinfer_b200.engine import StepItem

    layers = [delta_layer(mlp=dense()), attention_layer(window=40, keep_first=18, mlp=dense(32)), parallel_layer(window=50),
              attention_layer(window=70, keep_first=3, kv_from=1)]
    h = Harness(config(layers, vocab=100, width=48), tmp_path, dtype, max_tokens=384, slots=2)
    t = toks(100, 330, 9)
    r = h.cache.open_request()
    rows = [h.runner.step([StepItem(r, t[:5], list(range(5)))]).clone()]
    for p in range(5, len(t)):
        rows.append(h.runner.step([StepItem(r, t[p:p + 1], [0])]).clone())
    # of the attention that keeps 18 tokens (its pages serve a reader with a window of 70): the first two pages and
    # those of the last 70 positions are held; of the other: those of the last 50
    held = {g.spec.keep_first: sum(1 for p in blocks if p >= 0) for g, blocks in zip(h.cache.groups, r.blocks)}
    assert held[18] == 2 + len({p // 16 for p in range(330 - 70 + 1, 330)})
    assert held[0] == len({p // 16 for p in range(330 - 50 + 1, 330)})
    assert all(r.blocks[gi][0] >= 0 and r.blocks[gi][1] >= 0 and r.blocks[gi][2] < 0
               for gi, g in enumerate(h.cache.groups) if g.spec.keep_first)
    h.cache.close_request(r)
    h.check(torch.cat(rows), t, "330 positions")
    assert h.runner.graph_replays > 300


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_long_prompts_through_the_tiled_prompt_kernels(dtype, tmp_path):
    """Heads of 64 (the tcgen05 prompt kernel in bfloat16) and of 128 and 32 (the warp-MMA one) over prompts of
    several tiles of keys: windows that end in the middle of a tile, kept tokens a tile or more behind them, a layer
    that reads another's cache with a narrower window and more kept tokens, a distance bias over hundreds of keys;
    whole, in portions that start anywhere, and with the last tokens one by one."""
    layers = [attention_layer(heads=4, kv_heads=2, dim=64, vdim=64, softcap=15.0, window=150, keep_first=5, mlp=dense(40)),
              parallel_layer(heads=2, kv_heads=1, dim=64, vdim=32, window=210, r_heads=2, r_vdim=16, state=16),
              attention_layer(heads=4, kv_heads=2, dim=64, vdim=64, softcap=None, window=70, keep_first=140, kv_from=0),
              attention_layer(heads=2, kv_heads=1, dim=128, vdim=64, softcap=8.0, window=129, keep_first=1),
              parallel_layer(heads=3, kv_heads=3, dim=32, vdim=32, window=None, r_heads=1, r_vdim=8, state=8, conv=2)]
    h = Harness(config(layers, vocab=150, width=64), tmp_path, dtype, max_tokens=1216, slots=2, max_rows=640, seed=5)
    tokens = toks(150, 590, 77)
    h.check(h.alone(tokens, [590]), tokens, "whole")
    h.check(h.alone(tokens, [333, 2, 131, 100] + [1] * 24), tokens, "in portions")
    assert h.cache.pages_used() == [0] * len(h.cache.groups)


def test_a_token_far_back_shows_through_the_state_and_through_the_kept_tokens(tmp_path):
    """Recurrences whose rates let them remember for hundreds of tokens, and an attention that keeps its first
    token behind a short window: two prompts that differ in their first token only still differ 150 tokens on, and
    the engine follows the plain model in both."""
    for layers in ([delta_layer(heads=2, kv_heads=2, dim=32, vdim=32)], [parallel_layer(window=4, left_scale=0.01)],
                   [attention_layer(window=8, keep_first=1)]):
        cfg = config(layers, vocab=90, width=64, side=0)
        h = Harness(cfg, tmp_path, "float32", long_memory=True, sharpen=6.0)
        a = toks(90, 150, 4)
        b = [(a[0] + 1) % 90] + a[1:]
        la, lb = h.plain.logits(a)[-1], h.plain.logits(b)[-1]
        assert rel_err(la[None], lb[None]) > 10 * TOL["float32"], layers[0]["type"]
        for t in (a, b):
            h.check(h.alone(t, [120, 7, 1]), t)


def random_config(rnd):
    width = rnd.choice([32, 40, 64, 72, 96, 100])
    layers, owners = [], []
    for i in range(rnd.randint(1, 6)):
        mlp = rnd.choice([None, dense(rnd.choice([24, 50, 64]))])
        kind = rnd.choice(["attention", "delta", "parallel"])
        window = rnd.choice([None, 1, 5, 16, 31, 64, 200])
        if kind == "attention":
            if owners and rnd.random() < 0.4:
                j = rnd.choice(owners)
                m = layers[j]["mixer"]
                layers.append(attention_layer(heads=m["heads"], kv_heads=m["kv_heads"], dim=m["dim"], vdim=m["vdim"],
                                              scale=rnd.choice([0.1, 0.3]), softcap=rnd.choice([None, 4.0, 30.0]), window=window,
                                              keep_first=rnd.choice([None, 0, 1, 6, 17, 40]), kv_from=j, mlp=mlp))
                continue
            g = rnd.choice([1, 2, 3])
            layers.append(attention_layer(heads=g * rnd.choice([1, 2, 4]), kv_heads=g, dim=rnd.choice([4, 8, 12, 16, 32, 64]),
                                          vdim=rnd.choice([4, 8, 16, 24, 64]), scale=rnd.choice([0.1, 0.25, 0.4]),
                                          softcap=rnd.choice([None, 4.0, 30.0]), window=window,
                                          keep_first=rnd.choice([None, 0, 1, 6, 17, 40]), mlp=mlp))
            owners.append(i)
        elif kind == "delta":
            g = rnd.choice([1, 2, 3])
            layers.append(delta_layer(heads=g * rnd.choice([1, 2]), kv_heads=g, dim=rnd.choice([8, 16, 20, 32, 48, 80]),
                                      vdim=rnd.choice([8, 16, 24, 66, 100]), conv=rnd.choice([1, 2, 3, 4, 6]), mlp=mlp))
        else:
            g, rg = rnd.choice([1, 2]), rnd.choice([1, 2])
            rh, rv = rg * rnd.choice([1, 2, 3]), rnd.choice([8, 12, 16, 40])
            layers.append(parallel_layer(heads=g * rnd.choice([1, 2, 4]), kv_heads=g, dim=rnd.choice([8, 16, 24, 48]),
                                         vdim=rnd.choice([8, 16, 48]), scale=rnd.choice([0.1, 0.3]), window=window, r_heads=rh,
                                         r_vdim=rv, state=rnd.choice([8, 16, 24, 48, 100]), groups=rg,
                                         norm_groups=rnd.choice([d for d in (1, 2, 4) if (rh * rv) % d == 0]),
                                         conv=rnd.choice([2, 3, 4]), left_scale=rnd.choice([0.5, 1.0, 1.2]),
                                         right_scale=rnd.choice([0.5, 1.0, 2.0]), mlp=mlp))
    return config(layers, vocab=rnd.choice([97, 256, 1001]), width=width, scale=rnd.choice([1.0, 4.0, 16.0]),
                  eps=rnd.choice([1e-6, 1e-5, 3e-4]), logit_softcap=rnd.choice([None, 10.0, 30.0]),
                  side=rnd.choice([0, 4, 8, 11]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", range(12))
def test_random_configuration_cut_at_random(case, dtype, tmp_path):
    from nanoinfer_b200.engine import StepItem

    rnd = random.Random(7100 + case)
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
    from plain_kemuzen import PlainKemuzen

    cfg = config(FULL, vocab=130, width=64)
    d = write_model(cfg, str(tmp_path), torch.float32, seed=3)
    plain = PlainKemuzen(d)
    prompts = [toks(130, n, 40 + n) for n in (1, 9, 30, 55, 17)]
    eng = nb.Engine(d, dtype="float32", max_tokens=3 * 128, max_batch=3, max_rows=64)
    outs = eng.generate(prompts, nb.SamplingParams(max_new_tokens=20))
    for p, o in zip(prompts, outs):
        assert o == plain.greedy(p, 20)
    assert eng.runner.graph_replays > 0 and eng.cache.pages_used() == [0] * len(eng.cache.groups)


def test_trace_replay_of_a_model_folder(tmp_path):
    from plain_kemuzen import PlainKemuzen
    from trace_util import TraceSession

    cfg = config(FULL[:4], vocab=110, width=48)
    d = write_model(cfg, str(tmp_path / "m"), torch.float32, seed=8)
    plain = PlainKemuzen(d)
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
    from plain_kemuzen import PlainKemuzen

    d = str(tmp_path / "m")
    assert cli.main(["random-weights", "--config", "kemuzen-tiny", "--seed", "6", "--out", d, "--dtype", "float32"]) == 0
    capsys.readouterr()
    prompt = toks(512, 12, 77)
    assert cli.main(["--weights", d, "generate", "--dtype", "float32", "--prompt-ids", ",".join(map(str, prompt)),
                     "--tokens", "10", "--temperature", "0.0", "--profile"]) == 0
    captured = capsys.readouterr()
    printed = [int(t) for t in captured.out.split()]
    assert printed == PlainKemuzen(d).greedy(prompt, 10)
    assert "scan" in captured.err and "attn" in captured.err
