"""Mulavik on the GPU: every new kernel and every kernel option alone against plain torch, every mechanism alone
as a one-layer model, and whole models through the step function, cut into steps every way, against the plain
implementation (tests/plain_mulavik.py).  Test weights are made so that faults show (mulavik_util.write_model);
where random values would still hide one (a far key, the sink), the kernel test builds queries and keys by hand."""
import json
import math
import random
from types import SimpleNamespace

import pytest
import torch

from mulavik_util import (TOL, assert_close, attention_layer, config, dense, memory_layer, moe, rel_err, row_errs,
                          write_model)

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
DEV = "cuda"


def toks(vocab, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def step_ctx(entry_rows, positions, slots=None, n_pad=0):
    """A StepContext's worth of device tables for kernels that are driven without the step function:
    ``entry_rows`` rows per entry, in order; ``n_pad`` rows of no request behind them."""
    from nanoinfer_b200.kernels import ops
    from nanoinfer_b200.parts.base import Workspace

    start = [0]
    for n in entry_rows:
        start.append(start[-1] + n)
    row_entry = [e for e, n in enumerate(entry_rows) for _ in range(n)] + [-1] * n_pad
    pos = list(positions) + [0] * n_pad
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    return SimpleNamespace(n_rows=len(row_entry), n_entries=len(entry_rows), positions=i32(pos), row_entry=i32(row_entry),
                           entry_start=i32(start), entry_pos0=i32([positions[s] for s in start[:-1]]), entry_slot=i32(slots if slots is not None else list(range(len(entry_rows)))),
                           status=torch.zeros(1, dtype=torch.int32, device=DEV), workspace=Workspace(torch.device(DEV)),
                           host_entry_start=start, host_entry_pos0=[positions[s] for s in start[:-1]], max_rows=len(row_entry))


# =============================================================================== kernels alone
@pytest.mark.parametrize("C", [40, 264, 1536])
def test_norm_sum_norm_kernel_against_torch(C):
    from nanoinfer_b200.kernels import ops

    torch.manual_seed(C)
    T, R, eps = 9, 12, 3e-5
    x0, y0 = torch.randn(R, C, device=DEV) * 3, torch.randn(R, C, device=DEV) * 40
    w_out, w_next = torch.rand(C, device=DEV) + 0.5, torch.rand(C, device=DEV) + 0.5
    rms = lambda v, w: v.double() / torch.sqrt((v.double() ** 2).mean(-1, keepdim=True) + eps) * w.double()
    want = x0.double() + rms(y0, w_out)
    for dt in (torch.float32, torch.bfloat16):
        x, y, xn = x0.clone(), y0.clone(), torch.zeros(R, C, device=DEV, dtype=dt)
        ops.add_norm(x, y, w_out, eps, T, w_next, xn)
        assert float((x[:T] - want[:T]).abs().max()) < 1e-5 and torch.equal(x[T:], x0[T:])
        assert not y[:T].any() and torch.equal(y[T:], y0[T:])          # zeroed for the next sublayer
        assert float((xn[:T].double() - rms(want[:T], w_next)).abs().max()) < (1e-5 if dt == torch.float32 else 0.03)
        assert not xn[T:].any()
    x, y = x0.clone(), y0.clone()
    ops.add_norm(x, y, w_out, eps, T)
    assert float((x[:T] - want[:T]).abs().max()) < 1e-5 and not y[:T].any()


def test_gated_activation_kernel_against_torch():
    from nanoinfer_b200.kernels import ops

    torch.manual_seed(4)
    T, F = 13, 21
    pre = torch.randn(T + 2, 2 * F + 6, device=DEV) * 3
    g, u, r = pre[:T, 0:2 * F:2].double(), pre[:T, 1:2 * F:2].double(), pre[:T, 2 * F].double()
    silu = g * torch.sigmoid(g) * u
    for dt in (torch.float32, torch.bfloat16):
        out = torch.zeros(T + 2, F + 3, device=DEV, dtype=dt)
        ops.glu(pre, out, T, F, ops.ACT_SILU)
        tol = 1e-5 if dt == torch.float32 else 0.02
        assert float(((out[:T, :F].double() - silu) / (silu.abs() + 1)).abs().max()) < tol and not out[T:].any() and not out[:, F:].any()
        ops.glu(pre, out, T, F, ops.ACT_SILU, row_gate=2 * F)
        want = silu * torch.sigmoid(r)[:, None]
        assert float(((out[:T, :F].double() - want) / (want.abs() + 1)).abs().max()) < tol
    out = torch.zeros(T, F, device=DEV)
    ops.glu(pre, out, T, F, ops.ACT_RELU_SQ)
    assert float((out.double() - torch.clamp(g, min=0) ** 2 * u).abs().max()) < 1e-4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M", [3, 40, 300, 1600])
def test_products_with_the_square_of_relu(M, dtype):
    """Every product kernel the dispatcher may choose for these sizes applies the activation in its epilogue."""
    from nanoinfer_b200.kernels import ops

    torch.manual_seed(M)
    K, N = 192, 320
    a = torch.randn(M, K, device=DEV).to(DT[dtype])
    w = (torch.randn(N, K, device=DEV) * 0.1).to(DT[dtype])
    out = torch.zeros(M, N, device=DEV, dtype=DT[dtype])
    ops.linear(a, w, None, out, M, act=ops.ACT_CODES["relu2"])
    want = torch.clamp(a.double() @ w.double().T, min=0) ** 2
    assert float(((out.double() - want).abs() / (want.abs() + 1)).max()) < (1e-5 if dtype == "float32" else 0.02)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,dim,vdim,rot", [(4, 2, 16, 16, 8), (3, 3, 24, 8, 24), (2, 1, 12, 40, 4), (5, 1, 64, 32, 0),
                                             (1, 1, 6, 6, 6)])
def test_rotation_cast_and_cache_write_against_torch(H, G, dim, vdim, rot, dtype):
    from nanoinfer_b200.kernels import ops
    from plain_mulavik import rotate_pairs

    torch.manual_seed(H * 100 + dim)
    dt, page, hd = DT[dtype], 16, -(-max(dim, vdim) // 16) * 16
    rows, positions = [5, 1, 3], [0, 1, 2, 3, 4, 5000, 30, 31, 32]       # an entry across a page border, one far out
    ctx = step_ctx(rows, positions, n_pad=2)
    T = ctx.n_rows
    n_q, n_k, n_v = H * dim, G * dim, G * vdim
    ld = -(-(n_q + n_k + n_v) // 8) * 8
    proj = torch.randn(T, ld, device=DEV)
    n_pages = 320
    table = torch.full((3, 316), -1, dtype=torch.int32, device=DEV)
    table[0, 0], table[1, 5000 // page], table[2, 1], table[2, 2] = 7, 3, 11, 2
    cache = torch.full((n_pages, 2, G, page, hd), 9.0, device=DEV, dtype=dt)
    q_out = torch.full((T, H * hd), 9.0, device=DEV, dtype=dt)
    base = 300.0
    freqs = (base ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)).to(DEV) if rot else None
    ops.rope_append(proj, (0, n_q, n_q + n_k), H, G, dim, vdim, rot, freqs, ctx, q_out, cache, table)
    assert int(ctx.status.item()) == 0
    pos = torch.tensor(positions + [0, 0])
    tol = 1e-5 if dtype == "float32" else 0.02
    q_ref = rotate_pairs(proj[:, :n_q].double().cpu().view(T, H, dim), pos, base, rot)
    k_ref = rotate_pairs(proj[:, n_q:n_q + n_k].double().cpu().view(T, G, dim), pos, base, rot)
    v_ref = proj[:, n_q + n_k:n_q + n_k + n_v].double().cpu().view(T, G, vdim)
    got_q = q_out.double().cpu().view(T, H, hd)
    assert float((got_q[:, :, :dim] - q_ref).abs().max()) < tol * 4 and not got_q[:, :, dim:].any()
    seen = torch.zeros(n_pages, page, dtype=torch.bool)
    for t in range(T - 2):
        e = int(ctx.row_entry[t])
        pg, slot = int(table[e, positions[t] // page]), positions[t] % page
        seen[pg, slot] = True
        got_k, got_v = cache[pg, 0, :, slot].double().cpu(), cache[pg, 1, :, slot].double().cpu()
        assert float((got_k[:, :dim] - k_ref[t]).abs().max()) < tol * 4 and not got_k[:, dim:].any()
        assert float((got_v[:, :vdim] - v_ref[t]).abs().max()) < tol * 4 and not got_v[:, vdim:].any()
    untouched = cache.cpu().permute(0, 3, 1, 2, 4)[~seen]
    assert bool((untouched == 9.0).all())                # rows of no request and other slots: nothing written


def _paged(dtype, n_head, n_kv_head, hd, page, lengths, q_rows, seed):
    """Keys and values of ``lengths`` positions per entry in shuffled pages, and ``q_rows`` last queries each."""
    g = torch.Generator().manual_seed(seed)
    n_blocks = [-(-n // page) for n in lengths]
    ids = torch.randperm(sum(n_blocks) + 3, generator=g).tolist()
    table = torch.full((len(lengths), max(n_blocks) + 1), -1, dtype=torch.int32)
    cache = torch.full((sum(n_blocks) + 3, 2, n_kv_head, page, hd), 50.0)      # (what other requests left behind)
    ks, vs, qs = [], [], []
    for e, n in enumerate(lengths):
        k, v = torch.randn(n, n_kv_head, hd, generator=g), torch.randn(n, n_kv_head, hd, generator=g)
        k, v = k.to(dtype).float(), v.to(dtype).float()
        for b in range(n_blocks[e]):
            pg = ids.pop()
            table[e, b] = pg
            m = min(page, n - b * page)
            cache[pg, 0, :, :m] = k[b * page:b * page + m].transpose(0, 1)
            cache[pg, 1, :, :m] = v[b * page:b * page + m].transpose(0, 1)
        ks.append(k); vs.append(v)
        qs.append(torch.randn(q_rows[e], n_head, hd, generator=g).to(dtype).float())
    return cache, table, ks, vs, qs


def _sink_attention(q, k, v, scale, pos0, sink):
    """q [n, H, d], k, v [m, G, d]: row i (position pos0 + i) sees keys 0..pos0 + i."""
    H, G = q.shape[1], k.shape[1]
    out = torch.zeros(q.shape[0], H, v.shape[2], dtype=torch.float64)
    for h in range(H):
        s = (q[:, h].double() @ k[:, h // (H // G)].double().T) * scale
        for i in range(q.shape[0]):
            e = torch.exp(s[i, :pos0 + i + 1])
            out[i, h] = (e / (e.sum() + (1.0 if sink else 0.0))) @ v[:pos0 + i + 1, h // (H // G)].double()
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hd,n_head,n_kv_head", [(64, 4, 2), (32, 2, 2), (48, 3, 1), (128, 2, 1), (24, 2, 1), (96, 2, 2),
                                                 (160, 2, 1)])
def test_every_attention_kernel_with_the_sink(hd, n_head, n_kv_head, dtype):
    """Portions and single tokens side by side through the dispatcher (which picks the tcgen05, the warp-MMA or the
    general kernel for portions and the MMA or the streaming kernel for single tokens), with and without the
    sink; then each decode kernel with the keys split every way."""
    from nanoinfer_b200.kernels import ops
    from nanoinfer_b200.parts.attention import AttentionPlan

    dt, page, scale = DT[dtype], 16, 0.3 / math.sqrt(hd)
    lengths, q_rows = [200, 77, 450, 130, 16], [130, 1, 1, 40, 16]
    cache, table, ks, vs, qs = _paged(dt, n_head, n_kv_head, hd, page, lengths, q_rows, seed=hd)
    positions = [p for n, r in zip(lengths, q_rows) for p in range(n - r, n)]
    ctx = step_ctx(q_rows, positions)
    q = torch.cat(qs).view(-1, n_head * hd).to(dt).to(DEV)
    cache_d, table_d = cache.to(dt).to(DEV), table.to(DEV)
    tol = 3e-5 if dtype == "float32" else 2e-2
    for sink in (False, True):
        want = torch.cat([_sink_attention(qq, k, v, scale, n - r, sink) for qq, k, v, n, r in zip(qs, ks, vs, lengths, q_rows)])
        out = torch.full_like(q, 7.0)
        plan = AttentionPlan(ctx.host_entry_start, ctx.host_entry_pos0, device=torch.device(DEV))
        ops.attention(q, cache_d, out, table_d, ctx, n_head, scale, 0, plan, sink=sink)
        assert int(ctx.status.item()) == 0
        diff = float((out.double().cpu().view(want.shape) - want).abs().max())
        assert diff < tol, f"sink {sink}: {diff:.3e}"
    # the sink shows: with it the weights no longer add up to one
    no_sink = torch.cat([_sink_attention(qq, k, v, scale, n - r, False) for qq, k, v, n, r in zip(qs, ks, vs, lengths, q_rows)])
    assert float((no_sink - want).abs().max()) > 50 * tol
    # single tokens, the keys split into 1 to 16 pieces, on each decode kernel
    lib, lengths = ops.library(), [450, 77, 300]
    cache, table, ks, vs, qs = _paged(dt, n_head, n_kv_head, hd, page, lengths, [1, 1, 1], seed=hd + 1)
    want = torch.cat([_sink_attention(qq, k, v, scale, n - 1, True) for qq, k, v, n in zip(qs, ks, vs, lengths)])
    ctx = step_ctx([1, 1, 1], [n - 1 for n in lengths])
    q = torch.cat(qs).view(-1, n_head * hd).to(dt).to(DEV)
    cache_d, table_d = cache.to(dt).to(DEV), table.to(DEV)
    scratch = torch.zeros(ops.DECODE_RESIDENT_BLOCKS * (hd + 2), device=DEV)
    counters = torch.zeros(ops.DECODE_RESIDENT_BLOCKS, dtype=torch.int32, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    kernels = ["streaming"] + (["mma", "mma cluster"] if dtype == "bfloat16" and lib.nib_attention_decode_mma_supported(hd, page) else [])
    if hd > 128 or hd % 8:
        kernels = []
    for kernel in kernels:
        for ns in (1, 2, 3, 4, 7, 16):
            if ("cluster" in kernel) != (ns > 1 and "mma" in kernel):
                continue
            chunk = max(16, -(-(-(-max(lengths) // ns)) // 16) * 16)
            n_splits = -(-max(lengths) // chunk)
            out = torch.full_like(q, 7.0)
            args = (q.data_ptr(), q.stride(0), cache_d.data_ptr(), scratch.data_ptr(), out.data_ptr(), out.stride(0),
                    table_d.data_ptr(), table_d.shape[1], None, ctx.row_entry.data_ptr(), ctx.positions.data_ptr(), 3,
                    n_head, n_kv_head, hd, page, cache_d.shape[0], scale, 0, 1, chunk, n_splits, counters.data_ptr(),
                    ctx.status.data_ptr())
            plain = ops.AttnExtras().args()         # no options on the scores or the output
            code = lib.nib_attention_decode(0 if dtype == "float32" else 1, *args[:-4], *plain, *args[-4:], stream) \
                if kernel == "streaming" else \
                lib.nib_attention_decode_mma(*args, int("cluster" in kernel), 0, stream)
            assert code == 0 and int(ctx.status.item()) == 0, (kernel, n_splits)
            diff = float((out.double().cpu().view(want.shape) - want).abs().max())
            assert diff < tol, f"{kernel}, {n_splits} splits: {diff:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sink_takes_the_weight_when_no_key_matches_and_a_far_key_takes_it_when_one_does(dtype):
    """Scores far below zero: the output is next to nothing (without a sink it would be an average of values).
    Then one key far back is made to match the query: the output is that key's value, whichever page it is on."""
    from nanoinfer_b200.kernels import ops
    from nanoinfer_b200.parts.attention import AttentionPlan

    dt, hd, page, n = DT[dtype], 64, 16, 600
    for rows in (1, 40):                         # a single token, and the end of a portion
        for far in (None, 0, 15, 16, 255, 431, n - rows):
            cache, table, ks, vs, qs = _paged(dt, 2, 2, hd, page, [n], [rows], seed=7)
            qv = qs[0]
            for h in range(2):                   # every key points away from every query: scores around -70
                u = qv[:, h].mean(0)
                u = u / u.norm()
                kk = 0.25 * (ks[0][:, h] - (ks[0][:, h] @ u)[:, None] * u) - 6.0 * u
                ks[0][:, h] = kk
            qs[0] = qv = 4.0 * qv / qv.norm(dim=-1, keepdim=True) + 12.0 * qv.mean(0, keepdim=True) / qv.mean(0, keepdim=True).norm(dim=-1, keepdim=True)
            if far is not None:
                for h in range(2):
                    ks[0][far, h] = 6.0 * qv[:, h].mean(0) / qv[:, h].mean(0).norm()
            for b in range(-(-n // page)):
                m = min(page, n - b * page)
                cache[int(table[0, b]), 0, :, :m] = ks[0][b * page:b * page + m].transpose(0, 1)
            want = _sink_attention(qv.to(dt).float(), ks[0].to(dt).float(), vs[0], 1.0, n - rows, True)
            ctx = step_ctx([rows], list(range(n - rows, n)))
            q = qv.reshape(rows, -1).to(dt).to(DEV)
            out = torch.full_like(q, 7.0)
            plan = AttentionPlan(ctx.host_entry_start, ctx.host_entry_pos0, device=torch.device(DEV))
            ops.attention(q, cache.to(dt).to(DEV), out, table.to(DEV), ctx, 2, 1.0, 0, plan, sink=True)
            got = out.double().cpu().view(want.shape)
            assert float((got - want).abs().max()) < (1e-4 if dtype == "float32" else 3e-2), (rows, far)
            if far is None:
                assert float(got.abs().max()) < 1e-3
            else:
                assert float((got[-1] - vs[0][far].double()).abs().max()) < 3e-2, f"key {far} was not found"


def _memory_reference(proj, off, bi, bf, cap, norm_w, H, dim, vdim, eps, state):
    """plain_mulavik.mlstm's recurrence on ready-made projections (float64), one entry."""
    import torch.nn.functional as Fn
    n = proj.shape[0]
    q = proj[:, off[0]:off[0] + H * dim].view(n, H, dim) * dim ** -0.5
    k = proj[:, off[1]:off[1] + H * dim].view(n, H, dim)
    v = proj[:, off[2]:off[2] + H * vdim].view(n, H, vdim)
    g = proj[:, off[3]:off[3] + H * vdim]
    gi = cap * torch.tanh((proj[:, off[4]:off[4] + H] + bi) / cap)
    gf = Fn.logsigmoid(cap * torch.tanh((proj[:, off[5]:off[5] + H] + bf) / cap))
    S, nn, mx = state
    o = torch.zeros(n, H, vdim, dtype=torch.float64)
    for t in range(n):
        new = torch.maximum(gf[t] + mx, gi[t])
        keep, take = torch.exp(gf[t] + mx - new), torch.exp(gi[t] - new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        nn = keep[:, None] * nn + take[:, None] * k[t]
        mx = new
        den = torch.maximum((nn * q[t]).sum(-1).abs(), torch.exp(-mx)) + 1e-6
        o[t] = torch.einsum("hdv,hd->hv", S, q[t]) / den[:, None]
    o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps)
    return o.reshape(n, H * vdim) * norm_w * torch.sigmoid(g), (S, nn, mx)


@pytest.mark.parametrize("H,dim,vdim", [(2, 16, 24), (1, 40, 64), (3, 48, 70), (2, 64, 130), (1, 100, 8), (1, 256, 32)])
def test_matrix_memory_kernel_carries_its_state_in_the_slot(H, dim, vdim):
    """Three requests in shuffled slots, fed in portions of unequal sizes (single tokens among them) over several
    steps with rows of no request behind them: outputs and the state follow the recurrence in float64."""
    from nanoinfer_b200.kernels import ops

    torch.manual_seed(dim + vdim)
    cap, eps = 9.0, 1e-5
    off = (0, H * dim, 2 * H * dim, 2 * H * dim + H * vdim, 2 * H * dim + 2 * H * vdim, 2 * H * dim + 2 * H * vdim + H)
    ld = -(-(off[5] + H) // 8) * 8
    bi, bf = torch.randn(H, device=DEV), torch.rand(H, device=DEV) * 6 - 1
    norm_w = torch.rand(H * vdim, device=DEV) + 0.5
    per_head = ops.mlstm_state_floats(dim, vdim)
    state = torch.zeros(5, H * per_head, device=DEV)
    state[3] = 5.0                                # a slot nobody holds
    slots = [4, 0, 2]
    ref_state = [(torch.zeros(H, dim, vdim, dtype=torch.float64), torch.zeros(H, dim, dtype=torch.float64),
                  torch.zeros(H, dtype=torch.float64)) for _ in slots]
    for step, rows in enumerate([[7, 1, 30], [1, 1, 1], [2, 300, 1], [64, 1, 5]]):
        ctx = step_ctx(rows, [0] * sum(rows), slots=slots, n_pad=3)
        T = ctx.n_rows
        proj = torch.randn(T, ld, device=DEV)
        proj[:, off[4]:off[4] + 2 * H] *= 4.0
        for dt in (torch.bfloat16, torch.float32):           # (the float32 run is the one whose state stays)
            before = state.clone()
            out = torch.zeros(T, H * vdim, device=DEV, dtype=dt)
            ops.mlstm(proj, off, bi, bf, cap, norm_w, state, ctx, H, dim, vdim, eps, out, ctx.workspace)
            if dt == torch.bfloat16:
                got16, state = out, before
        at = 0
        for e, n in enumerate(rows):
            want, ref_state[e] = _memory_reference(proj[at:at + n].double().cpu(), off, bi.double().cpu(), bf.double().cpu(), cap,
                                                   norm_w.double().cpu(), H, dim, vdim, eps, ref_state[e])
            scale = float(want.abs().max()) + 1e-3
            assert float((out[at:at + n].double().cpu() - want).abs().max()) < 2e-4 * scale, (step, e)
            assert float((got16[at:at + n].double().cpu() - want).abs().max()) < 2e-2 * scale, (step, e)
            at += n
    dp = -(-dim // 16) * 16
    for e, slot in enumerate(slots):
        S, nn, mx = ref_state[e]
        got = state[slot].double().cpu().view(H, per_head)
        cols = got[:, :(vdim + 1) * dp].view(H, vdim + 1, dp)
        assert float((cols[:, :vdim, :dim].transpose(1, 2) - S).abs().max()) < 1e-4 * (float(S.abs().max()) + 1)
        assert float((cols[:, vdim, :dim] - nn).abs().max()) < 1e-4 * (float(nn.abs().max()) + 1)
        assert float((got[:, (vdim + 1) * dp] - mx).abs().max()) < 1e-5
    assert bool((state[3] == 5.0).all()) and not state[1].any()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,top,C,F,T", [(5, 1, 40, 12, 19), (4, 4, 64, 34, 19), (10, 1, 88, 24, 150), (4, 2, 72, 50, 150),
                                         (8, 3, 192, 80, 150)])
def test_gated_experts_with_sigmoid_scores_on_their_input(E, top, C, F, T, dtype):
    """The router's sigmoid scores and choices; then gated SiLU experts whose input is scaled by the score, row by
    row, expert by expert and all experts at once (the three forms the dispatcher chooses between), against torch;
    and the same experts with the score on the output."""
    from nanoinfer_b200.kernels import ops
    from nanoinfer_b200.parts.base import Workspace

    torch.manual_seed(E * 10 + top)
    dt = DT[dtype]
    h = torch.randn(T + 2, C, device=DEV).to(dt)
    wr = (torch.randn(E, C, device=DEV) * 0.5).to(dt)
    ids = torch.full((T + 2, top), -7, dtype=torch.int32, device=DEV)
    wts = torch.zeros(T + 2, top, device=DEV)
    ops.moe_route(h, wr, T, top, False, ids, wts, score="sigmoid")
    s = torch.sigmoid(h[:T].double() @ wr.double().T)
    score, chosen = torch.topk(s, top, -1)
    assert torch.equal(ids[:T].long(), chosen) and (ids[T:] == -7).all()
    assert float((wts[:T] - score).abs().max()) < 1e-5
    gate = (torch.randn(E, F, C, device=DEV) * 0.2).to(dt)
    up = (torch.randn(E, F, C, device=DEV) * 0.2).to(dt)
    down = (torch.randn(E, C, F, device=DEV) * 0.2).to(dt)
    both = torch.stack([gate, up], 2).reshape(E, 2 * F, C).contiguous()       # rows 2f, 2f + 1: gate and value of output f
    x0 = torch.randn(T + 2, C, device=DEV)
    tol = 2e-4 if dtype == "float32" else 0.05
    for on_input in (True, False):
        hs = h[:T].double()[:, None, :] * (score[:, :, None] if on_input else 1.0)          # [T, top, C]
        g = torch.einsum("tkc,tkfc->tkf", hs, gate.double()[chosen])
        u = torch.einsum("tkc,tkfc->tkf", hs, up.double()[chosen])
        mid = g * torch.sigmoid(g) * u
        add = torch.einsum("tkf,tkcf->tkc", mid, down.double()[chosen])
        want = x0[:T].double() + (add if on_input else add * score[:, :, None]).sum(1)
        ws = Workspace(torch.device(DEV))
        results = {}
        saved = (ops.MOE_DENSE, ops.MOE_GROUPED)
        try:
            for form, (d, g_) in {"rows": (False, False), "grouped": (False, True), "dense": (True, True)}.items():
                ops.MOE_DENSE, ops.MOE_GROUPED = d, g_
                if form == "dense" and not ops.moe_dense_pays(T, top, E):
                    continue
                x = x0.clone()
                inner = torch.zeros((T + 2) * top, F, device=DEV, dtype=dt)
                ops.moe_experts(h, both, down, ids, wts, inner, x, T, top, ops.ACT_SILU, ws, gated=True, weight_on_input=on_input)
                results[form] = x
                assert float((x[:T].double() - want).abs().max()) < tol * (float(want.abs().max()) + 1), (form, on_input)
                assert torch.equal(x[T:], x0[T:])
        finally:
            ops.MOE_DENSE, ops.MOE_GROUPED = saved
        assert "rows" in results and "grouped" in results


# =============================================================================== models through the step function
class Harness:
    def __init__(self, cfg, tmp_path, dtype, max_tokens=512, slots=4, page=16, max_rows=256, seed=1, sharpen=8.0,
                 long_memory=False):
        from nanoinfer_b200 import load_model
        from nanoinfer_b200.cache import CacheManager
        from nanoinfer_b200.engine import ModelRunner
        from plain_mulavik import PlainMulavik

        self.dir = write_model(cfg, str(tmp_path), DT[dtype], seed=seed, sharpen=sharpen, long_memory=long_memory)
        self.plain = PlainMulavik(self.dir)
        self.model = load_model(self.dir, DT[dtype], DEV)
        self.cache = CacheManager(self.model.kv_needs(), self.model.state_needs(), max_tokens=max_tokens,
                                  max_requests=slots, page_size=page, dtype=DT[dtype], device=torch.device(DEV),
                                  max_positions=None, padding=True)
        self.runner = ModelRunner(self.model, self.cache, max_rows=max_rows, max_entries=slots, check_status=True)
        self.dtype, self.vocab = dtype, cfg["vocab"]
        #: the routed feed-forwards by layer, and what each chose: {request key: {layer: {position: experts}}}
        self.routed = {i: blk.feed_forward for i, blk in enumerate(self.model.layers)
                       if getattr(blk.feed_forward, "last_ids", False) is not False}
        self.chose = {}

    def record(self, spans):
        """After a step whose rows were, in order, ``spans`` = (request key, first position, rows): keep what
        every router chose for them (its buffer holds the step's choices, replayed from a graph or not)."""
        for layer, part in self.routed.items():
            ids, row = part.last_ids.cpu(), 0
            for key, at, n in spans:
                mine = self.chose.setdefault(key, {}).setdefault(layer, {})
                for j in range(n):
                    mine[at + j] = ids[row + j].tolist()
                row += n

    def choices(self, key, n):
        """A request's recorded choices as {layer: [n, top]} (None in 32-bit, where the plain model's own stand)."""
        if self.dtype == "float32" or not self.routed:
            return None
        return {layer: torch.tensor([got[p] for p in range(n)]) for layer, got in self.chose[key].items()}

    def alone(self, tokens, cuts):
        """One request cut into portions of the sizes in ``cuts`` (cycled), all logits back."""
        from nanoinfer_b200.engine import StepItem

        r, at, k, rows = self.cache.open_request(), 0, 0, []
        self.chose.pop("alone", None)
        while at < len(tokens):
            n = min(cuts[k % len(cuts)], len(tokens) - at)
            rows.append(self.runner.step([StepItem(r, tokens[at:at + n], list(range(n)))]).clone())
            self.record([("alone", at, n)])
            at, k = at + n, k + 1
        self.cache.close_request(r)
        return torch.cat(rows)

    def check(self, got, tokens, what="", key="alone"):
        """Against the plain model; in bfloat16 the plain model follows the engine's choice of experts wherever
        its own router's call is close (and checks that the engine's choice was one of the close ones)."""
        ref = self.plain.logits(tokens, self.choices(key, len(tokens)))
        assert_close(row_errs(got, ref), self.dtype, what)


ONE_LAYER = {
    "attention": [attention_layer()],
    "attention, one head, values longer than keys, no rotation": [attention_layer(heads=1, kv_heads=1, dim=8, vdim=24, rot_dims=None)],
    "attention, every head its own keys, all of a head rotated": [attention_layer(heads=3, kv_heads=3, dim=12, vdim=6, rot_dims=12, base=50.0)],
    "attention, one key head for all, sizes no multiple of 8": [attention_layer(heads=5, kv_heads=1, dim=20, vdim=10, rot_dims=6, scale=0.4)],
    "attention, heads of 64 and 16": [attention_layer(heads=2, kv_heads=1, dim=64, vdim=16, rot_dims=48, scale=0.1)],
    "matrix memory": [memory_layer()],
    "matrix memory, one head of 40 by 72": [memory_layer(heads=1, dim=40, vdim=72, gate_cap=6.0)],
    "matrix memory, three heads, values shorter than keys": [memory_layer(heads=3, dim=32, vdim=8)],
    "dense feed-forward": [memory_layer(mlp=dense(72))],
    "routed feed-forward with a shared expert": [attention_layer(mlp=moe())],
    "routed, one expert a row, none shared": [memory_layer(mlp=moe(experts=5, top=1, shared=0))],
    "routed, every expert chosen": [memory_layer(mlp=moe(experts=3, top=3, ff=40, shared=8))],
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(ONE_LAYER))
def test_each_mechanism_alone_as_a_one_layer_model(name, dtype, tmp_path):
    h = Harness(config(ONE_LAYER[name], vocab=150, width=48), tmp_path, dtype)
    t = toks(150, 75, 3)
    h.check(h.alone(t, [1000]), t, name)
    h.check(h.alone(t, [40, 1, 1, 2, 3, 1]), t, name + " in portions")


FULL = [memory_layer(heads=2, dim=24, vdim=40, mlp=dense(80)), attention_layer(mlp=moe()),
        attention_layer(heads=3, kv_heads=1, dim=8, vdim=24, rot_dims=4, base=100.0, mlp=None),
        memory_layer(heads=4, dim=16, vdim=16, gate_cap=8.0, mlp=moe(experts=7, top=3, ff=16, shared=24)),
        attention_layer(heads=2, kv_heads=2, dim=32, vdim=16, rot_dims=32, mlp=dense(40)), memory_layer(mlp=None)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_token_by_token_and_portions_agree(dtype, tmp_path):
    h = Harness(config(FULL, vocab=190, width=64, scale=11.0, eps=1e-6), tmp_path, dtype)
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
        h.record([(i, live[i][1], n) for i, n in meta])
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
        h.check(torch.cat(got[i]), t, f"request {i}", key=i)
    assert max(len(u) for u in slot_users.values()) >= 2 and max(len(u) for u in page_users.values()) >= 2
    assert h.cache.pages_used() == [0] * len(h.cache.groups) and h.cache.slots.n_free == 3


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_lengths_around_page_edges_and_the_first_tokens(dtype, tmp_path):
    layers = [attention_layer(mlp=None), memory_layer(mlp=None), attention_layer(heads=2, kv_heads=1, dim=16, vdim=32, mlp=None)]
    h = Harness(config(layers, vocab=120, width=40), tmp_path, dtype, sharpen=12.0)
    for n in (1, 2, 3, 15, 16, 17, 18, 31, 32, 33, 47, 48, 49):
        t = toks(120, n + 3, n)
        h.check(h.alone(t, [n, 1, 1, 1]), t, f"{n} tokens, then three alone")
        h.check(h.alone(t, [1, 1, 1, n]), t, f"three alone, then {n}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype, tmp_path):
    from nanoinfer_b200.engine import StepItem

    layers = [memory_layer(mlp=dense()), attention_layer(mlp=moe()), memory_layer(heads=1, dim=32, vdim=16)]
    h = Harness(config(layers, vocab=100, width=48), tmp_path, dtype, max_tokens=384, slots=2)
    t = toks(100, 330, 9)
    r = h.cache.open_request()
    rows = [h.runner.step([StepItem(r, t[:5], list(range(5)))]).clone()]
    h.record([("alone", 0, 5)])
    for p in range(5, len(t)):
        rows.append(h.runner.step([StepItem(r, t[p:p + 1], [0])]).clone())
        h.record([("alone", p, 1)])
    h.cache.close_request(r)
    h.check(torch.cat(rows), t, "330 positions")
    assert h.runner.graph_replays > 300


def test_a_token_far_back_shows_through_the_state(tmp_path):
    """The gate biases of the test weights let the matrix memory remember for hundreds of tokens: two prompts that
    differ in their first token only still differ 150 tokens on, and the engine follows the plain model in both."""
    h = Harness(config([memory_layer(heads=2, dim=32, vdim=32, mlp=None)], vocab=90, width=64), tmp_path, "float32",
                long_memory=True)
    a = toks(90, 150, 4)
    b = [(a[0] + 1) % 90] + a[1:]
    la, lb = h.plain.logits(a)[-1], h.plain.logits(b)[-1]
    assert rel_err(la[None], lb[None]) > 10 * TOL["float32"]
    for t in (a, b):
        h.check(h.alone(t, [120, 7, 1]), t)


def random_config(rnd):
    width = rnd.choice([32, 40, 64, 72, 96, 100])
    layers = []
    for i in range(rnd.randint(1, 5)):
        mlp = rnd.choice([None, dense(rnd.choice([24, 50, 64])),
                          moe(experts=rnd.choice([2, 5, 8, 11]), top=rnd.choice([1, 2]), ff=rnd.choice([8, 20, 32]),
                              shared=rnd.choice([0, 12, 32]))])
        if rnd.random() < 0.5:
            layers.append(memory_layer(heads=rnd.choice([1, 2, 3]), dim=rnd.choice([8, 16, 20, 32, 48, 80]),
                                       vdim=rnd.choice([8, 16, 24, 66, 100]), gate_cap=rnd.choice([5.0, 9.0, 15.0]), mlp=mlp))
        else:
            g = rnd.choice([1, 2, 3])
            dim = rnd.choice([4, 8, 12, 16, 32, 64])
            layers.append(attention_layer(heads=g * rnd.choice([1, 2, 4]), kv_heads=g, dim=dim, vdim=rnd.choice([4, 8, 16, 24, 64]),
                                          rot_dims=rnd.choice([None, 0, dim, dim // 4 * 2]), base=rnd.choice([10.0, 10000.0, 500000.0]),
                                          scale=rnd.choice([0.1, 0.25, 0.4]), mlp=mlp))
    return config(layers, vocab=rnd.choice([97, 256, 1001]), width=width, scale=rnd.choice([1.0, 4.0, 16.0]),
                  eps=rnd.choice([1e-6, 1e-5, 3e-4]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", range(12))
def test_random_configuration_cut_at_random(case, dtype, tmp_path):
    from nanoinfer_b200.engine import StepItem

    rnd = random.Random(5300 + case)
    cfg = random_config(rnd)
    page = rnd.choice([16, 32, 48])
    lens = [rnd.randint(1, 150) for _ in range(rnd.randint(2, 6))]
    pages_of = lambda n: -(-n // page)
    pages = max(max(pages_of(n) for n in lens) + 2, int(0.6 * sum(pages_of(n) for n in lens)))
    h = Harness(cfg, tmp_path, dtype, max_tokens=pages * page, slots=3, page=page, max_rows=rnd.choice([64, 160]),
                seed=case + 1, sharpen=rnd.choice([4.0, 8.0]))
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
        h.record([(i, at, n) for i, at, n, _ in meta])
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
    want = [h.plain.logits(t, h.choices(i, len(t))) for i, t in enumerate(prompts)]
    keys = sorted(got)
    errs = row_errs(torch.stack([got[k] for k in keys]), torch.stack([want[i][p] for i, p in keys]))
    assert_close(errs, dtype, f"case {case} {json.dumps(cfg)} at (request, position) {keys}")


def test_greedy_generation_through_the_engine_and_its_scheduler(tmp_path):
    import nanoinfer_b200 as nb
    from plain_mulavik import PlainMulavik

    cfg = config(FULL, vocab=130, width=64)
    d = write_model(cfg, str(tmp_path), torch.float32, seed=3)
    plain = PlainMulavik(d)
    prompts = [toks(130, n, 40 + n) for n in (1, 9, 30, 55, 17)]
    eng = nb.Engine(d, dtype="float32", max_tokens=3 * 128, max_batch=3, max_rows=64)
    outs = eng.generate(prompts, nb.SamplingParams(max_new_tokens=20))
    for p, o in zip(prompts, outs):
        assert o == plain.greedy(p, 20)
    assert eng.runner.graph_replays > 0 and eng.cache.pages_used() == [0] * len(eng.cache.groups)


def test_trace_replay_of_a_model_folder(tmp_path):
    from plain_mulavik import PlainMulavik
    from trace_util import TraceSession

    cfg = config(FULL[:4], vocab=110, width=48)
    d = write_model(cfg, str(tmp_path / "m"), torch.float32, seed=8)
    plain = PlainMulavik(d)
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
    import nanoinfer_b200 as nb
    from nanoinfer_b200 import cli
    from plain_mulavik import PlainMulavik

    d = str(tmp_path / "m")
    assert cli.main(["random-weights", "--config", "mulavik-tiny", "--seed", "6", "--out", d, "--dtype", "float32"]) == 0
    capsys.readouterr()
    prompt = toks(512, 12, 77)
    assert cli.main(["--weights", d, "generate", "--dtype", "float32", "--prompt-ids", ",".join(map(str, prompt)),
                     "--tokens", "10", "--temperature", "0.0", "--profile"]) == 0
    captured = capsys.readouterr()
    printed = [int(t) for t in captured.out.split()]
    assert printed == PlainMulavik(d).greedy(prompt, 10)
    assert "mlstm" in captured.err and "attn" in captured.err and "experts_up" in captured.err
