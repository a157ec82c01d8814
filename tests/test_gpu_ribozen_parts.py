"""Each mechanism of the Ribozen design alone, the kernel against a plain
function in 64 bits (the building blocks of tests/plain_ribozen.py and the
recurrences written out here): the state-space recurrence in both its forms
under every cut of a sequence into steps, with state rows used again; the
matrix memory; bias, the norm over whole projections and the rotate-half turn
with ramped rates and the cache write; attention with kept first keys and
capped scores on all three kernels, with keys just inside and just outside the
window and the kept range, at page borders, in prompts and decoded alone; the
router's sigmoid scores and the weight on an expert's input; the layer scale
in the norm's kernel; the convolution's bias; the gates."""
import math

import pytest
import torch

import plain_ribozen as pr

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def i32(values):
    return torch.tensor(list(values), dtype=torch.int32, device=DEV)


def tiles(q_lens, size):
    req, q0 = [], []
    for b, n in enumerate(q_lens):
        for s in range(0, n, size):
            req.append(b); q0.append(s)
    return i32(req), i32(q0), len(req)


def tol_of(dtype, tight=2e-5, loose=2e-2):
    return dict(atol=tight, rtol=tight) if dtype == torch.float32 else dict(atol=loose, rtol=loose)


def feed_in_cuts(seq_lens, cuts, state_rows, run_step):
    """Feeds sequences in their cuts, the live requests of a step as one batch.
    Requests take the lowest free state row and give it back when they end, so
    rows are used again; ``run_step(live, q_lens, starts, slots, fresh)`` runs
    one step."""
    free = list(range(state_rows))
    slot_of, at = {}, [0] * len(seq_lens)
    step = 0
    while any(step < len(c) for c in cuts):
        live = [r for r in range(len(seq_lens)) if step < len(cuts[r])]
        fresh = [r not in slot_of for r in live]
        for r in live:
            if r not in slot_of:
                slot_of[r] = free.pop(0)
        q_lens = [cuts[r][step] for r in live]
        run_step(live, q_lens, [at[r] for r in live], [slot_of[r] for r in live], fresh)
        for r, n in zip(live, q_lens):
            at[r] += n
            if at[r] == seq_lens[r]:
                free.append(slot_of.pop(r))
        step += 1


# ------------------------------------------------------------------ the state-space recurrence
def plain_scan(x, B, C, dt_raw, z, dt_bias, a_log, d_skip, rows_per_head, rows_per_group, per_row, scale):
    """x [T, R], B, C [T, G, N], dt_raw [T, R or H], z [T, R] or None: out [T, R] in 64 bits."""
    T, R = x.shape
    N = B.shape[-1]
    dt = pr.softplus(dt_raw.double() + dt_bias.double())
    S = torch.zeros(R, N, dtype=torch.float64)
    out = torch.zeros(T, R, dtype=torch.float64)
    rows = torch.arange(R)
    entry = rows if per_row else rows // rows_per_head
    A = -torch.exp(a_log.double())
    A = A if per_row else A[entry][:, None].expand(R, N)
    for t in range(T):
        step = dt[t][entry]
        Bt, Ct = B[t].double()[rows // rows_per_group], C[t].double()[rows // rows_per_group]
        S = torch.exp(step[:, None] * A) * S + (step * x[t].double())[:, None] * Bt
        out[t] = (S * Ct).sum(-1) + d_skip.double()[entry] * x[t].double()
    if z is not None:
        out = out * pr.silu(z.double())
    return out * scale


SCANS = [
    # heads, rows per head, state, groups, per row, lengths, cuts
    (3, 5, 7, 3, False, (9, 30), ((9,), (2, 1, 27))),
    (4, 16, 64, 2, False, (40, 3, 21), ((17, 23), (1, 1, 1), (21,))),
    (1, 20, 5, 1, True, (33, 6), ((1, 32), (2, 2, 2))),
    (1, 64, 16, 1, True, (70, 18, 5), ((64, 2, 4), (18,), (1, 4))),
    (2, 24, 130, 1, False, (19,), ((3, 16),)),
    (1, 8, 512, 1, False, (18,), ((2, 16),)),                       # more shared memory than a block has by default
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", SCANS)
def test_state_space_recurrence_under_cuts(case, dtype):
    from lyapunov_engine_b200 import ops
    H, P, N, G, per_row, lens, cuts = case
    R = H * P
    g = torch.Generator().manual_seed(N + R)
    entries = R if per_row else H
    rows_per_group = R // G
    a_log = (torch.rand(R, N, generator=g) * 3 - 3) if per_row else (torch.rand(H, generator=g) * 3 - 3)
    dt_bias = torch.rand(entries, generator=g) * 3 - 3
    d_skip = torch.randn(entries, generator=g)
    seqs = []
    for n in lens:
        x, B, C = torch.randn(n, R, generator=g), torch.randn(n, G, N, generator=g), torch.randn(n, G, N, generator=g)
        dt, z = torch.randn(n, entries, generator=g), torch.randn(n, R, generator=g)
        seqs.append([v.to(dtype).float() for v in (x, B, C, dt, z)])
    want = [plain_scan(x, B, C, dt, z, dt_bias, a_log, d_skip, P, rows_per_group, per_row, 0.8) for x, B, C, dt, z in seqs]
    state = torch.full((3, R, N), 9.0, device=DEV)            # rows hold stale numbers; a fresh request's row is zeroed
    got = [[] for _ in seqs]
    wide = R + 2 * G * N + entries + R                        # one row: x | B | C | dt | z

    def run_step(live, q_lens, starts, slots, fresh):
        for s, f in zip(slots, fresh):
            if f:
                state[s].zero_()
        rows = torch.cat([torch.cat([v[a:a + n].reshape(n, -1) for v in seqs[r]], dim=1) for r, n, a in zip(live, q_lens, starts)])
        rows = rows.to(dtype).to(DEV)
        T = rows.shape[0]
        out = torch.zeros(T, R, dtype=dtype, device=DEV)
        cu = i32([0] + torch.tensor(q_lens).cumsum(0).tolist())
        dt_at = R + 2 * G * N
        ops.ssm_scan(out, rows[:, :R], rows, R, R + G * N, rows[:, dt_at:dt_at + entries], rows[:, dt_at + entries:wide],
                     dt_bias.to(DEV), a_log.to(DEV).contiguous(), d_skip.to(DEV), state, i32(slots), cu, len(live), N, P,
                     rows_per_group, per_row=per_row, out_scale=0.8)
        t0 = 0
        for r, n in zip(live, q_lens):
            got[r].append(out[t0:t0 + n].float().cpu())
            t0 += n

    feed_in_cuts(lens, cuts, 3, run_step)
    for r in range(len(seqs)):
        torch.testing.assert_close(torch.cat(got[r]).double(), want[r], **tol_of(dtype, tight=1e-4, loose=3e-2))


def test_a_request_without_a_state_row_gives_zeros():
    from lyapunov_engine_b200 import ops
    R, N = 8, 4
    rows = torch.randn(3, R + 2 * N + 1 + R, device=DEV)
    out = torch.ones(3, R, device=DEV)
    state = torch.ones(2, R, N, device=DEV)
    ops.ssm_scan(out, rows[:, :R], rows, R, R + N, rows[:, R + 2 * N:R + 2 * N + 1], rows[:, R + 2 * N + 1:],
                 torch.zeros(1, device=DEV), torch.zeros(1, device=DEV), torch.zeros(1, device=DEV), state, i32([-1]),
                 i32([0, 3]), 1, N, R, R, per_row=False)
    assert float(out.abs().max()) == 0.0 and float((state - 1).abs().max()) == 0.0


# ------------------------------------------------------------------ the matrix memory
def plain_memory(q, k, v, gi, gf, bi, bf, cap, scale):
    """q, k [T, H, d], v [T, H, e], gi, gf [T, H] pre-activations: o [T, H, e] in 64 bits."""
    T, H, d = q.shape
    q, k, v = q.double() * scale, k.double(), v.double()
    i = cap * torch.tanh((gi.double() + bi.double()) / cap)
    f = pr.log_sigmoid(cap * torch.tanh((gf.double() + bf.double()) / cap))
    out = torch.zeros(T, H, v.shape[-1], dtype=torch.float64)
    for h in range(H):
        S = torch.zeros(d, v.shape[-1], dtype=torch.float64)
        n = torch.zeros(d, dtype=torch.float64)
        m = torch.zeros((), dtype=torch.float64)
        for t in range(T):
            m_new = torch.maximum(f[t, h] + m, i[t, h])
            keep, take = torch.exp(f[t, h] + m - m_new), torch.exp(i[t, h] - m_new)
            S = keep * S + take * k[t, h][:, None] * v[t, h][None, :]
            n = keep * n + take * k[t, h]
            m = m_new
            out[t, h] = S.T @ q[t, h] / (torch.maximum(torch.abs(n @ q[t, h]), torch.exp(-m)) + 1e-6)
    return out


MEMORIES = [
    # heads, dim, vdim, cap, lengths, cuts
    (2, 12, 20, 6.0, (9, 30), ((9,), (2, 1, 27))),
    (1, 64, 64, 12.0, (40, 21), ((17, 23), (1, 20))),
    (3, 5, 3, 2.0, (33, 6, 18), ((1, 32), (2, 2, 2), (18,))),
    (2, 130, 8, 15.0, (19,), ((3, 16),)),
    (1, 512, 4, 9.0, (18,), ((2, 16),)),                            # more shared memory than a block has by default
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", MEMORIES)
def test_matrix_memory_under_cuts(case, dtype):
    from lyapunov_engine_b200 import ops
    H, d, e, cap, lens, cuts = case
    g = torch.Generator().manual_seed(d + e)
    bi, bf = torch.randn(H, generator=g), torch.randn(H, generator=g) + 2.0
    seqs = []
    for n in lens:
        q, k, v = torch.randn(n, H, d, generator=g), torch.randn(n, H, d, generator=g), torch.randn(n, H, e, generator=g)
        gi, gf = 3 * torch.randn(n, H, generator=g), 3 * torch.randn(n, H, generator=g)
        seqs.append([x.to(dtype).float() for x in (q, k, v, gi, gf)])
    want = [plain_memory(q, k, v, gi, gf, bi, bf, cap, d ** -0.5) for q, k, v, gi, gf in seqs]
    state = torch.full((3, *ops.mlstm_state_shape(H, d, e)), 9.0, device=DEV)
    got = [[] for _ in seqs]

    def run_step(live, q_lens, starts, slots, fresh):
        for s, f in zip(slots, fresh):
            if f:
                state[s].zero_()
        rows = torch.cat([torch.cat([x[a:a + n].reshape(n, -1) for x in seqs[r]], dim=1) for r, n, a in zip(live, q_lens, starts)])
        rows = rows.to(dtype).to(DEV)
        out = torch.zeros(rows.shape[0], H * e, device=DEV)
        cu = i32([0] + torch.tensor(q_lens).cumsum(0).tolist())
        ops.mlstm_scan(out, rows, 0, H * d, 2 * H * d, 2 * H * d + H * e, 2 * H * d + H * e + H, bi.to(DEV), bf.to(DEV), state,
                       i32(slots), cu, len(live), H, d, e, cap, d ** -0.5)
        t0 = 0
        for r, n in zip(live, q_lens):
            got[r].append(out[t0:t0 + n].cpu())
            t0 += n

    feed_in_cuts(lens, cuts, 3, run_step)
    for r in range(len(seqs)):
        torch.testing.assert_close(torch.cat(got[r]).double().view(-1, H, e), want[r], atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_head_norm_with_a_weight_per_head_and_a_sigmoid_gate(dtype):
    from lyapunov_engine_b200 import ops
    g = torch.Generator().manual_seed(3)
    T, H, e = 7, 3, 20
    o, gate, w = torch.randn(T, H * e, generator=g), torch.randn(T, H * e, generator=g).to(dtype), 1 + 0.2 * torch.randn(H * e, generator=g)
    out = torch.zeros(T, H * e + 8, dtype=dtype, device=DEV)
    ops.head_norm_gate(out[:, :H * e], o.to(DEV), gate.to(DEV), w.to(DEV), 1e-5, H, e, sigmoid=True, out_scale=0.7)
    want = pr.unit_rms(o.double().view(T, H, e), 1e-5).reshape(T, H * e) * w.double() * torch.sigmoid(gate.double()) * 0.7
    torch.testing.assert_close(out[:, :H * e].double().cpu(), want, **tol_of(dtype))
    assert float(out[:, H * e:].abs().max()) == 0.0


# ------------------------------------------------------------------ bias, norm over whole projections, turn, cache write
ENCODINGS = [
    # heads, kv heads, dim, vdim, padded, rot, base, scaling, page
    (4, 2, 16, 24, 32, 8, 1e4, {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}, 8),
    (3, 1, 24, 10, 32, 10, 1e3, None, 4),
    (2, 2, 64, 64, 64, 64, 5e5, {"factor": 6.0, "original": 1024, "fast": 16.0, "slow": 2.0}, 16),
    (1, 1, 16, 16, 16, 0, 1e4, None, 16),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", ENCODINGS)
def test_bias_norm_turn_and_store(case, dtype):
    from lyapunov_engine_b200 import ops
    from lyapunov_engine_b200.parts.rope import ramped_rates
    nh, nkv, d, e, hd, rot, base, scaling, page = case
    g = torch.Generator().manual_seed(d + rot)
    positions = [0, 1, 5, page - 1, page, 3 * page + 2, 700, 701]
    T = len(positions)

    def padded(t, heads, size):
        out = torch.zeros(t.shape[0], heads, hd) if t.dim() == 2 else torch.zeros(heads, hd)
        out[..., :size] = t.view(*t.shape[:-1], heads, size)
        return out.reshape(*t.shape[:-1], heads * hd)

    q, k, v = torch.randn(T, nh * d, generator=g), torch.randn(T, nkv * d, generator=g), torch.randn(T, nkv * e, generator=g)
    q, k, v = (x.to(dtype).float() for x in (q, k, v))
    bq, bk, bv = 0.3 * torch.randn(nh * d, generator=g), 0.3 * torch.randn(nkv * d, generator=g), 0.3 * torch.randn(nkv * e, generator=g)
    wq, wk = 1 + 0.3 * torch.randn(nh * d, generator=g), 1 + 0.3 * torch.randn(nkv * d, generator=g)
    rows = torch.cat([padded(q, nh, d), padded(k, nkv, d), padded(v, nkv, e), torch.full((T, 8), 5.0)], dim=1).to(dtype).to(DEV)
    bias = torch.cat([padded(bq, nh, d), padded(bk, nkv, d), padded(bv, nkv, e)]).to(DEV)
    rates, magnitude = ramped_rates(rot, base, scaling)
    plain_rates, plain_magnitude = pr.scaled_rates(rot, base, scaling) if rot else (rates[:0], 1.0)
    torch.testing.assert_close(rates[:rot // 2], plain_rates.double(), rtol=1e-12, atol=0)
    assert abs(magnitude - plain_magnitude) < 1e-12
    pages = positions[-1] // page + 2
    k_cache = torch.full((pages, nkv, page, hd), 7.0, dtype=dtype, device=DEV)
    v_cache = torch.full((pages, nkv, page, hd), 7.0, dtype=dtype, device=DEV)
    table = i32(range(pages - 1)).view(1, -1)
    status = ops.new_status(DEV)
    ops.rope_qknorm_store(rows, bias, padded(wq, nh, d).to(DEV), padded(wk, nkv, d).to(DEV), 1e-5, nh * d, nkv * d,
                          rates.to(DEV), rot, magnitude, k_cache, v_cache, i32(positions), i32([0] * T), table, nh, nkv, hd,
                          page, True, status)
    ops.check_status(status)
    pos = torch.tensor(positions)
    want_q = pr.rotate_half((pr.unit_rms(q.double() + bq.double(), 1e-5) * wq.double()).view(T, nh, d), pos, rot, base, scaling)
    want_k = pr.rotate_half((pr.unit_rms(k.double() + bk.double(), 1e-5) * wk.double()).view(T, nkv, d), pos, rot, base, scaling)
    want_v = (v.double() + bv.double()).view(T, nkv, e)
    tol = tol_of(dtype, tight=3e-5)
    got_q = rows[:, :nh * hd].double().cpu().view(T, nh, hd)
    torch.testing.assert_close(got_q[..., :d], want_q, **tol)
    assert float(got_q[..., d:].abs().max()) == 0.0 if hd > d else True
    assert float((rows[:, (nh + 2 * nkv) * hd:].float() - 5.0).abs().max()) == 0.0        # columns behind q | k | v are left alone
    for t, p in enumerate(positions):
        torch.testing.assert_close(k_cache[p // page, :, p % page, :d].double().cpu(), want_k[t], **tol)
        torch.testing.assert_close(v_cache[p // page, :, p % page, :e].double().cpu(), want_v[t], **tol)
    untouched = [p for p in range((pages - 1) * page) if p not in positions]
    assert all(float((k_cache[p // page, :, p % page].float() - 7.0).abs().max()) == 0.0 for p in untouched[:50])


# ------------------------------------------------------------------ attention: kept first keys, capped scores
def build_attention(dtype, nh, nkv, hd, page, q_lens, ctx_before, seed, window, keep, cap, scale):
    """Random keys and values in scattered pages; every request's last query
    looks hard for one key: the last kept one, the first one behind the kept
    range or the oldest one in the window, in turn."""
    g = torch.Generator().manual_seed(seed)
    B = len(q_lens)
    totals = [c + q for c, q in zip(ctx_before, q_lens)]
    max_blocks = max((t + page - 1) // page for t in totals) + 1
    needed = sum((t + page - 1) // page for t in totals)
    num_pages = needed + 3
    perm = torch.randperm(num_pages - 1, generator=g)[:needed].tolist()
    table = torch.full((B, max_blocks), num_pages - 1, dtype=torch.int32)
    k_cache = torch.randn(num_pages, nkv, page, hd, generator=g).to(dtype)
    v_cache = torch.randn(num_pages, nkv, page, hd, generator=g).to(dtype)
    T = sum(q_lens)
    q = torch.randn(T, nh * hd, generator=g)
    ks, vs, nxt = [], [], 0
    for b in range(B):
        k, v = torch.randn(nkv, totals[b], hd, generator=g), torch.randn(nkv, totals[b], hd, generator=g)
        p_last = totals[b] - 1
        lo = max(0, p_last - window + 1) if window else 0
        spots = [s for s in (keep - 1, keep, lo - 1, lo) if 0 <= s <= p_last]
        if spots:
            spot = spots[b % len(spots)]
            t_last = sum(q_lens[:b + 1]) - 1
            for h in range(nh):
                k[h // (nh // nkv), spot] = q[t_last, h * hd:(h + 1) * hd] * 2.0 / (scale * hd ** 0.5 * 4)
        k, v = k.to(dtype), v.to(dtype)
        ks.append(k.double()); vs.append(v.double())
        for i in range((totals[b] + page - 1) // page):
            pg = perm[nxt]; nxt += 1
            table[b, i] = pg
            n = min(page, totals[b] - i * page)
            k_cache[pg, :, :n] = k[:, i * page:i * page + n]
            v_cache[pg, :, :n] = v[:, i * page:i * page + n]
    q = q.to(dtype)
    want = torch.zeros(T, nh * hd, dtype=torch.float64)
    t0 = 0
    for b in range(B):
        for j in range(q_lens[b]):
            p = ctx_before[b] + j
            keys = torch.arange(p + 1)
            seen = ((p - keys < window) | (keys < keep)) if window else torch.ones(p + 1, dtype=torch.bool)
            qq = q[t0 + j].double().view(nh, 1, hd)
            kk = ks[b][:, :p + 1].repeat_interleave(nh // nkv, 0)
            vv = vs[b][:, :p + 1].repeat_interleave(nh // nkv, 0)
            s = torch.matmul(qq, kk.transpose(-1, -2)) * scale
            if cap:
                s = cap * torch.tanh(s / cap)
            s = s.masked_fill(~seen[None, None, :], -math.inf)
            want[t0 + j] = torch.matmul(torch.softmax(s, -1), vv).reshape(-1)
        t0 += q_lens[b]
    cu = i32([0] + torch.tensor(q_lens).cumsum(0).tolist())
    return dict(q=q.to(DEV), k=k_cache.to(DEV), v=v_cache.to(DEV), table=table.to(DEV), cu=cu, ctx=i32(ctx_before), want=want, T=T)


KEPT = [
    # nh, nkv, hd, page, q_lens, ctx_before, window, keep, cap, scale
    (4, 2, 16, 4, [5, 1, 17, 1], [0, 9, 30, 3], 8, 3, 6.0, 0.4),
    (4, 2, 64, 16, [200, 1, 1, 130, 1], [0, 120, 123, 150, 700], 120, 5, 40.0, 0.11),       # sizes the tensor cores take whole
    (2, 2, 32, 8, [33, 1, 1, 2], [100, 69, 70, 300], 20, 70, 0.0, 0.3),                        # more kept keys than the window holds, in two tiles
    (6, 3, 48, 16, [1, 1, 1, 1], [15, 16, 17, 400], 16, 1, 3.0, 0.2),
    (2, 1, 128, 32, [140, 1], [120, 513], 65, 33, 30.0, 0.09),
    (3, 3, 80, 2, [9, 1], [30, 77], 12, 0, 10.0, 0.1),                                         # a window alone, capped
    (4, 4, 16, 16, [40, 1], [0, 90], None, 0, 5.0, 0.5),                                       # every key, capped
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", KEPT)
def test_kept_keys_and_capped_scores_on_the_32_bit_pipes(case, dtype):
    from lyapunov_engine_b200 import ops
    nh, nkv, hd, page, q_lens, ctx_before, window, keep, cap, scale = case
    c = build_attention(dtype, nh, nkv, hd, page, q_lens, ctx_before, hd + page, window, keep, cap, scale)
    out = torch.zeros(c["T"], nh * hd, dtype=dtype, device=DEV)
    status = ops.new_status(DEV)
    tr, tq, n = tiles(q_lens, 16)
    ops.attention_generic(out, c["q"], c["q"].stride(0), c["k"], c["v"], c["table"], c["cu"], c["ctx"], tr, tq, n, nh, nkv, hd,
                          page, window, scale, status, keep_first=keep, softcap=cap)
    ops.check_status(status)
    torch.testing.assert_close(out.double().cpu(), c["want"], **tol_of(dtype, tight=1e-4))


@pytest.mark.parametrize("splits", [1, 2, 5])
@pytest.mark.parametrize("case", [k for k in KEPT if k[2] <= 128])
def test_kept_keys_and_capped_scores_on_the_tensor_cores(case, splits):
    """Requests with several tokens go to the prefill kernel, single tokens to
    the split-key decode kernel (the kept keys and the window as one axis that
    the splits cut), exactly as in a mixed step."""
    from lyapunov_engine_b200 import ops
    nh, nkv, hd, page, q_lens, ctx_before, window, keep, cap, scale = case
    dtype = torch.bfloat16
    c = build_attention(dtype, nh, nkv, hd, page, q_lens, ctx_before, hd + page + 1, window, keep, cap, scale)
    assert ops.attention_mma_available(hd)
    out = torch.zeros(c["T"], nh * hd, dtype=dtype, device=DEV)
    status = ops.new_status(DEV)
    multi = [b for b, n in enumerate(q_lens) if n > 1]
    single = [b for b, n in enumerate(q_lens) if n == 1]
    if multi:
        req, q0 = [], []
        for b in multi:
            for s in range(0, q_lens[b], 128):
                req.append(b); q0.append(s)
        ops.attention_prefill_bf16(out, c["q"], c["q"].stride(0), c["k"], c["v"], c["table"], c["cu"], c["ctx"], i32(req), i32(q0),
                                   len(req), nh, nkv, hd, page, window, scale, status, keep_first=keep, softcap=cap)
    if single:
        floats = ops.attention_decode_scratch_floats(hd, len(single), nh, splits)
        scratch = torch.zeros(max(floats, 1), device=DEV)
        ops.attention_decode_bf16(out, scratch, c["q"], c["q"].stride(0), c["k"], c["v"], c["table"], c["cu"], c["ctx"],
                                  i32(single), len(single), nh, nkv, hd, page, window, scale, splits, status,
                                  keep_first=keep, softcap=cap)
    ops.check_status(status)
    torch.testing.assert_close(out.double().cpu(), c["want"], atol=2e-2, rtol=2e-2)


# ------------------------------------------------------------------ routed experts: sigmoid scores, weight on the input
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(5, 48, 6, 2), (70, 64, 16, 1), (3, 20, 1, 1), (9, 32, 4, 4)])
def test_router_with_sigmoid_scores(shape, dtype):
    from lyapunov_engine_b200 import ops
    T, W, E, top = shape
    g = torch.Generator().manual_seed(T + E)
    h, wr = torch.randn(T, W, generator=g).to(dtype), torch.randn(E, W, generator=g)
    ids = torch.zeros(T, top, dtype=torch.int32, device=DEV)
    share = torch.zeros(T, top, device=DEV)
    ops.moe_route(ids, share, None, h.to(DEV), wr.to(DEV), None, None, top, scoring=ops.MOE_SIGMOID)
    z = h.double() @ wr.double().T
    want = torch.topk(z, top, dim=-1)
    assert torch.equal(ids.cpu().long(), want.indices)
    torch.testing.assert_close(share.double().cpu(), torch.sigmoid(want.values), atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(5, 48, 40, 6, 2), (300, 128, 128, 4, 1), (3, 24, 20, 1, 1)])
def test_an_experts_weight_on_its_input(shape, dtype):
    """The routed feed-forward as a part, weights on the experts' inputs,
    against the plain function; rows enough for the tensor-core products too."""
    from lyapunov_engine_b200 import ops
    from lyapunov_engine_b200.engine.runtime import Runtime
    from lyapunov_engine_b200.parts.base import FEED_FORWARDS, PartSpec
    T, W, F, E, top = shape
    g = torch.Generator().manual_seed(T + E)
    w = {f"m.e{e}.{part}": (torch.randn(*(s), generator=g) / math.sqrt(s[1])).to(torch.bfloat16).double()
         for e in range(E) for part, s in (("gate", (F, W)), ("up", (F, W)), ("down", (W, F)))}
    w["m.router"] = (4 * torch.randn(E, W, generator=g) / math.sqrt(W)).to(torch.bfloat16).double()
    h = torch.randn(T, W, generator=g).to(dtype)
    part = FEED_FORWARDS.build(PartSpec("routed_experts", {
        "hidden_size": W, "intermediate_size": F, "num_experts": E, "top": top, "router_name": "m.router",
        "router_bias_name": None, "expert_names": "m.e{expert}.{part}", "scoring": "sigmoid", "weight_on": "input"}))
    rt = Runtime(DEV, dtype)
    part.bind(lambda name: w[name].to(torch.float32 if name.endswith("router") else dtype).to(DEV), rt)

    class Ctx:
        workspace, status = rt.workspace, rt.status
    out = part.forward(h.to(DEV), Ctx)
    ops.check_status(rt.status)
    want = pr.routed_experts(h.double(), w, "m.", {"router": {"experts": E, "top": top}}, None)
    torch.testing.assert_close(out.double().cpu(), want, **tol_of(dtype, tight=1e-4, loose=4e-2))


# ------------------------------------------------------------------ small pieces
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("partials", [0, 1, 3])
@pytest.mark.parametrize("width", [96, 100, 2048])
def test_layer_scale_in_the_norms_kernel(width, partials, dtype):
    from lyapunov_engine_b200 import ops
    g = torch.Generator().manual_seed(width)
    T = 5
    resid, w, ls = torch.randn(T, width, generator=g), 1 + 0.1 * torch.randn(width, generator=g), torch.rand(width, generator=g) + 0.3
    delta = torch.randn(max(partials, 1), T, width, generator=g) if partials else torch.randn(T, width, generator=g).to(dtype)
    r = resid.clone().to(DEV)
    out = torch.zeros(T, width, dtype=dtype, device=DEV)
    ops.rmsnorm(out, r, delta.to(DEV), w.to(DEV), 1e-5, delta_scale=ls.to(DEV))
    total = resid.double() + ls.double() * (delta.double().sum(0) if partials else delta.double())
    torch.testing.assert_close(r.double().cpu(), total, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(out.double().cpu(), pr.unit_rms(total, 1e-5) * w.double(), **tol_of(dtype))
    rows = i32([3, 0])
    r2 = resid.clone().to(DEV)
    out2 = torch.zeros(2, width, dtype=dtype, device=DEV)
    ops.rmsnorm(out2, r2, delta.to(DEV), w.to(DEV), 1e-5, rows=rows, delta_scale=ls.to(DEV))
    torch.testing.assert_close(out2.double().cpu(), (pr.unit_rms(total, 1e-5) * w.double())[[3, 0]], **tol_of(dtype))
    assert torch.equal(r2.cpu(), resid)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("channels,taps", [(24, 4), (20, 2), (64, 1)])
def test_convolution_with_bias_and_silu_under_cuts(channels, taps, dtype):
    from lyapunov_engine_b200 import ops
    g = torch.Generator().manual_seed(channels)
    lens, cuts = (21, 6), ((1, 2, 18), (2, 4))
    w_taps, bias = 0.5 * torch.randn(channels, taps, generator=g), 0.3 * torch.randn(channels, generator=g)
    seqs = [torch.randn(n, channels + 8, generator=g).to(dtype).float() for n in lens]
    want = [pr.silu(pr.causal_conv(x[:, :channels].double(), w_taps.double(), bias.double())) for x in seqs]
    state = torch.full((3, max(taps - 1, 1), channels), 9.0, device=DEV)
    got = [[] for _ in seqs]

    def run_step(live, q_lens, starts, slots, fresh):
        for s, f in zip(slots, fresh):
            if f:
                state[s].zero_()
        rows = torch.cat([seqs[r][a:a + n] for r, n, a in zip(live, q_lens, starts)]).to(dtype).to(DEV)
        out = torch.zeros(rows.shape[0], channels, dtype=dtype, device=DEV)
        cu = i32([0] + torch.tensor(q_lens).cumsum(0).tolist())
        tr, tq, n = tiles(q_lens, ops.SHORT_CONV_TILE)
        ops.short_conv_general(out, rows[:, :channels], w_taps.t().contiguous().to(DEV), state if taps > 1 else None, i32(slots),
                               cu, tr, tq, n, add_input=False, silu=True, bias=bias.to(DEV))
        t0 = 0
        for r, n in zip(live, q_lens):
            got[r].append(out[t0:t0 + n].double().cpu())
            t0 += n

    feed_in_cuts(lens, cuts, 3, run_step)
    for r in range(len(seqs)):
        torch.testing.assert_close(torch.cat(got[r]), want[r], **tol_of(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_gate_per_entry_and_the_scaled_embedding(dtype):
    from lyapunov_engine_b200 import ops
    g = torch.Generator().manual_seed(1)
    x, gate = torch.randn(6, 40, generator=g).to(dtype), torch.randn(6, 72, generator=g).to(dtype)
    out = torch.zeros(6, 64, dtype=dtype, device=DEV)
    ops.sigmoid_gate(out[:, 8:48], x.to(DEV), gate.to(DEV)[:, 16:56], 0.6)
    torch.testing.assert_close(out[:, 8:48].double().cpu(), x.double() * torch.sigmoid(gate.double()[:, 16:56]) * 0.6, **tol_of(dtype))
    assert float(out[:, :8].abs().max()) == 0.0 and float(out[:, 48:].abs().max()) == 0.0
    table = torch.randn(11, 24, generator=g).to(dtype)
    resid = torch.zeros(3, 24, device=DEV)
    status = ops.new_status(DEV)
    ops.embed(resid, table.to(DEV), i32([10, 0, 4]), status, 17.5)
    ops.check_status(status)
    torch.testing.assert_close(resid.cpu(), table[[10, 0, 4]].float() * 17.5, atol=1e-6, rtol=1e-6)
