"""Each mechanism of the Zepilix design alone, the kernel against the plain
function of tests/plain_zepilix.py in 64 bits: the gated delta rule under
every cut of a sequence into steps (state rows used again, a write far back
that decides a read), its gated norm per head, the convolution with silu, the
turn of neighbouring pairs with the weightless norm behind it and its cache
write (the values are the keys as projected), the latent with its turned key
part, the pair of norms that lets a normed addend into the stream, the gated
row of a token's table, what a pass adds before its first layer, and the
feed-forward's biases in the epilogues of the gated products."""
import math

import pytest
import torch

import plain_zepilix as pz

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def i32(values):
    return torch.tensor(list(values), dtype=torch.int32, device=DEV)


def _tiles(q_lens, size):
    req, q0 = [], []
    for b, n in enumerate(q_lens):
        for s in range(0, n, size):
            req.append(b); q0.append(s)
    return i32(req), i32(q0), len(req)


def tol_of(dtype, tight=1e-5, loose=2e-2):
    return dict(atol=tight, rtol=tight) if dtype == torch.float32 else dict(atol=loose, rtol=loose)


# ------------------------------------------------------------------ the gated delta rule
def plain_delta(q, k, v, a, b, a_log, dt_bias, H, G, d, e):
    """q, k [T, G, d] before they are made unit vectors, v [T, H, e], a, b [T, H]: o [T, H, e] in 64 bits."""
    q, k, v, a, b = (x.double() for x in (q, k, v, a, b))
    qn = q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    kn = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    g = torch.exp(-torch.exp(a_log.double())[None] * torch.nn.functional.softplus(a + dt_bias.double()[None]))
    beta = torch.sigmoid(b)
    return torch.stack([pz.delta_rule_head(qn[:, j // (H // G)], kn[:, j // (H // G)], v[:, j], g[:, j], beta[:, j])
                        for j in range(H)], dim=1)


def run_delta(seqs, cuts, slots_of, state_rows, H, G, d, e, a_log, dt_bias, dtype, stale=7.0):
    """Feeds every sequence (q, k, v, a, b) in its cuts, the live requests of a
    step as one batch, from state rows that hold ``stale`` numbers."""
    from lyapunov_engine_b200 import ops
    C = 2 * G * d + H * e
    state = torch.full((state_rows, H, e, d), stale, device=DEV)
    got = [[] for _ in seqs]
    at = [0] * len(seqs)
    step = 0
    while any(step < len(c) for c in cuts):
        live = [r for r in range(len(seqs)) if step < len(cuts[r])]
        q_lens = [cuts[r][step] for r in live]
        rows_qkv, rows_ab = [], []
        for r, n in zip(live, q_lens):
            q, k, v, a, b = (x[at[r]:at[r] + n] for x in seqs[r])
            rows_qkv.append(torch.cat([q.reshape(n, -1), k.reshape(n, -1), v.reshape(n, -1)], dim=1))
            rows_ab.append(torch.cat([b, a], dim=1))
        qkv = torch.cat(rows_qkv).to(dtype).to(DEV).contiguous()
        # the step sizes and decays stand at odd columns of wider rows, as they do behind a product
        ab = torch.zeros(qkv.shape[0], 3 + 2 * H + 5, dtype=dtype, device=DEV)
        ab[:, 3:3 + 2 * H] = torch.cat(rows_ab).to(dtype).to(DEV)
        cu = i32([0] + list(torch.tensor(q_lens).cumsum(0)))
        slots = i32(slots_of[r] for r in live)
        ops.zero_fresh_state(state, slots, i32(at[r] for r in live), len(live))
        out = torch.full((qkv.shape[0], H * e), 5.0, device=DEV)
        ops.gated_delta_scan(out, qkv, 0, G * d, 2 * G * d, ab, 3, 3 + H, a_log.to(DEV), dt_bias.to(DEV), state, slots, cu,
                             len(live), H, G, d, e, 1e-6, d ** -0.5)
        o = 0
        for r, n in zip(live, q_lens):
            got[r].append(out[o:o + n].cpu().view(n, H, e))
            o += n
            at[r] += n
        step += 1
    assert C == qkv.shape[1]
    return [torch.cat(g) for g in got], state


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,e", [(2, 1, 32, 32), (4, 2, 16, 24), (3, 3, 20, 12), (1, 1, 64, 100), (2, 1, 128, 64),
                                     (2, 2, 48, 16), (1, 1, 1, 1), (2, 1, 256, 40), (1, 1, 200, 130), (1, 1, 320, 8), (1, 1, 520, 4)])
def test_delta_rule_under_every_cut(H, G, d, e, dtype):
    """Three requests in cuts of unequal sizes, down to one token and across
    the kernel's tiles of tokens, on state rows that earlier requests left
    full; the result equals the recurrence over each whole sequence."""
    g = torch.Generator().manual_seed(H * 100 + d)
    lens = (37, 5, 70)
    a_log, dt_bias = torch.randn(H, generator=g) * 0.5 - 1.0, torch.randn(H, generator=g) * 0.5
    seqs = []
    for n in lens:
        q, k = torch.randn(n, G, d, generator=g), torch.randn(n, G, d, generator=g)
        v, a, b = torch.randn(n, H, e, generator=g), torch.randn(n, H, generator=g) * 2, torch.randn(n, H, generator=g) * 2
        seqs.append(tuple(x.to(dtype).float() for x in (q, k, v, a, b)))       # (what the kernel is given, exactly)
    want = [plain_delta(*s, a_log, dt_bias, H, G, d, e).float() for s in seqs]
    cuts = [[1, 1, 2, 1, 17, 1, 2, 12], [2, 1, 1, 1], [33, 1, 1, 1, 16, 1, 17]]
    got, _ = run_delta(seqs, cuts, [2, 0, 3], 5, H, G, d, e, a_log, dt_bias, dtype)
    for r in range(3):
        torch.testing.assert_close(got[r], want[r], atol=3e-5, rtol=3e-5)
    whole, state = run_delta(seqs[2:], [[lens[2]]], [1], 2, H, G, d, e, a_log, dt_bias, dtype)
    torch.testing.assert_close(whole[0], want[2], atol=3e-5, rtol=3e-5)
    assert float(state[0].min()) == 7.0                           # rows of no request of the step stay as they are


def test_delta_rule_a_far_write_decides_and_rows_of_no_request():
    """A key written once, 300 tokens back, with no decay since and every
    later key at right angles to it: reading with that key as the query gives
    its value back.  A state that loses the write, or decays where it must
    not, gives something else by the value's whole size."""
    from lyapunov_engine_b200 import ops
    H, G, d, e, T = 2, 1, 64, 48, 301
    g = torch.Generator().manual_seed(1)
    basis = torch.linalg.qr(torch.randn(d, d, generator=g))[0]
    k = basis[torch.randint(1, d, (T,), generator=g)].clone()
    k[0] = basis[0]
    q = k.clone()
    q[-1] = basis[0]
    v = torch.randn(T, H, e, generator=g)
    v[0] = 40.0 * torch.randn(H, e, generator=g)
    a = torch.full((T, H), -60.0)                    # softplus(-60) = 0: no decay
    b = torch.full((T, H), 60.0)                     # step size 1: a write replaces what the key held
    seq = (q.view(T, G, d), k.view(T, G, d), v, a, b)
    a_log, dt_bias = torch.zeros(H), torch.zeros(H)
    want = plain_delta(*seq, a_log, dt_bias, H, G, d, e).float()
    torch.testing.assert_close(want[-1], v[0] * d ** -0.5, atol=1e-4, rtol=1e-4)
    for cuts in ([[T]], [[250, 50, 1]], [[1] * T]):
        got, _ = run_delta([seq], cuts, [0], 1, H, G, d, e, a_log, dt_bias, torch.float32)
        torch.testing.assert_close(got[0], want, atol=1e-4, rtol=1e-4)
    # a row that stands for no request starts from zero, gives zeros and keeps nothing
    state = torch.full((1, H, e, d), 3.0, device=DEV)
    qkv = torch.cat([q[:2], k[:2], v[:2].reshape(2, -1)], dim=1).to(DEV).contiguous()
    ab = torch.zeros(2, 2 * H, device=DEV)
    out = torch.full((2, H * e), 5.0, device=DEV)
    ops.gated_delta_scan(out, qkv, 0, d, 2 * d, ab, 0, H, a_log.to(DEV), dt_bias.to(DEV), state, i32([-1]), i32([0, 2]), 1,
                         H, G, d, e, 1e-6, d ** -0.5)
    assert float(out.abs().max()) == 0.0 and float(state.min()) == 3.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H,e", [(1, 2, 32), (9, 3, 24), (70, 1, 100), (5, 4, 128), (3, 2, 5)])
def test_norm_per_head_with_gate(T, H, e, dtype):
    from lyapunov_engine_b200 import ops
    g = torch.Generator().manual_seed(T + e)
    o = torch.randn(T, H, e, generator=g) * 3.0
    z = torch.randn(T, H * e + 6, generator=g).to(dtype)
    w = 1.0 + 0.3 * torch.randn(e, generator=g)
    want = pz.unit_rms(o.double(), 1e-5) * w.double()[None, None] * pz.silu(z[:, 3:3 + H * e].double()).view(T, H, e)
    out = torch.zeros(T, H * e, dtype=dtype, device=DEV)
    ops.head_norm_gate(out, o.view(T, H * e).to(DEV), z.to(DEV)[:, 3:3 + H * e], w.to(DEV), 1e-5, H, e)
    torch.testing.assert_close(out.float().cpu(), want.float().view(T, H * e), **tol_of(dtype))


# ------------------------------------------------------------------ the convolution with silu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps,C", [(1, 72), (2, 200), (4, 200), (5, 52), (3, 37)])
def test_convolution_with_silu_on_the_first_columns_of_wider_rows(taps, C, dtype):
    """conv(x) then silu, without the token's own input beside the sum, on
    columns [0, C) of rows that go on behind them; two requests under cuts
    shorter than the taps, from state rows with stale inputs."""
    from lyapunov_engine_b200 import ops
    g = torch.Generator().manual_seed(taps * 10 + C)
    w = 0.6 * torch.randn(C, taps, generator=g)
    seqs = [torch.randn(n, C + 11, generator=g).to(dtype) for n in (29, 40)]
    want = [pz.conv_silu(s[:, :C].double(), w.double()).float() for s in seqs]
    cuts = [[1, 2, 1, 1, 20, 4], [3, 1, 1, 33, 2]]
    state = torch.full((3, taps - 1, C), 9.0, device=DEV) if taps > 1 else None
    wt = w.t().contiguous().to(DEV)
    got, at = [[], []], [0, 0]
    for step in range(6):
        live = [r for r in range(2) if step < len(cuts[r])]
        q_lens = [cuts[r][step] for r in live]
        h = torch.cat([seqs[r][at[r]:at[r] + n] for r, n in zip(live, q_lens)]).to(DEV)
        cu = i32([0] + list(torch.tensor(q_lens).cumsum(0)))
        slots = i32([2, 0][r] for r in live)
        if state is not None:
            ops.zero_fresh_state(state, slots, i32(at[r] for r in live), len(live))
        out = torch.zeros(h.shape[0], C, dtype=dtype, device=DEV)
        if all(n == 1 for n in q_lens):
            ops.short_conv_general(out, h[:, :C], wt, state, slots, cu, None, None, len(live), add_input=False, silu=True)
        else:
            tr, tq, n = _tiles(q_lens, ops.SHORT_CONV_TILE)
            ops.short_conv_general(out, h[:, :C], wt, state, slots, cu, tr, tq, n, add_input=False, silu=True)
        o = 0
        for r, n in zip(live, q_lens):
            got[r].append(out[o:o + n].float().cpu())
            o += n
            at[r] += n
    for r in range(2):
        torch.testing.assert_close(torch.cat(got[r]), want[r], **tol_of(dtype, loose=3e-2))


# ------------------------------------------------------------------ the turn of pairs, the norm behind it, the cache write
def _paged(positions_of, page, max_blocks, seed):
    """Per request its positions of the step; pages dealt out of order."""
    g = torch.Generator().manual_seed(seed)
    R = len(positions_of)
    order = torch.randperm(R * max_blocks, generator=g).view(R, max_blocks)
    positions = i32(p for ps in positions_of for p in ps)
    request_of = i32(r for r, ps in enumerate(positions_of) for _ in ps)
    return positions, request_of, order.to(torch.int32).to(DEV).contiguous(), R * max_blocks


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,rot,unit", [(4, 2, 32, 16, True), (3, 1, 24, 10, True), (2, 2, 64, 64, True),
                                            (8, 1, 128, 32, False), (1, 1, 16, 0, True), (2, 1, 80, 80, True)])
def test_turn_of_pairs_norm_and_cache_write(H, G, d, rot, unit, dtype):
    """Queries in place, keys into their pages, the values' pool receives the
    keys as projected.  Positions up to a million: the angle is position times
    rate in 32 bits."""
    from lyapunov_engine_b200 import ops
    from lyapunov_engine_b200.parts.rope import pair_rates
    page, base, eps = 8, 5e4, 1e-5
    positions_of = [[0, 1, 2, 3, 4, 5, 6, 7, 8, 9], [17], [30, 31, 32]]
    positions, request_of, table, pages = _paged(positions_of, page, 5, H + d)
    T = positions.numel()
    g = torch.Generator().manual_seed(d + rot)
    rows = (torch.randn(T, (H + G) * d + 8, generator=g) * 2.0).to(dtype)
    pos = positions.cpu().long()
    q = rows[:, :H * d].double().view(T, H, d)
    k = rows[:, H * d:(H + G) * d].double().view(T, G, d)
    tq, tk = pz.turn_pairs(q, pos, rot, base), pz.turn_pairs(k, pos, rot, base)
    if unit:
        tq, tk = pz.unit_rms(tq, eps), pz.unit_rms(tk, eps)
    dev_rows = rows.to(DEV)
    kc = torch.zeros(pages, G, page, d, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    status = ops.new_status(DEV)
    ops.rope_norm_store(dev_rows, kc, vc, pair_rates(max(rot, 2), base).to(DEV), positions, request_of, table, H, G, d, 0, rot,
                        eps if unit else None, d, page, True, True, status)
    ops.check_status(status)
    tol = tol_of(dtype, tight=2e-5)
    torch.testing.assert_close(dev_rows[:, :H * d].float().cpu().view(T, H, d), tq.float(), **tol)
    assert torch.equal(dev_rows[:, (H + G) * d:].cpu(), rows[:, (H + G) * d:])
    for t in range(T):
        r, p = int(request_of[t]), int(pos[t])
        pg = int(table[r, p // page])
        torch.testing.assert_close(kc[pg, :, p % page].float().cpu(), tk[t].float(), **tol)
        assert torch.equal(vc[pg, :, p % page].cpu(), rows[t, H * d:(H + G) * d].view(G, d))
    # far positions, queries only, the turn on a part in the middle of the head (columns [d - rot, d))
    far = i32([1000003, 65536, 999])
    rows3 = (torch.randn(3, H * d, generator=g)).to(dtype)
    dev3 = rows3.to(DEV)
    ops.rope_norm_store(dev3, None, None, pair_rates(max(rot, 2), base).to(DEV), far, i32([0, 0, 0]), table, H, 0, d, d - rot, rot,
                        None, d, 1, False, False, status)
    q3 = rows3.double().view(3, H, d).clone()
    q3[..., d - rot:] = pz.turn_pairs(q3[..., d - rot:].contiguous(), far.cpu().long(), rot, base)
    # (the 32-bit angle of position 1,000,003 times a rate near 1 is good to about 0.06 radians' worth of its last bits)
    torch.testing.assert_close(dev3.float().cpu().view(3, H, d)[1:], q3.float()[1:], atol=2e-2, rtol=2e-2)
    a32 = (torch.tensor(1000003.0) * pair_rates(max(rot, 2), base)).double()             # the angle as 32 bits make it
    if rot:
        x = rows3[0].double().view(H, d)[:, d - rot:]
        c, s = torch.cos(a32)[None, :rot // 2], torch.sin(a32)[None, :rot // 2]
        want0 = torch.stack([x[:, 0::2] * c - x[:, 1::2] * s, x[:, 1::2] * c + x[:, 0::2] * s], dim=-1).reshape(H, rot)
        torch.testing.assert_close(dev3.float().cpu().view(3, H, d)[0, :, d - rot:], want0.float(), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rank,rot,rank2", [(64, 16, 80), (40, 8, 56), (12, 4, 16), (16, 0, 8), (112, 16, 64), (50, 6, 20)])
def test_latent_norm_turned_key_part_and_cache_write(rank, rot, rank2, dtype):
    """A row holds the queries' latent, then the keys' latent and the turned
    part: the first is normed into rows of its own, the second normed and the
    third turned into the layer's one pool (zeros behind them)."""
    from lyapunov_engine_b200 import ops
    from lyapunov_engine_b200.parts.rope import pair_rates
    page, base, eps = 4, 1e6, 1e-5
    padded = (rank + rot + 15) // 16 * 16
    positions_of = [[3, 4, 5, 6, 7, 8], [0], [21, 22]]
    positions, request_of, table, pages = _paged(positions_of, page, 6, rank)
    T = positions.numel()
    g = torch.Generator().manual_seed(rank + rot)
    src = (torch.randn(T, rank2 + rank + rot + 3, generator=g) * 2.0).to(dtype)
    w, w2 = 1.0 + 0.3 * torch.randn(rank, generator=g), 1.0 + 0.3 * torch.randn(rank2, generator=g)
    pos = positions.cpu().long()
    c = pz.unit_rms(src[:, rank2:rank2 + rank].double(), eps) * w.double()[None]
    kr = pz.turn_pairs(src[:, rank2 + rank:rank2 + rank + rot].double().view(T, 1, rot), pos, rot, base)[:, 0]
    cq = pz.unit_rms(src[:, :rank2].double(), eps) * w2.double()[None]
    cache = torch.full((pages, 1, page, padded), 3.0, dtype=dtype, device=DEV)
    out2 = torch.zeros(T, rank2, dtype=dtype, device=DEV)
    status = ops.new_status(DEV)
    ops.latent_rope_store(src.to(DEV), rank2, rank, rot, padded, w.to(DEV), eps, pair_rates(max(rot, 2), base).to(DEV), cache,
                          positions, request_of, table, page, status, second=(0, rank2, w2.to(DEV), out2))
    ops.check_status(status)
    tol = tol_of(dtype, tight=2e-5)
    torch.testing.assert_close(out2.float().cpu(), cq.float(), **tol)
    for t in range(T):
        r, p = int(request_of[t]), int(pos[t])
        row = cache[int(table[r, p // page]), 0, p % page].float().cpu()
        torch.testing.assert_close(row[:rank], c[t].float(), **tol)
        torch.testing.assert_close(row[rank:rank + rot], kr[t].float(), **tol)
        assert float(row[rank + rot:].abs().sum()) == 0.0


# ------------------------------------------------------------------ the stream: two norms of one row, addends, inputs
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W,parts", [(96, 0), (256, 1), (100, 3), (2048, 2), (66, 0), (4100, 1)])
def test_pair_of_norms_with_a_normed_addend(W, parts, dtype):
    """The addend enters the 32-bit stream divided by its root mean square and
    times a plain weight; two norms with weights around zero read the new row."""
    from lyapunov_engine_b200 import ops
    g = torch.Generator().manual_seed(W + parts)
    T, eps, eps_a = 6, 1e-5, 1e-6
    x = torch.randn(T, W, generator=g) * 4.0
    y = torch.randn(max(parts, 1), T, W, generator=g)
    addend = (y if parts else y[0].to(dtype)).contiguous()
    ysum = addend.double().sum(0) if parts else addend.double()
    wa = 1.0 + 0.3 * torch.randn(W, generator=g)
    w1, w2 = 0.2 * torch.randn(W, generator=g), 0.2 * torch.randn(W, generator=g)
    new = x.double() + pz.unit_rms(ysum, eps_a) * wa.double()[None]
    want1, want2 = pz.offset_norm(new, w1.double(), eps), pz.offset_norm(new, w2.double(), eps)
    resid = x.clone().to(DEV)
    o1, o2 = (torch.zeros(T, W, dtype=dtype, device=DEV) for _ in range(2))
    # (the part hands the kernel 1 + w: the offset is folded into the weight once, when the weights are bound)
    ops.rmsnorm_pair(o1, o2, resid, (1.0 + w1).to(DEV), (1.0 + w2).to(DEV), eps, addend=addend.to(DEV), addend_weight=wa.to(DEV),
                     addend_eps=eps_a)
    torch.testing.assert_close(resid.cpu(), new.float(), atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(o1.float().cpu(), want1.float(), **tol_of(dtype, tight=2e-5))
    torch.testing.assert_close(o2.float().cpu(), want2.float(), **tol_of(dtype, tight=2e-5))
    # a plain addend, one norm
    resid = x.clone().to(DEV)
    ops.rmsnorm_pair(o1, None, resid, (1.0 + w1).to(DEV), None, eps, addend=addend.to(DEV))
    torch.testing.assert_close(resid.cpu(), (x.double() + ysum).float(), atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(o1.float().cpu(), pz.offset_norm(x.double() + ysum, w1.double(), eps).float(),
                               **tol_of(dtype, tight=2e-5))
    # chosen rows: the stream stays as it is, the addend still enters what is normed
    resid = x.clone().to(DEV)
    some = torch.zeros(2, W, dtype=dtype, device=DEV)
    ops.rmsnorm_pair(some, None, resid, (1.0 + w2).to(DEV), None, eps, addend=addend.to(DEV), addend_weight=wa.to(DEV),
                     addend_eps=eps_a, rows=i32([4, 1]))
    assert torch.equal(resid.cpu(), x)
    torch.testing.assert_close(some.float().cpu(), want2.float()[[4, 1]], **tol_of(dtype, tight=2e-5))
    # the addend alone
    resid = x.clone().to(DEV)
    ops.rmsnorm_pair(None, None, resid, None, None, eps, addend=addend.to(DEV), addend_weight=wa.to(DEV), addend_eps=eps_a)
    torch.testing.assert_close(resid.cpu(), new.float(), atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W,pa,pf", [(96, 0, 0), (256, 2, 0), (100, 0, 3), (2048, 1, 2)])
def test_sum_of_two_sub_layers_into_the_stream(W, pa, pf, dtype):
    from lyapunov_engine_b200 import ops
    g = torch.Generator().manual_seed(W + pa + pf)
    T = 5
    x = torch.randn(T, W, generator=g)
    a, f = torch.randn(max(pa, 1), T, W, generator=g), torch.randn(max(pf, 1), T, W, generator=g)
    a = (a if pa else a[0].to(dtype)).contiguous()
    f = (f if pf else f[0].to(dtype)).contiguous()
    bias = torch.randn(W, generator=g)
    total = lambda t, p: t.double().sum(0) if p else t.double()
    want = x.double() + total(a, pa) + total(f, pf) + bias.double()[None]
    resid, copy = x.clone().to(DEV), torch.zeros(T, W, dtype=dtype, device=DEV)
    ops.residual_add(resid, a.to(DEV), f.to(DEV), bias.to(DEV), copy)
    torch.testing.assert_close(resid.cpu(), want.float(), atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(copy.float().cpu(), want.float(), **tol_of(dtype))
    resid = x.clone().to(DEV)
    ops.residual_add(resid, a.to(DEV))
    torch.testing.assert_close(resid.cpu(), (x.double() + total(a, pa)).float(), atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D,col,width", [(16, 32, 64), (24, 0, 24), (5, 10, 15), (8, 8, 40), (256, 256, 1024)])
def test_gated_row_of_a_tokens_table(D, col, width, dtype):
    from lyapunov_engine_b200 import ops
    g = torch.Generator().manual_seed(D + col)
    T, V = 9, 50
    z = (torch.randn(T, D, generator=g) * 2.5).to(dtype)
    table = torch.randn(V, width, generator=g).to(dtype)
    ids = torch.randint(0, V, (T,), generator=g)
    want = pz.gelu_tanh(z.double()) * table.double()[ids][:, col:col + D]
    out = torch.zeros(T, D, dtype=dtype, device=DEV)
    status = ops.new_status(DEV)
    ops.gate_rows(out, z.to(DEV), table.to(DEV), col, ids.to(torch.int32).to(DEV), status)
    ops.check_status(status)
    torch.testing.assert_close(out.float().cpu(), want.float(), **tol_of(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W", [64, 100, 2048])
def test_what_a_pass_adds_before_its_first_layer(W, dtype):
    from lyapunov_engine_b200 import ops
    g = torch.Generator().manual_seed(W)
    T, V = 7, 30
    x, vec = torch.randn(T, W, generator=g), torch.randn(W, generator=g)
    table = torch.randn(V, W, generator=g).to(dtype)
    ids = torch.randint(0, V, (T,), generator=g)
    status = ops.new_status(DEV)
    for tb, vc in ((table, vec), (None, vec), (table, None)):
        resid = x.clone().to(DEV)
        ops.stream_entry(resid, tb.to(DEV) if tb is not None else None, ids.to(torch.int32).to(DEV),
                         vc.to(DEV) if vc is not None else None, status)
        want = x.double() + (tb.double()[ids] if tb is not None else 0.0) + (vc.double()[None] if vc is not None else 0.0)
        torch.testing.assert_close(resid.cpu(), want.float(), atol=1e-6, rtol=1e-6)
    ops.check_status(status)


# ------------------------------------------------------------------ the feed-forward's biases
@pytest.mark.parametrize("rows", [1, 5, 16, 64, 65, 200, 700])
def test_gate_and_up_biases_in_every_kernel(rows):
    """silu(x Wg^T + bg) * (x Wu^T + bu): the stand-alone kernel in both types,
    and in bfloat16 both product kernels that add the biases to their 32-bit
    sums before the activation.  The biases are as large as the products."""
    from lyapunov_engine_b200 import ops
    from lyapunov_engine_b200.engine.runtime import Workspace
    K, I = 256, 328
    g = torch.Generator().manual_seed(rows)
    x = torch.randn(rows, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * I, K, generator=g) * 0.08).to(torch.bfloat16)
    bias = torch.randn(2 * I, generator=g) * 1.5
    gu = x.double() @ w.double().t() + bias.double()[None]
    want = (pz.silu(gu[:, :I]) * gu[:, I:]).float()
    for dtype in (torch.float32, torch.bfloat16):
        out = torch.zeros(rows, I, dtype=dtype, device=DEV)
        ops.glu(out, (x.double() @ w.double().t()).to(dtype).to(DEV), bias=bias.to(DEV))
        torch.testing.assert_close(out.float().cpu(), want, **tol_of(dtype, loose=4e-2))
    ws = Workspace(torch.device(DEV))
    out = torch.zeros(rows, I, dtype=torch.bfloat16, device=DEV)
    ops.gated_linear_bias(out, x.to(DEV), w.to(DEV), bias.to(DEV), ws, ops.new_status(DEV))      # the kernel the step takes
    torch.testing.assert_close(out.float().cpu(), want, atol=2e-2, rtol=2e-2)
    out.zero_()
    ops.gemm_tc(out, x.to(DEV), w.to(DEV), gated=True, bias=bias.to(DEV))
    ops.check_status(ops.tc_status(DEV))
    torch.testing.assert_close(out.float().cpu(), want, atol=2e-2, rtol=2e-2)
    if rows <= 64:
        out.zero_()
        ops.gemm_skinny(out, x.to(DEV), w.to(DEV), gated=True, bias=bias.to(DEV))
        torch.testing.assert_close(out.float().cpu(), want, atol=2e-2, rtol=2e-2)
    out32 = torch.zeros(rows, I, dtype=torch.float32, device=DEV)
    ops.gated_linear_bias(out32, x.float().to(DEV), w.float().to(DEV), bias.to(DEV), ws, ops.new_status(DEV))
    torch.testing.assert_close(out32.cpu(), want, atol=2e-4, rtol=2e-4)
