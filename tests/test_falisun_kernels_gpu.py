"""The kernels that came with the Falisun design, each alone against the plain float64 statement of its mechanism
(tests/plain_falisun.py), at sizes of their own: the normed and scaled join, the latent cache row and the rotation, the
per-head products, attention over latent rows (far keys, edges of pages, chunks and splits, the first positions, the
causal edge), the short convolution and the state-space scan across cuts and slots, the grouped norm, the router and the
experts' products."""
import math

import pytest
import torch

import plain_falisun as P

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
F64 = torch.float64


@pytest.fixture(scope="module")
def ops():
    from mini_llm_b200 import ops as o
    o.library()
    return o


def rnd(*shape, seed=0, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def _tol(dtype):
    return 2e-5 if dtype == torch.float32 else 1.2e-2


def _rel(got, want):
    return (got.double().cpu() - want).abs().max().item() / max(1.0, want.abs().max().item())


class _Ctx:
    """What the kernels read of a step: (context length, new tokens) per request."""

    def __init__(self, seqs, slots=None):
        from mini_llm_b200.engine.context import Workspace
        token_seq, positions, cu = [], [], [0]
        for s, (c, ql) in enumerate(seqs):
            token_seq += [s] * ql
            positions += list(range(c - ql, c))
            cu.append(cu[-1] + ql)
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
        self.token_seq, self.positions, self.cu_q = i32(token_seq), i32(positions), i32(cu)
        self.state_slots = i32(slots if slots is not None else list(range(len(seqs))))
        self.T, self.S = len(token_seq), len(seqs)
        self.max_ctx_len = max(c for c, _ in seqs)
        self.ws = Workspace(torch.device(DEV), 64)


# ------------------------------------------------------------------------------------------------ join
@pytest.mark.parametrize("R,D,eps", [(5, 48, 1e-5), (3, 1001, 1e-3), (2, 4096, 1e-6), (1, 8, 0.5)])
def test_norm_scale_add(ops, R, D, eps):
    y, x = rnd(R, D, seed=1, scale=3.0), rnd(R, D, seed=2)
    w, ls = rnd(D, seed=3) + 1.0, rnd(D, seed=4, scale=0.5)
    want = x.double().cpu() + P.rms_norm(y.double().cpu(), w.double().cpu(), eps) * ls.double().cpu()
    ops.norm_scale_add(y, w, ls, x, eps)
    assert _rel(x, want) < 2e-6
    x2 = torch.zeros(R, D, device=DEV)
    ops.norm_scale_add(y, w, None, x2, eps)
    assert _rel(x2, P.rms_norm(y.double().cpu(), w.double().cpu(), eps)) < 2e-6
    tiny = torch.full((1, 64), 1e-4, device=DEV)        # eps stands inside the root
    out = torch.zeros(1, 64, device=DEV)
    ops.norm_scale_add(tiny, torch.ones(64, device=DEV), None, out, 1e-2)
    assert abs(out[0, 0].item() - 1e-4 / math.sqrt(1e-8 + 1e-2)) < 1e-9


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("R,D,top,eps", [(5, 48, 2, 1e-5), (3, 1001, 1, 1e-3), (2, 4096, 3, 1e-6), (33, 20000, 2, 1e-5)])
def test_join_takes_the_weighted_pairs_and_norms_for_the_next_branch(ops, out_dtype, R, D, top, eps):
    """One kernel: the weighted sum over a token's experts (with or without a result to add it to), the norm and scale
    of that sum, the residual sum, and the next branch's norm of the new stream (plain weights or weights around zero)."""
    y, x0 = rnd(R, D, seed=1, scale=3.0), rnd(R, D, seed=2)
    w, ls, nw = rnd(D, seed=3) + 1.0, rnd(D, seed=4, scale=0.5), rnd(D, seed=5, scale=0.3) + 0.2
    pairs, pw = rnd(R * top, D, seed=6, scale=2.0), torch.rand(R, top, generator=torch.Generator().manual_seed(7)).to(DEV)
    mix = (pw.double().cpu()[:, :, None] * pairs.double().cpu().view(R, top, D)).sum(1)
    for with_y in (True, False):
        for offset in (0.0, 1.0):
            x = x0.clone()
            h = torch.zeros(R, D, device=DEV, dtype=out_dtype)
            ops.norm_scale_add(y if with_y else None, w, ls, x, eps, pairs=pairs, pair_weights=pw, top=top, next_weight=nw,
                               next_eps=2 * eps, next_offset=offset, next_out=h)
            v = mix + (y.double().cpu() if with_y else 0.0)
            want = x0.double().cpu() + P.rms_norm(v, w.double().cpu(), eps) * ls.double().cpu()
            assert _rel(x, want) < 2e-6
            assert _rel(h, P.rms_norm(want, nw.double().cpu() + offset, 2 * eps)) < (2e-6 if out_dtype == torch.float32 else 1e-2)
    x = x0.clone()
    ops.norm_scale_add(None, w, None, x, eps, pairs=pairs, pair_weights=pw, top=top)
    assert _rel(x, x0.double().cpu() + P.rms_norm(mix, w.double().cpu(), eps)) < 2e-6


# ------------------------------------------------------------------------------------------------ latent rows, rotation
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,dn,dr,R,dims,scaling", [(3, 16, 8, 40, 8, dict(factor=4.0, original=32, fast=8.0, slow=1.0)),
                                                   (2, 8, 16, 136, 8, None), (1, 4, 4, 12, 0, None),
                                                   (5, 32, 64, 64, 64, dict(factor=40.0, original=4096, fast=32.0, slow=1.0))])
def test_latent_rows_and_rotated_queries(ops, dtype, H, dn, dr, R, dims, scaling):
    from mini_llm_b200.parts.rotary import rotary_table
    eps, page, base = 1e-5, 8, 50.0
    ctx = _Ctx([(700, 5), (3, 3), (4100, 2)])
    T = ctx.T
    dq, dk, row = dn + dr, R + dr, -(-(R + dr) // 8) * 8
    width = H * dq + dk + 3
    proj = rnd(T, width, seed=5, scale=1.5, dtype=dtype)
    nw = rnd(R, seed=6) * 0.3 + 1.0
    pages = torch.zeros(2 * T // page + 2, 1, page, row, dtype=dtype, device=DEV)
    slots = torch.randperm(pages.shape[0] * page, generator=torch.Generator().manual_seed(1))[:T].to(torch.int32).to(DEV)
    f, m = rotary_table(dims, base, scaling)
    freq = torch.tensor(f, dtype=F64).float().to(DEV)
    qa = torch.zeros(T, H * dk, device=DEV)
    ops.latent_prepare(proj, 0, H * dq, ctx, slots, freq, m, nw, eps, pages, qa, heads=H, dim=dn, rot_dim=dr, rank=R,
                       rot_dims=dims, write=True)
    pos = ctx.positions.cpu().long()
    d = proj.double().cpu()[:, H * dq:H * dq + dk]
    c = P.rms_norm(d[:, :R], nw.double().cpu(), eps)
    kr = P.rotate(d[:, R:], pos, dims, base, scaling)
    rows = pages.view(-1, row)[slots.long()].double().cpu()
    assert _rel(rows[:, :R], c) < _tol(dtype) and _rel(rows[:, R:dk], kr) < _tol(dtype)
    assert torch.all(rows[:, dk:] == 0) and pages.view(-1, row).abs().sum(1).count_nonzero().item() == T
    q = proj.double().cpu()[:, :H * dq].view(T, H, dq)
    qr = P.rotate(q[..., dn:].transpose(0, 1), pos, dims, base, scaling).transpose(0, 1)
    got = qa.view(T, H, dk)[..., R:]
    assert _rel(got, qr) < 2e-6               # also at positions in the thousands: the angle is the 32-bit product p * f
    # a layer that writes no row leaves the pages alone
    before = pages.clone()
    ops.latent_prepare(proj, 0, None, ctx, slots, freq, m, nw, eps, pages, qa, heads=H, dim=dn, rot_dim=dr, rank=R,
                       rot_dims=dims, write=False)
    assert torch.equal(before, pages)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H,N,K", [(1, 3, 40, 16), (37, 2, 136, 24), (70, 5, 8, 64), (5, 1, 65, 33)])
def test_headwise_linear(ops, dtype, T, H, N, K):
    x = rnd(T, H * (K + 4) + 2, seed=1, dtype=dtype)
    W = rnd(H, N, K, seed=2, scale=K ** -0.5, dtype=dtype)
    out = torch.zeros(T, H * (N + 3), device=DEV)
    ops.headwise_linear(x, K + 4, W, out, N + 3)
    xs = x.double().cpu()[:, :H * (K + 4)].view(T, H, K + 4)[..., :K]
    want = torch.einsum("thk,hnk->thn", xs, W.double().cpu())
    assert _rel(out.view(T, H, N + 3)[..., :N], want) < 2e-5 and torch.all(out.view(T, H, N + 3)[..., N:] == 0)
    # 32-bit in, the weights' dtype out, with a sigmoid gate
    y = rnd(T, H * K, seed=3)
    g = rnd(T, H * N + 8, seed=4, dtype=dtype)
    out2 = torch.zeros(T, H * N, dtype=dtype, device=DEV)
    ops.headwise_linear(y, K, W, out2, N, gate=g[:, 8:])
    want2 = torch.einsum("thk,hnk->thn", y.double().cpu().view(T, H, K), W.double().cpu()) \
        * torch.sigmoid(g.double().cpu()[:, 8:].view(T, H, N))
    assert _rel(out2.view(T, H, N), want2) < _tol(dtype)


@pytest.mark.parametrize("T,H,N,K", [(17, 3, 40, 16), (200, 2, 136, 72), (64, 5, 8, 64), (130, 1, 65, 8)])
def test_headwise_linear_on_tensor_cores(ops, T, H, N, K):
    """More than 16 tokens, bfloat16 weights, 16-byte aligned rows: both directions against float64."""
    x = rnd(T, H * (K + 8) + 16, seed=1, dtype=torch.bfloat16)
    W = rnd(H, N, K, seed=2, scale=K ** -0.5, dtype=torch.bfloat16)
    out = torch.zeros(T, H * (N + 3), device=DEV)
    ops.headwise_linear(x[:, :H * (K + 8)], K + 8, W, out, N + 3)
    xs = x.double().cpu()[:, :H * (K + 8)].view(T, H, K + 8)[..., :K]
    want = torch.einsum("thk,hnk->thn", xs, W.double().cpu())
    assert _rel(out.view(T, H, N + 3)[..., :N], want) < 2e-5 and torch.all(out.view(T, H, N + 3)[..., N:] == 0)
    y = rnd(T, H * K, seed=3)
    g = rnd(T, H * N + 8, seed=4, dtype=torch.bfloat16)
    out2 = torch.zeros(T, H * N, dtype=torch.bfloat16, device=DEV)
    ops.headwise_linear(y, K, W, out2, N, gate=g[:, 8:])
    want2 = torch.einsum("thk,hnk->thn", y.double().cpu().view(T, H, K), W.double().cpu()) \
        * torch.sigmoid(g.double().cpu()[:, 8:].view(T, H, N))
    assert _rel(out2.view(T, H, N), want2) < 1.2e-2
    # the 32-bit inputs keep about 16 bits: against a 32-bit result of the same product the difference is far below bfloat16's
    out3 = torch.zeros(T, H * N, device=DEV)
    ops.headwise_linear(y, K, W.float(), out3, N)
    want3 = torch.einsum("thk,hnk->thn", y.double().cpu().view(T, H, K), W.double().cpu())
    assert _rel(out3.view(T, H, N), want3) < 2e-5


def _latent_case(dtype, seqs, H, R, dr, page, seed, sharp=None):
    """Cache rows in shuffled pages, queries for the new tokens.  ``sharp``: {request: [positions]}: the rows there answer
    a direction that all of the request's queries share with a score that stands out, so a row that is dropped, wrongly
    admitted or read from the wrong page moves the result by O(1)."""
    g = torch.Generator().manual_seed(seed)
    dk, row = R + dr, -(-(R + dr) // 8) * 8
    num_pages = sum((c + page - 1) // page for c, _ in seqs) + 3
    perm = torch.randperm(num_pages, generator=g).tolist()
    pages = torch.zeros(num_pages, 1, page, row)
    ctx = _Ctx(seqs)
    u = torch.randn(dk, generator=g)
    u /= u.norm()
    tables, dense, qs = [], [], []
    for s, (c, ql) in enumerate(seqs):
        tab = [perm.pop() for _ in range((c + page - 1) // page)]
        tables.append(tab)
        rows = torch.randn(c, dk, generator=g)
        q = torch.randn(ql, H, dk, generator=g)
        if sharp and s in sharp:
            rows, q = 0.3 * rows, 0.3 * q
            rows -= (rows @ u)[:, None] * u[None, :]
            for j in sharp[s]:
                rows[j] += 6.0 * u
            q += 5.0 * u
        rows = rows.to(dtype).float()
        dense.append(rows)
        qs.append(q)
        for j in range(c):
            pages[tab[j // page], 0, j % page, :dk] = rows[j]
    mp = max(len(t) for t in tables)
    bt = torch.zeros(len(seqs), mp + 2, dtype=torch.int32)
    for s, t in enumerate(tables):
        bt[s, :len(t)] = torch.tensor(t, dtype=torch.int32)
    return ctx, torch.cat(qs).reshape(ctx.T, H * dk).to(DEV), pages.to(dtype).to(DEV), bt.to(DEV), dense


def _latent_want(ctx, qa, dense, seqs, H, R, scale):
    out, t = [], 0
    dk = qa.shape[1] // H
    for s, (c, ql) in enumerate(seqs):
        rows = dense[s].double()
        for i in range(ql):
            p = c - ql + i
            q = qa[t].double().cpu().view(H, dk)
            w = torch.softmax((q @ rows[:p + 1].t()) * scale, -1)
            out.append((w @ rows[:p + 1, :R]).reshape(-1))
            t += 1
    return torch.stack(out)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,R,dr,page", [(3, 40, 8, 8), (10, 136, 16, 16), (1, 24, 4, 64), (17, 300, 2, 4)])
def test_latent_attention_mixed_batches(ops, dtype, H, R, dr, page):
    """Portions that start mid-page and mid-chunk beside single tokens, a portion of two tokens, a first token, contexts
    on both sides of a split of 256 keys."""
    seqs = [(300, 45), (1, 1), (257, 1), (256, 1), (19, 2), (600, 1), (70, 70)]
    scale = 0.3
    ctx, qa, pages, bt, dense = _latent_case(dtype, seqs, H, R, dr, page, seed=3)
    out = torch.zeros(ctx.T, H * R, device=DEV)
    ops.latent_attention(qa, pages, bt, ctx, out, heads=H, rank=R, scale=scale)
    assert _rel(out, _latent_want(ctx, qa, dense, seqs, H, R, scale)) < 2e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_attention_sharp_keys_at_every_edge(ops, dtype):
    """One dominant key among hundreds, placed at position 0, at the edges of pages (16), chunks (32) and splits (256), far
    back, and at the query's own position: a query sees it from its own position on and not one token earlier."""
    H, R, dr, page, scale = 4, 72, 8, 16, 1.0
    for j in (0, 15, 16, 31, 32, 255, 256, 511, 512, 700):
        # queries at j - 1 (must not see the key at j), j (its own position) and far later, in a prompt portion and alone
        seqs = [(j + 1, 2 if j else 1), (900, 1), (900, 130)] + ([(j, 1)] if j else [])
        sharp = {0: [j], 1: [j], 2: [j]}
        if j:
            sharp[3] = []
        ctx, qa, pages, bt, dense = _latent_case(dtype, seqs, H, R, dr, page, seed=10 + j, sharp=sharp)
        out = torch.zeros(ctx.T, H * R, device=DEV)
        ops.latent_attention(qa, pages, bt, ctx, out, heads=H, rank=R, scale=scale)
        want = _latent_want(ctx, qa, dense, seqs, H, R, scale)
        assert _rel(out, want) < 2e-5, j
        # the dominant row carries the result where it is visible
        seen = out[-1 if not j else -2].view(H, R).double().cpu()
        assert (seen - dense[2][j, :R].double()).abs().max() < 0.2 * dense[2][j, :R].abs().max(), j
        if j:
            first = out[0].view(H, R).double().cpu()            # the query at j - 1 of request 0
            assert (first - dense[0][j, :R].double()).abs().max() > 0.5 * dense[0][j, :R].abs().max(), j


@pytest.mark.parametrize("H,R,dr,page", [(3, 40, 8, 8), (2, 136, 8, 16), (1, 24, 8, 64), (5, 304, 16, 4), (2, 512, 64, 16)])
def test_latent_attention_on_tensor_cores(ops, H, R, dr, page):
    """The kernel for prompt portions over a bfloat16 cache against the plain statement and against the 32-bit kernel:
    tiles of up to 64 tokens that start mid-page and mid-tile, single tokens beside them, sharp keys at tile edges."""
    from mini_llm_b200.engine.context import attention_tiles
    seqs = [(300, 45), (1, 1), (257, 1), (33, 33), (19, 2), (600, 130), (64, 64)]
    for sharp in (None, {0: [0, 31, 32, 255, 256], 5: [469, 470, 511, 512, 599], 6: [63]}):
        scale = 1.0 if sharp else 0.3
        ctx, qa, pages, bt, dense = _latent_case(torch.bfloat16, seqs, H, R, dr, page, seed=4, sharp=sharp)
        tiles = attention_tiles([q for _, q in seqs], [c - q for c, q in seqs])
        ctx.attn_tiles, ctx.n_tiles, ctx.decode_only = torch.tensor(tiles, dtype=torch.int32, device=DEV), len(tiles) // 3, False
        out = torch.zeros(ctx.T, H * R, device=DEV)
        n0 = ops.attention_launches.get("latent_mma", 0)
        ops.latent_attention(qa, pages, bt, ctx, out, heads=H, rank=R, scale=scale)
        assert ops.attention_launches.get("latent_mma", 0) == n0 + 1
        want = _latent_want(ctx, qa, dense, seqs, H, R, scale)
        # queries enter as hi + lo bfloat16 terms; rows beyond 568 columns leave no room for the lo term
        assert _rel(out, want) < (2e-4 if R + dr <= 568 else 3e-2)
        ref = torch.zeros(ctx.T, H * R, device=DEV)
        ops.latent_attention(qa, pages, bt, ctx, ref, heads=H, rank=R, scale=scale, impl="split")
        assert _rel(ref, want) < 2e-5
        # with queries that are bfloat16 numbers already, only the weights' 16 bits and ex2 are left
        qb = qa.to(torch.bfloat16).float()
        ops.latent_attention(qb, pages, bt, ctx, out, heads=H, rank=R, scale=scale)
        assert _rel(out, _latent_want(ctx, qb, dense, seqs, H, R, scale)) < 2e-4


def test_latent_attention_gives_a_token_the_same_bits_alone_and_in_a_portion(ops):
    H, R, dr, page = 5, 48, 8, 8
    ctx, qa, pages, bt, _ = _latent_case(torch.float32, [(400, 100)], H, R, dr, page, seed=2)
    out = torch.zeros(ctx.T, H * R, device=DEV)
    ops.latent_attention(qa, pages, bt, ctx, out, heads=H, rank=R, scale=0.2)
    for i in (0, 37, 99):
        one = _Ctx([(301 + i, 1)])
        o1 = torch.zeros(1, H * R, device=DEV)
        ops.latent_attention(qa[i:i + 1].contiguous(), pages, bt, one, o1, heads=H, rank=R, scale=0.2)
        assert torch.equal(o1[0], out[i])


# ------------------------------------------------------------------------------------------------ state-space mixer
def _ssd_run(ops, dtype, Hm, Pd, N, G, taps, cuts_per_request, slots, seed):
    """Runs conv + scan over requests cut into portions, several requests per step; returns (got y, want y) per request."""
    g = torch.Generator().manual_seed(seed)
    inner, C = Hm * Pd, Hm * Pd + 2 * G * N
    width = 2 * inner + 2 * G * N + Hm
    lens = [sum(c) for c in cuts_per_request]
    proj = [(torch.randn(n, width, generator=g) * 1.3).to(dtype) for n in lens]
    cw, cb = torch.randn(C, taps, generator=g) * 0.6, torch.randn(C, generator=g) * 0.2
    dtb = torch.empty(Hm).uniform_(-4.0, 1.0, generator=g)
    A_log = torch.empty(Hm).uniform_(-3.0, 1.5, generator=g)
    A_log[0] = -12.0                                   # a head that never forgets ...
    if Hm > 1:
        A_log[1] = 4.0                                 # ... next to one that forgets at once
    Dh = torch.empty(Hm).uniform_(0.3, 1.5, generator=g)
    ssm = Hm * N * Pd
    state = torch.zeros(max(slots) + 2, ssm + (taps - 1) * C, device=DEV)
    state[[s for s in range(state.shape[0]) if s not in slots]] = 7.0          # other requests' slots: never touched
    got = [[] for _ in lens]
    at = [0] * len(lens)
    dev = lambda t: t.to(DEV)
    steps = max(len(c) for c in cuts_per_request)
    for k in range(steps):
        who = [r for r, c in enumerate(cuts_per_request) if k < len(c) and c[k] > 0]
        if not who:
            continue
        seqs = [(at[r] + cuts_per_request[r][k], cuts_per_request[r][k]) for r in who]
        ctx = _Ctx(seqs, slots=[slots[r] for r in who])
        x = torch.cat([proj[r][at[r]:at[r] + cuts_per_request[r][k]] for r in who]).to(DEV)
        xbc = torch.zeros(ctx.T, C, device=DEV)
        ops.ssd_conv(x, inner, dev(cw), dev(cb), state, ssm, ctx, xbc)
        y = torch.zeros(ctx.T, inner, device=DEV)
        ops.ssd_scan(xbc, x, inner + C, dev(dtb), dev(A_log), dev(Dh), state, ctx, y, heads=Hm, vdim=Pd, state_rows=N, groups=G)
        o = 0
        for r in who:
            n = cuts_per_request[r][k]
            got[r].append(y[o:o + n].cpu())
            o += n
            at[r] += n
    want = []
    for r, n in enumerate(lens):
        p = proj[r].double()
        xbc = P.silu(P.short_convolution(p[:, inner:inner + C], cw.double(), cb.double()))
        dt = torch.nn.functional.softplus(p[:, inner + C:] + dtb.double()[None], threshold=1e9)
        want.append(P.selective_scan(xbc[:, :inner].reshape(n, Hm, Pd), xbc[:, inner:inner + G * N].reshape(n, G, N),
                                     xbc[:, inner + G * N:].reshape(n, G, N), dt, A_log.double(), Dh.double(), G).reshape(n, inner))
    untouched = [s for s in range(state.shape[0]) if s not in slots]
    assert torch.all(state[untouched] == 7.0)
    return [torch.cat(g_) for g_ in got], want, state


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Hm,Pd,N,G,taps", [(4, 12, 20, 2, 4), (6, 16, 64, 3, 3), (1, 40, 8, 1, 2), (2, 33, 130, 1, 1), (8, 4, 1, 8, 5)])
def test_convolution_and_scan_across_cuts_batches_and_slots(ops, dtype, Hm, Pd, N, G, taps):
    """Three requests of unequal length cut into unequal portions (down to one token, shorter than the convolution's reach),
    batched together, with slots given out of order; against each request run whole by the plain statement."""
    cuts = [[30, 2, 1, 1, 40, 1, 1, 14], [0, 2, 1, 1, 9, 0, 3], [1, 1, 1, 70, 0, 0, 0, 1, 17]]
    got, want, _ = _ssd_run(ops, dtype, Hm, Pd, N, G, taps, cuts, slots=[2, 0, 3], seed=5)
    for g_, w in zip(got, want):
        assert _rel(g_, w) < 3e-5
    # the state after all tokens is the same bits however they were cut
    _, _, s1 = _ssd_run(ops, dtype, Hm, Pd, N, G, taps, [[90]], slots=[1], seed=9)
    _, _, s2 = _ssd_run(ops, dtype, Hm, Pd, N, G, taps, [[1, 7, 33, 2, 16, 31]], slots=[1], seed=9)
    assert torch.equal(s1[1], s2[1])


def test_long_scan_keeps_what_a_slow_head_saw_at_the_start(ops):
    got, want, _ = _ssd_run(ops, torch.float32, 2, 8, 16, 1, 3, [[1500, 1, 1, 1]], slots=[0], seed=3)
    assert _rel(got[0][-3:], want[0][-3:]) < 3e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,W,groups", [(5, 48, 1), (9, 96, 3), (2, 2048, 2), (3, 40, 40)])
def test_gated_group_norm(ops, dtype, T, W, groups):
    eps = 1e-5
    y = rnd(T, W, seed=1, scale=2.0)
    z = rnd(T, W + 8, seed=2, dtype=dtype)
    w = rnd(W, seed=3) * 0.3 + 1.0
    out = torch.zeros(T, W + 16, dtype=dtype, device=DEV)
    ops.gated_group_norm(y, z[:, 8:], w, out[:, :W], groups, eps)
    v = y.double().cpu() * P.silu(z.double().cpu()[:, 8:])
    want = P.rms_norm(v.view(T, groups, W // groups), 1.0, eps).reshape(T, W) * w.double().cpu()
    assert _rel(out[:, :W], want) < _tol(dtype) and torch.all(out[:, W:] == 0)


# ------------------------------------------------------------------------------------------------ routed feed-forward
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,D,E,top,groups,keep,F,shared", [(50, 64, 12, 2, 2, 1, 24, 40), (1, 32, 4, 1, 1, 1, 16, None),
                                                            (130, 96, 8, 3, 4, 2, 40, None), (7, 40, 3, 3, 3, 3, 9, 5),
                                                            (300, 48, 64, 6, 8, 3, 8, None)])
def test_router_and_experts(ops, dtype, T, D, E, top, groups, keep, F, shared):
    from mini_llm_b200.engine.runner import Runtime
    from mini_llm_b200.parts.moe import MoEFeedForward
    h = rnd(T, D, seed=1, dtype=dtype)
    g = torch.Generator().manual_seed(2)
    w = {"router": torch.randn(E, D, generator=g) * 3.0 / math.sqrt(D)}
    names = [f"e{e}" for e in range(E)] + (["shared"] if shared else [])
    for n in names:
        Fn = shared if n == "shared" else F
        w[n + ".gate"], w[n + ".up"] = torch.randn(Fn, D, generator=g) / math.sqrt(D), torch.randn(Fn, D, generator=g) / math.sqrt(D)
        w[n + ".down"] = torch.randn(D, Fn, generator=g) / math.sqrt(Fn)
    w = {k: v.to(dtype) for k, v in w.items()}
    r = dict(experts=E, top=top, groups=dict(count=groups, keep=keep) if groups > 1 else None)
    wd = {k: v.double() for k, v in w.items()}
    hd = h.double().cpu()
    s, chosen, weights = P.route(hd, wd["router"], r)
    # the router alone: the same experts (as sets; no score is close to another here) and weights
    idx = torch.zeros(T, top, dtype=torch.int32, device=DEV)
    wt = torch.zeros(T, top, device=DEV)
    off = torch.zeros(E + 1, dtype=torch.int32, device=DEV)
    order = torch.zeros(T * top, dtype=torch.int32, device=DEV)
    ops.moe_route(h, w["router"].to(DEV), idx, wt, off, order, top=top, groups=groups, keep=keep)
    clear = torch.ones(T, dtype=torch.bool)      # both sides see the same inputs: no score is close enough to another to flip
    gi, gw = idx.cpu().long(), wt.double().cpu()
    for t in range(T):
        if clear[t]:
            assert sorted(gi[t].tolist()) == sorted(chosen[t].tolist()), t
            a = dict(zip(gi[t].tolist(), gw[t].tolist()))
            for e, v in zip(chosen[t].tolist(), weights[t].tolist()):
                assert abs(a[e] - v) < (1e-5 if dtype == torch.float32 else 1e-5) * max(1.0, v), t
    o = off.cpu().tolist()
    assert o[0] == 0 and o[-1] == T * top and all(a <= b for a, b in zip(o, o[1:]))
    od = order.cpu().long()
    assert sorted(od.tolist()) == list(range(T * top))
    flat = gi.reshape(-1)
    for e in range(E):
        assert torch.all(flat[od[o[e]:o[e + 1]]] == e)
    # the whole feed-forward through the part
    ff = MoEFeedForward(D, E, top, F, groups=groups, keep=keep, shared_size=shared)
    params = {"router": w["router"].to(DEV)}
    for e in range(E):
        for n in ("gate", "up", "down"):
            params[f"expert{e}.{n}"] = w[f"e{e}.{n}"].to(DEV)
    if shared:
        for n in ("gate", "up", "down"):
            params[f"shared.{n}"] = w[f"shared.{n}"].to(DEV)
    ff.bind(params, Runtime(dtype=dtype, device=torch.device(DEV)))
    ctx = _Ctx([(T, T)])
    y = torch.full((T, D), 3.0, device=DEV)
    ff.forward(h, ctx, y, accumulate=False)
    store = P.to_bf16 if dtype == torch.bfloat16 else P._keep
    want = P.mixture_of_experts(hd, wd, dict(router=r, shared=dict(ff=shared) if shared else None), store)
    err = (y.double().cpu() - want).norm(dim=1) / want.norm(dim=1).clamp(min=1e-9)
    assert (err[clear] < (3e-5 if dtype == torch.float32 else 1.5e-2)).all()
    y2 = torch.full((T, D), 3.0, device=DEV)
    ff.forward(h, ctx, y2, accumulate=True)
    assert (y2 - 3.0 - y).abs().max() < 1e-4 * max(1.0, y.abs().max().item())
