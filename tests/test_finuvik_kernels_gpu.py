"""The kernels that came with the Finuvik design, each alone against the plain float64 statement of its mechanism
(tests/plain_finuvik.py), at sizes of their own: RMS norm (single and paired), the gated activation, the cache
write, distance-bias attention in its three kernels, the gated linear recurrence."""
import math

import pytest
import torch

import plain_finuvik as P

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


# ------------------------------------------------------------------------------------------------ norm, activation
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,D", [(3, 40), (2, 33), (5, 256)])
def test_rmsnorm_per_head_into_a_column_slice(ops, out_dtype, heads, D):
    R, eps = 9, 1e-5
    x = rnd(R, heads * D, seed=1, scale=2.0)
    w = rnd(D, seed=2) + 1.0
    wide = torch.zeros(R, heads * D + 16, device=DEV, dtype=out_dtype)
    out = wide[:, 16:]
    ops.rmsnorm(x, w, eps, out, unit_offset=False, heads=heads, scale=0.6)
    want = 0.6 * P.rms_norm(x.double().cpu().view(R, heads, D), w.double().cpu(), eps, False).reshape(R, heads * D)
    assert (out.double().cpu() - want).abs().max() < _tol(out_dtype) * max(1.0, want.abs().max().item())
    assert torch.all(wide[:, :16] == 0)


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("R,D,eps", [(5, 48, 1e-5), (33, 1600, 1e-6), (3, 1001, 1e-3), (2, 4096, 1e-5), (1, 8, 0.5)])
def test_rmsnorm(ops, out_dtype, R, D, eps):
    x = rnd(R, D, seed=4, scale=3.0) + 0.5
    w1, w2 = rnd(D, seed=5, scale=0.3), rnd(D, seed=6, scale=0.3)
    for offset in (True, False):
        out = torch.empty(R, D, device=DEV, dtype=out_dtype)
        ops.rmsnorm(x, w1, eps, out, unit_offset=offset)
        want = P.rms_norm(x.double().cpu(), w1.double().cpu(), eps, offset)
        assert (out.double().cpu() - want).abs().max() < _tol(out_dtype) * max(1.0, want.abs().max().item())
    # two weight vectors from one sum of squares give what two calls give
    a, b = torch.empty(R, D, device=DEV, dtype=out_dtype), torch.empty(R, D, device=DEV, dtype=out_dtype)
    ops.rmsnorm(x, w1, eps, a, weight2=w2, out2=b)
    one = torch.empty(R, D, device=DEV, dtype=out_dtype)
    ops.rmsnorm(x, w1, eps, one)
    assert torch.equal(a, one)
    ops.rmsnorm(x, w2, eps, one)
    assert torch.equal(b, one)
    # gathered rows
    rows = torch.tensor([R - 1, 0, R - 1], dtype=torch.int32, device=DEV)
    out2 = torch.empty(3, D, device=DEV, dtype=out_dtype)
    ops.rmsnorm(x, w2, eps, out2, rows=rows)
    assert torch.equal(out2, one[rows.long()])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,N,K,eps", [(1, 96, 64, 1e-5), (8, 1184, 768, 1e-6), (16, 200, 1600, 1e-5), (3, 4096, 2048, 1e-5),
                                       (40, 64, 128, 1e-5)])
def test_products_take_an_rms_norm_into_their_loads(ops, dtype, M, N, K, eps):
    """A product whose input is an RMS norm that has not been evaluated: with few rows the streaming products norm the
    rows themselves (no centring, w + 1 as the factor), with more rows the norm is evaluated first; both against the
    oracle and against each other."""
    from mini_llm_b200.engine.context import Workspace
    ws = Workspace(torch.device(DEV), 64)
    x = rnd(M + 3, K, seed=31, scale=2.0) + 0.7
    w = rnd(K, seed=32, scale=0.2)
    W = rnd(N, K, seed=33, scale=K ** -0.5, dtype=dtype)
    rows = torch.tensor(list(range(M, 0, -1)), dtype=torch.int32, device=DEV)
    gamma, beta = (w + 1.0).contiguous(), torch.zeros_like(w)
    lazy = ops.NormedInput(x, gamma, beta, eps, rows, ws, dtype, rms=True)
    out = torch.empty(M, N, device=DEV, dtype=dtype)
    n0 = ops.launches
    ops.linear(lazy, W, None, out=out)
    fused = ops.launches - n0 == 1
    assert fused == (M <= 16)
    h = P.rms_norm(x.double().cpu()[rows.long().cpu()], w.double().cpu(), eps, True)
    if dtype == torch.bfloat16:
        h = P.to_bf16(h)
    want = h @ W.double().cpu().t()
    tol = 3e-5 if dtype == torch.float32 else 1.2e-2
    assert (out.double().cpu() - want).abs().max() < tol * max(1.0, want.abs().max().item())
    # the same through the norm kernel and the plain product
    hn = torch.empty(M, K, device=DEV, dtype=dtype)
    ops.rmsnorm(x, w, eps, hn, rows=rows, unit_offset=True)
    out2 = torch.empty(M, N, device=DEV, dtype=dtype)
    ops.linear(hn, W, None, out=out2)
    assert (out.double() - out2.double()).abs().max() < tol * max(1.0, want.abs().max().item())
    ops.check_device_errors()


def test_rmsnorm_keeps_eps_inside_the_root(ops):
    # a row of tiny values: x / sqrt(mean + eps) is far from x / (sqrt(mean) + eps)
    x = torch.full((1, 64), 1e-4, device=DEV)
    w = torch.zeros(64, device=DEV)
    out = torch.empty(1, 64, device=DEV)
    ops.rmsnorm(x, w, 1e-4, out)
    assert abs(out[0, 0].item() - 1e-4 / math.sqrt(1e-8 + 1e-4)) < 1e-8


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("act", ["relu", "silu", "gelu_tanh"])
def test_gated_act(ops, dtype, act):
    T, F = 37, 50
    wide = rnd(T, 2 * F + 6, seed=7, scale=2.0, dtype=dtype)
    gu = wide[:, :2 * F]
    out = torch.empty(T, F, device=DEV, dtype=dtype)
    ops.gated_act(gu, out, act)
    g, u = gu[:, :F].double(), gu[:, F:].double()
    f = {"relu": torch.relu, "silu": torch.nn.functional.silu,
         "gelu_tanh": lambda z: torch.nn.functional.gelu(z, approximate="tanh")}[act]
    want = f(g) * u
    assert (out.double() - want).abs().max() < _tol(dtype) * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_paged_write(ops, dtype):
    T, heads, d, page, pages = 19, 3, 20, 4, 11
    src = rnd(T, heads * d + 8, seed=8, dtype=dtype)[:, 8:]
    pool = torch.zeros(pages, heads, page, d, device=DEV, dtype=dtype)
    g = torch.Generator().manual_seed(9)
    slots = torch.randperm(pages * page, generator=g)[:T].to(torch.int32).to(DEV)
    ops.paged_write(src, pool, slots)
    for t in range(T):
        s = int(slots[t])
        assert torch.equal(pool[s // page, :, s % page].reshape(-1), src[t])
    assert int((pool != 0).sum()) <= T * heads * d


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dk,dkp", [(16, 16), (12, 16), (3, 8)])
def test_paged_write_kv(ops, dtype, dk, dkp):
    T, heads, dv, page, pages = 23, 2, 5, 8, 7
    wide = rnd(T, heads * (dk + dv) + 3, seed=8, dtype=dtype)
    k, v = wide[:, 3:3 + heads * dk], wide[:, 3 + heads * dk:]
    kp = torch.zeros(pages, heads, page, dkp, device=DEV, dtype=dtype)
    vp = torch.zeros(pages, heads, page, dv, device=DEV, dtype=dtype)
    g = torch.Generator().manual_seed(10)
    slots = torch.randperm(pages * page, generator=g)[:T].to(torch.int32).to(DEV)
    ops.paged_write_kv(k, v, kp, vp, slots)
    for t in range(T):
        s = int(slots[t])
        assert torch.equal(kp[s // page, :, s % page, :dk].reshape(-1), k[t])
        assert torch.equal(vp[s // page, :, s % page].reshape(-1), v[t])
    assert torch.all(kp[..., dk:] == 0)


# ------------------------------------------------------------------------------------------------ attention
class _Ctx:
    pass


def _case(dtype, seqs, H, G, dk, dv, page, seed, sharp=None, r=(0.5, 0.2)):
    """seqs: (context length, new tokens) per request.  Builds pages in a shuffled order, dense copies, the tile
    list and the tables of a head-wise distance bias and a query factor.  ``sharp``: {request: [positions]}: the
    keys there answer a component common to the request's queries with a score that stands out, and carry value
    rows of their own, so a key that is dropped or wrongly admitted moves the result by O(1)."""
    from mini_llm_b200.engine.context import Workspace, attention_tiles
    g = torch.Generator().manual_seed(seed)
    num_pages = sum((c + page - 1) // page for c, _ in seqs) + 3
    perm = torch.randperm(num_pages, generator=g).tolist()
    k_pages = torch.zeros(num_pages, G, page, -(-dk // 8) * 8)      # key rows padded to a multiple of 8, the padding zero
    v_pages = torch.zeros(num_pages, G, page, dv)
    tables, dense, token_seq, positions = [], [], [], []
    for s, (c, ql) in enumerate(seqs):
        tab = [perm.pop() for _ in range((c + page - 1) // page)]
        tables.append(tab)
        dense.append((torch.randn(c, G, dk, generator=g), torch.randn(c, G, dv, generator=g)))
        token_seq += [s] * ql
        positions += list(range(c - ql, c))
    T = len(token_seq)
    q = torch.randn(T, H * dk, generator=g)
    scale = dk ** -0.5
    if sharp:
        for s, where in sharp.items():
            u = torch.randn(G, dk, generator=g)
            u = u / u.norm(dim=1, keepdim=True) * math.sqrt(dk)
            rows = [t for t, ts in enumerate(token_seq) if ts == s]
            q[rows] = q[rows] * 0.3 + u.repeat_interleave(H // G, dim=0).reshape(1, H * dk) * 1.5
            K, V = dense[s]
            for i, p in enumerate(where):
                K[p] = u * (30.0 / math.sqrt(dk))           # score 1.5 * 30 = 45 before bias and factor
                V[p] = 2.0 * (i + 1)
    for s, tab in enumerate(tables):
        K, V = dense[s]
        for p in range(K.shape[0]):
            k_pages[tab[p // page], :, p % page, :dk] = K[p]
            v_pages[tab[p // page], :, p % page] = V[p]
    mp = max(len(t) for t in tables)
    bt = torch.zeros(len(seqs), mp, dtype=torch.int32)
    for s, t in enumerate(tables):
        bt[s, :len(t)] = torch.tensor(t, dtype=torch.int32)
    n = max(c for c, _ in seqs)
    r1 = torch.linspace(r[0], 2 * r[0], H, dtype=F64)
    r2 = torch.linspace(r[1], 3 * r[1], H, dtype=F64)
    dist_bias = (-r1[:, None] * torch.log1p(r2[:, None] * torch.arange(n, dtype=F64)[None])).float()
    q_scale = P.query_temperature(torch.arange(n), 0.4, 5).float()
    ctx = _Ctx()
    ctx.token_seq = torch.tensor(token_seq, dtype=torch.int32, device=DEV)
    ctx.positions = torch.tensor(positions, dtype=torch.int32, device=DEV)
    ctx.ws = Workspace(torch.device(DEV), 64)
    ctx.max_ctx_len = n
    ctx.decode_only = all(ql == 1 for _, ql in seqs)
    tiles = attention_tiles([ql for _, ql in seqs], [c - ql for c, ql in seqs])
    ctx.attn_tiles = torch.tensor(tiles, dtype=torch.int32, device=DEV)
    ctx.n_tiles = len(tiles) // 3
    return dict(q=q.to(dtype).to(DEV), k_pages=k_pages.to(dtype).to(DEV), v_pages=v_pages.to(dtype).to(DEV),
                bt=bt.to(DEV), token_seq=token_seq, positions=positions, dense=dense, ctx=ctx, scale=scale,
                dist_bias=dist_bias.to(DEV), q_scale=q_scale.to(DEV), H=H, G=G, dk=dk, dv=dv, dtype=dtype)


def _want(case, window=None, use_bias=True, use_qscale=True, out_scale=1.0):
    H, G, dk, dv, dtype = case["H"], case["G"], case["dk"], case["dv"], case["dtype"]
    q = case["q"].cpu().double()
    out = torch.zeros(q.shape[0], H * dv, dtype=F64)
    db, qs = case["dist_bias"].cpu().double(), case["q_scale"].cpu().double()
    for t, (s, p) in enumerate(zip(case["token_seq"], case["positions"])):
        K, V = (x.to(dtype).double() for x in case["dense"][s])
        lo = max(0, p - window + 1) if window else 0
        for h in range(H):
            g = h // (H // G)
            sc = (K[lo:p + 1, g] @ q[t, h * dk:(h + 1) * dk]) * case["scale"] * (qs[p] if use_qscale else 1.0)
            if use_bias:
                sc = sc + db[h][p - torch.arange(lo, p + 1)]
            out[t, h * dv:(h + 1) * dv] = out_scale * (torch.softmax(sc, 0) @ V[lo:p + 1, g])
    return out


def _run(ops, case, impl, window=None, use_bias=True, use_qscale=True, out_scale=1.0):
    H, dv = case["H"], case["dv"]
    wide = torch.zeros(case["q"].shape[0], H * dv + 8, device=DEV, dtype=case["dtype"])
    out = wide[:, 8:] if case["dtype"] == torch.float32 else wide[:, :H * dv]
    ops.biased_attention(case["q"], case["k_pages"], case["v_pages"], case["bt"], case["ctx"], out, num_heads=H,
                         num_kv_heads=case["G"], scale=case["scale"], dist_bias=case["dist_bias"] if use_bias else None,
                         q_scale=case["q_scale"] if use_qscale else None, out_scale=out_scale, window=window, impl=impl)
    ops.check_device_errors()
    return out.double().cpu()


SHAPES = [(4, 2, 16, 24, 8), (3, 3, 32, 32, 16), (6, 1, 96, 40, 4), (2, 2, 8, 1, 16), (8, 2, 64, 256, 32), (1, 1, 256, 8, 16),
          (4, 2, 12, 20, 8), (2, 1, 50, 7, 16)]          # the last two: key sizes that are no multiple of 8


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dk,dv,page", SHAPES)
@pytest.mark.parametrize("impl", ["simt", "tiled"])
def test_distance_bias_attention_mixed_batch(ops, dtype, impl, H, G, dk, dv, page):
    # prompt portions that start in the middle of a page, a whole prompt, single tokens, a portion of two
    seqs = [(150, 97), (31, 31), (200, 1), (67, 2), (1, 1), (130, 65)]
    case = _case(dtype, seqs, H, G, dk, dv, page, seed=H * 100 + dk)
    for kw in (dict(), dict(use_bias=False), dict(use_qscale=False, out_scale=0.7), dict(window=37)):
        got, want = _run(ops, case, impl, **kw), _want(case, **kw)
        assert (got - want).abs().max() < _tol(dtype) * 2 * max(1.0, want.abs().max().item()), (impl, kw)


@pytest.mark.parametrize("H,G,dk,dv,page", [(3, 3, 32, 32, 16), (4, 2, 64, 128, 16), (2, 1, 128, 16, 8), (6, 2, 96, 48, 4),
                                            (2, 2, 16, 16, 32)])
def test_distance_bias_attention_on_tensor_cores(ops, H, G, dk, dv, page):
    # the same mixed batch through the mma.sync kernel (bfloat16 only): against the oracle and against the tiled kernel
    seqs = [(150, 97), (31, 31), (200, 1), (67, 2), (1, 1), (130, 65), (260, 129)]
    case = _case(torch.bfloat16, seqs, H, G, dk, dv, page, seed=H * 100 + dk + 1)
    for kw in (dict(), dict(use_bias=False), dict(use_qscale=False, out_scale=0.7), dict(window=37), dict(window=64)):
        got, want = _run(ops, case, "mma", **kw), _want(case, **kw)
        assert (got - want).abs().max() < _tol(torch.bfloat16) * 2 * max(1.0, want.abs().max().item()), kw
    assert ops.attention_launches.get("bias_mma", 0) >= 5
    # left to itself the wrapper takes this kernel for bfloat16 prompt portions of such sizes
    before = ops.attention_launches.get("bias_mma", 0)
    _run(ops, case, None)
    assert ops.attention_launches["bias_mma"] == before + 1


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dk,dv,page", SHAPES)
def test_distance_bias_attention_single_tokens(ops, dtype, H, G, dk, dv, page):
    # contexts on both sides of a split of keys (256) and of a page
    seqs = [(c, 1) for c in (1, 2, 255, 256, 257, 300, 512, 513, 700, 33)]
    case = _case(dtype, seqs, H, G, dk, dv, page, seed=H * 10 + dv)
    for kw in (dict(), dict(window=100), dict(use_bias=False, use_qscale=False, out_scale=1.3)):
        want = _want(case, **kw)
        for impl in ("split", "simt"):
            got = _run(ops, case, impl, **kw)
            assert (got - want).abs().max() < _tol(dtype) * 2 * max(1.0, want.abs().max().item()), (impl, kw)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("impl", ["simt", "tiled", "split", "mma"])
def test_distance_bias_attention_finds_one_far_key_among_hundreds(ops, impl, dtype):
    if impl == "mma" and dtype != torch.bfloat16:
        pytest.skip("the tensor-core kernel is bfloat16 only")
    # the sharp key lies 600 and more positions back, in the first page; the bias takes about 3 off its score of
    # 45+, so it still carries the whole weight; its value row is 2.0 everywhere
    ql = 1 if impl == "split" else 40
    seqs = [(640, ql), (701, ql)]
    case = _case(dtype, seqs, 4, 2, 32, 32 if impl == "mma" else 24, 16, seed=5, sharp={0: [3], 1: [16]}, r=(0.3, 0.1))
    got, want = _run(ops, case, impl), _want(case)
    assert (got - want).abs().max() < _tol(dtype) * 2 * max(1.0, want.abs().max().item())
    assert (got - 2.0).abs().max() < 0.05          # nothing but the far key counts


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("impl", ["simt", "tiled", "split", "mma"])
@pytest.mark.parametrize("window", [None, 48])
def test_distance_bias_attention_edges_with_sharp_keys(ops, impl, dtype, window):
    if impl == "mma" and dtype != torch.bfloat16:
        pytest.skip("the tensor-core kernel is bfloat16 only")
    # sharp keys at the borders of pages (16), key chunks (32), tiles (64) and splits (256), at the first positions,
    # and (with a window) just inside and just outside the window of the queries near the end
    c = 330
    ql = 1 if impl == "split" else 70
    where = [0, 1, 15, 16, 31, 32, 63, 64, 255, 256, 257, c - 49, c - 48, c - 47, c - 2]
    case = _case(dtype, [(c, ql), (c - 1, ql)], 2, 1, 16, 16, 16, seed=6, sharp={0: where, 1: where[:-1]}, r=(0.2, 0.05))
    got, want = _run(ops, case, impl, window=window), _want(case, window=window)
    assert (got - want).abs().max() < _tol(dtype) * 2 * max(1.0, want.abs().max().item())


def test_distance_bias_attention_result_does_not_depend_on_the_batch(ops):
    # a token's sums run in an order that depends on its position only: alone or beside others, bit for bit
    H, G, dk, dv, page = 4, 2, 32, 48, 8
    from mini_llm_b200.engine.context import attention_tiles
    both = _case(torch.float32, [(90, 40), (200, 70)], H, G, dk, dv, page, seed=11)
    got = _run(ops, both, "tiled")
    alone = dict(both)                                   # the first request of the two, same pages and table
    alone["q"] = both["q"][:40].contiguous()
    alone["token_seq"], alone["positions"] = both["token_seq"][:40], both["positions"][:40]
    ctx = _Ctx()
    ctx.token_seq, ctx.positions = both["ctx"].token_seq[:40].contiguous(), both["ctx"].positions[:40].contiguous()
    ctx.ws, ctx.max_ctx_len, ctx.decode_only = both["ctx"].ws, 200, False
    tiles = attention_tiles([40], [50])
    ctx.attn_tiles, ctx.n_tiles = torch.tensor(tiles, dtype=torch.int32, device=DEV), len(tiles) // 3
    alone["ctx"] = ctx
    assert torch.equal(_run(ops, alone, "tiled"), got[:40])


def test_decode_attention_in_a_large_batch_equals_the_small_batch_bit_for_bit(ops):
    # 80 single tokens make a grid in which the split kernel stages small tiles; 5 of them alone make one in which it
    # stages a whole split at once: the chunks a warp walks and their order are the same, so are the bits
    H, G, dk, dv, page = 8, 2, 32, 48, 16
    seqs = [(600 - 7 * i, 1) for i in range(80)]
    big = _case(torch.float32, seqs, H, G, dk, dv, page, seed=21)
    got = _run(ops, big, "split")
    want = _want(big)
    assert (got - want).abs().max() < _tol(torch.float32) * 2 * max(1.0, want.abs().max().item())
    small = dict(big)
    small["q"] = big["q"][:5].contiguous()
    small["token_seq"], small["positions"] = big["token_seq"][:5], big["positions"][:5]
    ctx = _Ctx()
    ctx.token_seq, ctx.positions = big["ctx"].token_seq[:5].contiguous(), big["ctx"].positions[:5].contiguous()
    ctx.ws, ctx.max_ctx_len, ctx.decode_only, ctx.n_tiles, ctx.attn_tiles = big["ctx"].ws, 600, True, 0, None
    small["ctx"] = ctx
    assert torch.equal(_run(ops, small, "split"), got[:5])


def test_distance_bias_attention_refuses_sizes_it_cannot_take(ops):
    case = _case(torch.float32, [(20, 5)], 2, 1, 16, 16, 8, seed=1)
    with pytest.raises(ops.KernelError):      # key rows of the pages that are no multiple of 8
        ops.biased_attention(torch.zeros(5, 2 * 12, device=DEV), case["k_pages"][..., :12].contiguous(), case["v_pages"],
                             case["bt"], case["ctx"], torch.zeros(5, 32, device=DEV), num_heads=2, num_kv_heads=1, scale=1.0)
    with pytest.raises(ops.KernelError):      # queries longer than the key rows
        ops.biased_attention(torch.zeros(5, 2 * 24, device=DEV), case["k_pages"], case["v_pages"], case["bt"], case["ctx"],
                             torch.zeros(5, 32, device=DEV), num_heads=2, num_kv_heads=1, scale=1.0)
    with pytest.raises(ops.KernelError):      # a context beyond the bias table
        ops.biased_attention(case["q"], case["k_pages"], case["v_pages"], case["bt"], case["ctx"],
                             torch.zeros(5, 32, device=DEV), num_heads=2, num_kv_heads=1, scale=1.0,
                             dist_bias=case["dist_bias"][:, :10].contiguous())


# ------------------------------------------------------------------------------------------------ recurrence
_WS = {}


def _rec_ctx(q_lens, slots):
    ctx = _Ctx()
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    ctx.cu_q = torch.tensor(cu, dtype=torch.int32, device=DEV)
    ctx.state_slots = torch.tensor(slots, dtype=torch.int32, device=DEV)
    ctx.S = len(q_lens)
    from mini_llm_b200.engine.context import Workspace
    ctx.ws = _WS.setdefault("ws", Workspace(torch.device(DEV), 64))
    return ctx


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Hr,ek,ev", [(2, 16, 40), (3, 8, 16), (1, 64, 64), (2, 96, 33), (1, 130, 96), (4, 32, 1), (1, 1, 32),
                                      (2, 128, 130), (1, 6, 200)])
@pytest.mark.parametrize("impl", [None, "step", "wide"])
def test_gated_recurrence_in_portions_and_batches(ops, dtype, impl, Hr, ek, ev):
    if impl == "wide" and ek > ops.REC_WIDE_MAX_ROWS:
        pytest.skip("the kernel for prompt portions takes up to 128 rows")
    eps, out_scale = 1e-5, 0.9
    lens = [45, 3, 20]
    g = torch.Generator().manual_seed(Hr * 7 + ek)
    f_bias = torch.randn(Hr * ek, generator=g).to(DEV)
    lower = (torch.rand(Hr * ek, generator=g) * 0.99).to(DEV)          # some channels keep their rows for long
    norm_w = (torch.rand(ev, generator=g) + 0.5).to(DEV)
    data, want = [], []
    for n in lens:
        a = torch.randn(n, Hr * ek, generator=g).to(dtype)
        z = (torch.randn(n, Hr * ek, generator=g) * 2).to(dtype)
        v = torch.randn(n, Hr * ev, generator=g).to(dtype)
        data.append((a, z, v))
        q = torch.nn.functional.silu(a.double()).view(n, Hr, ek)
        f = P.forget_gate(z.double(), f_bias.double().cpu(), lower.double().cpu()).view(n, Hr, ek)
        o, _ = P.gated_recurrence(q, f, v.double().view(n, Hr, ev))
        want.append(out_scale * P.rms_norm(o, norm_w.double().cpu(), eps, False).reshape(n, Hr * ev))
    state = torch.zeros(5, Hr, ek, ev, device=DEV)
    state[3] = 7.0                                                      # a slot nobody uses stays as it is
    # the three requests in unequal portions, batched together, in slots 4, 0, 2; the last portions are single tokens
    cuts = {0: [17, 2, 25, 1], 1: [2, 1], 2: [1, 16, 1, 1, 1]}
    slots = {0: 4, 1: 0, 2: 2}
    pos = {s: 0 for s in cuts}
    got = {s: [] for s in cuts}
    while any(cuts.values()):
        live = [s for s in cuts if cuts[s]]
        ns = [cuts[s].pop(0) for s in live]
        parts = [tuple(x[pos[s]:pos[s] + n] for x in data[s]) for s, n in zip(live, ns)]
        wide = torch.cat([torch.cat(p, 1) for p in parts], 0).to(DEV)   # a | z | v as columns of one buffer
        T = wide.shape[0]
        a, z, v = wide[:, :Hr * ek], wide[:, Hr * ek:2 * Hr * ek], wide[:, 2 * Hr * ek:]
        out = torch.empty(T, Hr * ev, device=DEV, dtype=dtype)
        ops.gated_recurrence(a, z, v, f_bias, lower, norm_w, eps, state, _rec_ctx(ns, [slots[s] for s in live]), out,
                             heads=Hr, out_scale=out_scale, impl=impl)
        k = 0
        for s, n in zip(live, ns):
            got[s].append(out[k:k + n].double().cpu())
            k += n
            pos[s] += n
    ops.check_device_errors()
    tol = 3e-5 if dtype == torch.float32 else 1.2e-2
    for s in cuts:
        assert (torch.cat(got[s]) - want[s]).abs().max() < tol * max(1.0, want[s].abs().max().item()), s
    assert torch.all(state[3] == 7.0) and torch.all(state[1] == 0.0)


def test_gated_recurrence_kernels_leave_the_same_state(ops):
    Hr, ek, ev, n = 2, 24, 72, 70
    a, z, v = rnd(n, Hr * ek, seed=1), rnd(n, Hr * ek, seed=2, scale=2.0), rnd(n, Hr * ev, seed=3)
    fb, lo, nw = rnd(Hr * ek, seed=4), torch.rand(Hr * ek, device=DEV), torch.rand(ev, device=DEV) + 0.5
    states, outs = [], []
    for impl in ("step", "wide"):
        state = torch.zeros(1, Hr, ek, ev, device=DEV)
        out = torch.empty(n, Hr * ev, device=DEV)
        ops.gated_recurrence(a, z, v, fb, lo, nw, 1e-5, state, _rec_ctx([n], [0]), out, heads=Hr, impl=impl)
        states.append(state)
        outs.append(out)
    assert torch.equal(states[0], states[1])
    assert (outs[0] - outs[1]).abs().max() < 1e-5


def test_gated_recurrence_reads_without_writing(ops):
    Hr, ek, ev = 2, 16, 24
    a, z, v = rnd(6, Hr * ek, seed=1), rnd(6, Hr * ek, seed=2), rnd(6, Hr * ev, seed=3)
    fb, lo, nw = rnd(Hr * ek, seed=4), torch.rand(Hr * ek, device=DEV) * 0.5, torch.ones(ev, device=DEV)
    state = rnd(2, Hr, ek, ev, seed=5)
    before = state.clone()
    out = torch.empty(6, Hr * ev, device=DEV)
    ops.gated_recurrence(a, z, v, fb, lo, nw, 1e-5, state, _rec_ctx([6], [1]), out, heads=Hr, write_state=False)
    assert torch.equal(state, before)
    ops.gated_recurrence(a, z, v, fb, lo, nw, 1e-5, state, _rec_ctx([6], [1]), out, heads=Hr)
    assert torch.equal(state[0], before[0]) and not torch.equal(state[1], before[1])


def test_gated_recurrence_keeps_a_row_written_long_ago(ops):
    # channel 0 never forgets (lower bound 1) and channel 1 forgets at once (gate 0): after 300 tokens the output of a
    # query on channel 0 is still zero (nothing was ever written through a closed gate), and a query on channel 1
    # returns exactly the last value; the state is what the recurrence says, not an approximation of it
    Hr, ek, ev, n = 1, 2, 8, 300
    lower = torch.tensor([1.0, 0.0], device=DEV)
    f_bias = torch.tensor([0.0, -1e4], device=DEV)
    a = torch.zeros(n, 2, device=DEV)
    a[:, 1] = 20.0                                       # silu(20) = 20 to 1e-8
    z = torch.zeros(n, 2, device=DEV)
    v = rnd(n, ev, seed=3)
    state = torch.zeros(1, 1, 2, ev, device=DEV)
    state[0, 0, 0] = 5.0                                 # something that was there before
    out = torch.empty(n, ev, device=DEV)
    ops.gated_recurrence(a, z, v, f_bias, lower, torch.ones(ev, device=DEV), 0.0, state, _rec_ctx([n], [0]), out, heads=1)
    assert torch.all(state[0, 0, 0] == 5.0)
    assert torch.allclose(state[0, 0, 1], v[-1])
    want = v / v.pow(2).mean(-1, keepdim=True).sqrt()
    assert (out - want).abs().max() < 1e-5
