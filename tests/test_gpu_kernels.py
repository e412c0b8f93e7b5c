"""Each CUDA kernel alone against a plain float32/float64 restatement, at sizes other than
the engine's (tails, sizes that are no power of two, length 1, several head sizes)."""
import math

import numpy as np
import pytest
import torch

import plain_llama as pl

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _rand(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed_rmsnorm_swiglu_gather(dtype):
    from oracle_engine_b200.csrc import ops
    V, D, n = 77, 200, 9
    table = _rand(V, D, dtype=dtype)
    ids = torch.tensor([0, 76, 5, 5, 33, 1, 2, 3, 70], dtype=torch.int32, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    x = torch.empty(n, D, device=DEV)
    ops.embed_gather(x, table, ids, err)
    assert torch.equal(x, table.float()[ids.long()]) and err.item() == 0
    bad = torch.tensor([3, 77, -1], dtype=torch.int32, device=DEV)
    xb = torch.empty(3, D, device=DEV)
    ops.embed_gather(xb, table, bad, err)
    assert err.item() == 1 and torch.equal(xb[1], torch.zeros(D, device=DEV)) and torch.equal(xb[0], table.float()[3])

    # few rows: a block per row; from 1,024 rows of up to 4,096 columns (a prompt step) bfloat16 takes a warp per row
    for rows, D2, eps in ((5, 200, 1e-5), (5, 3, 1e-6), (5, 1031, 1e-2), (1024, 200, 1e-5), (1031, 3076, 1e-6),
                          (1100, 4096, 1e-5), (1025, 2052, 1e-5), (1024, 4100, 1e-5), (1030, 1031, 1e-5)):
        xr = _rand(rows, D2, scale=3.0, seed=1)
        w = _rand(D2, seed=2)
        y = torch.empty(rows, D2, dtype=dtype, device=DEV)
        ops.rmsnorm(y, xr, w, eps)
        want = pl.rms_norm(xr.double().cpu(), w.double().cpu(), eps)
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        assert (y.double().cpu() - want).abs().max() < tol * max(1.0, want.abs().max())

    for FF in (160, 7, 515):
        gu = _rand(6, 2 * FF, dtype=dtype, scale=2.0, seed=3)
        out = torch.empty(6, FF, dtype=dtype, device=DEV)
        ops.swiglu(out, gu)
        g, u = gu.double().cpu()[:, :FF], gu.double().cpu()[:, FF:]
        want = g / (1 + torch.exp(-g)) * u
        tol = 1e-6 if dtype == torch.float32 else 1e-2
        assert (out.double().cpu() - want).abs().max() < tol * max(1.0, want.abs().max())

    rows = torch.tensor([4, 0, 4], dtype=torch.int32, device=DEV)
    src = _rand(5, 33, seed=4)
    dst = torch.empty(3, 33, device=DEV)
    ops.gather_rows_f32(dst, src, rows)
    assert torch.equal(dst, src[rows.long()])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,N,K", [(1, 5, 3), (7, 65, 130), (130, 64, 17), (64, 200, 256)])
def test_gemm_simple(dtype, M, N, K):
    from oracle_engine_b200.csrc import ops
    a, w = _rand(M, K, dtype=dtype, seed=1), _rand(N, K, dtype=dtype, seed=2)
    want = a.double() @ w.double().T
    tol = 1e-5 * math.sqrt(K)
    out = torch.empty(M, N, dtype=dtype, device=DEV)
    ops.gemm_simple(out, a, w)
    assert (out.double() - want).abs().max() < (tol if dtype == torch.float32 else 0.01 * want.abs().max() + tol)
    out32 = torch.empty(M, N, device=DEV)
    ops.gemm_simple(out32, a, w)
    assert (out32.double() - want).abs().max() < tol
    base = _rand(M, N, seed=3)
    acc = base.clone()
    ops.gemm_simple(acc, a, w, accumulate=True)
    assert (acc.double() - (base.double() + want)).abs().max() < tol
    # a row's result does not depend on the other rows (bit for bit)
    one = torch.empty(1, N, device=DEV)
    ops.gemm_simple(one, a[M - 1:M], w)
    assert torch.equal(one[0], out32[M - 1])
    # a view with a row stride
    wide = _rand(M, K + 8, dtype=dtype, seed=5)
    outv = torch.empty(M, N, device=DEV)
    ops.gemm_simple(outv, wide[:, :K], w)
    assert (outv.double() - wide[:, :K].double() @ w.double().T).abs().max() < tol


@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (8, 3072, 1024), (5, 136, 72), (16, 50, 8), (9, 333, 4096), (3, 16, 520)])
def test_gemm_skinny(M, N, K):
    from oracle_engine_b200.csrc import ops_tc
    a, w = _rand(M, K, dtype=torch.bfloat16, scale=0.5, seed=1), _rand(N, K, dtype=torch.bfloat16, scale=0.5, seed=2)
    want = a.double() @ w.double().T
    tol = 2e-6 * K + 1e-5
    out32 = torch.full((M, N), 9.0, device=DEV)
    ops_tc.gemm(out32, a, w, kernel="skinny")
    assert (out32.double() - want).abs().max() < tol
    out16 = torch.full((M, N), 9.0, dtype=torch.bfloat16, device=DEV)
    ops_tc.gemm(out16, a, w, kernel="skinny")
    assert (out16.double() - want).abs().max() < 0.005 * want.abs().max() + tol
    base = _rand(M, N, seed=3)
    acc = base.clone()
    ops_tc.gemm(acc, a, w, accumulate=True, kernel="skinny")
    assert (acc.double() - (base.double() + want)).abs().max() < tol
    if N % 2 == 0:
        act = torch.full((M, N // 2), 9.0, dtype=torch.bfloat16, device=DEV)
        ops_tc.gemm(act, a, w, swiglu=True, kernel="skinny")
        gate, up = want[:, 0::2], want[:, 1::2]
        ref = gate / (1 + torch.exp(-gate)) * up
        assert (act.double() - ref).abs().max() < 0.005 * ref.abs().max() + 10 * tol
    # a token's result does not depend on the other tokens of the step (bit for bit)
    one = torch.empty(1, N, device=DEV)
    ops_tc.gemm(one, a[M - 1:M], w, kernel="skinny")
    assert torch.equal(one[0], out32[M - 1])


@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (8, 3072, 1024), (5, 136, 72), (64, 520, 4096), (100, 333, 200),
                                   (128, 48, 64), (129, 48, 200), (300, 1000, 520), (1000, 264, 72)])
def test_gemm_tcgen05(M, N, K):
    from oracle_engine_b200.csrc import ops_tc
    import functools
    ops_tc = type("tc", (), {"gemm": staticmethod(functools.partial(ops_tc.gemm, kernel="tcgen05")),
                             "device_error": staticmethod(ops_tc.device_error),
                             "gemm_supported": staticmethod(ops_tc.gemm_supported)})
    a, w = _rand(M, K, dtype=torch.bfloat16, scale=0.5, seed=1), _rand(N, K, dtype=torch.bfloat16, scale=0.5, seed=2)
    want = a.double() @ w.double().T
    tol = 2e-6 * K + 1e-5
    out32 = torch.full((M, N), 9.0, device=DEV)
    ops_tc.gemm(out32, a, w)
    assert (out32.double() - want).abs().max() < tol
    out16 = torch.full((M, N), 9.0, dtype=torch.bfloat16, device=DEV)
    ops_tc.gemm(out16, a, w)
    assert (out16.double() - want).abs().max() < 0.005 * want.abs().max() + tol
    base = _rand(M, N, seed=3)
    acc = base.clone()
    ops_tc.gemm(acc, a, w, accumulate=True)
    assert (acc.double() - (base.double() + want)).abs().max() < tol
    nosplit = torch.empty(M, N, device=DEV)
    ops_tc.gemm(nosplit, a, w, split_k=False)
    assert (nosplit.double() - want).abs().max() < tol
    again = torch.empty(M, N, device=DEV)
    ops_tc.gemm(again, a, w)
    assert torch.equal(again, out32)                     # split sums are added in a fixed order
    if N % 2 == 0:
        # fused activation: weight rows alternate gate, up
        act = torch.full((M, N // 2), 9.0, dtype=torch.bfloat16, device=DEV)
        ops_tc.gemm(act, a, w, swiglu=True)
        gate, up = want[:, 0::2], want[:, 1::2]
        ref = gate / (1 + torch.exp(-gate)) * up
        assert (act.double() - ref).abs().max() < 0.005 * ref.abs().max() + 10 * tol
    assert ops_tc.device_error() == 0
    assert not ops_tc.gemm_supported(a[:, :K - 1], w[:, :K - 1].contiguous(), out32)      # rows not 16-byte aligned


@pytest.mark.parametrize("M,N,K,max_tile", [(300, 1000, 520, 128), (256, 256, 64, 128), (1000, 264, 72, 0), (513, 3072, 1024, 0),
                                            (2048, 640, 200, 0), (129, 40, 8, 0), (600, 3000, 320, -176),
                                            (300, 520, 136, -240), (512, 300, 64, -144), (2048, 3072, 256, 0)])
def test_gemm_pair(M, N, K, max_tile):
    """The two-SM kernel: row and column edges, both halves of the weight tile, all epilogues; tile widths
    that are odd multiples of 16 (max_tile < 0 forces a width), whose last group of columns is half."""
    from oracle_engine_b200.csrc import ops_tc
    with ops_tc.knobs(pair_max_tile=max_tile):
        a, w = _rand(M, K, dtype=torch.bfloat16, scale=0.5, seed=1), _rand(N, K, dtype=torch.bfloat16, scale=0.5, seed=2)
        want = a.double() @ w.double().T
        tol = 2e-6 * K + 1e-5
        out32 = torch.full((M, N), 9.0, device=DEV)
        ops_tc.gemm(out32, a, w, kernel="pair")
        assert (out32.double() - want).abs().max() < tol
        out16 = torch.full((M, N), 9.0, dtype=torch.bfloat16, device=DEV)
        ops_tc.gemm(out16, a, w, kernel="pair")
        assert (out16.double() - want).abs().max() < 0.005 * want.abs().max() + tol
        base = _rand(M, N, seed=3)
        acc = base.clone()
        ops_tc.gemm(acc, a, w, accumulate=True, kernel="pair")
        assert (acc.double() - (base.double() + want)).abs().max() < tol
        again = torch.empty(M, N, device=DEV)
        ops_tc.gemm(again, a, w, kernel="pair")
        assert torch.equal(again, out32)
        if N % 2 == 0:
            act = torch.full((M, N // 2), 9.0, dtype=torch.bfloat16, device=DEV)
            ops_tc.gemm(act, a, w, swiglu=True, kernel="pair")
            gate, up = want[:, 0::2], want[:, 1::2]
            ref = gate / (1 + torch.exp(-gate)) * up
            assert (act.double() - ref).abs().max() < 0.005 * ref.abs().max() + 10 * tol
        # the one-SM kernel computes the same sums in the same order
        one = torch.empty(M, N, device=DEV)
        ops_tc.gemm(one, a, w, kernel="tcgen05", split_k=False)
        assert torch.equal(one, out32)
        assert ops_tc.device_error() == 0


@pytest.mark.parametrize("M,N,K", [(300, 512, 1664), (2048, 3072, 512), (1100, 5000, 328)])
def test_gemm_stream_k(M, N, K):
    """The stream-K schedule, forced: tiles cut into many pieces (more than the four that are
    added up at a time), whole tiles after the shared ones, row, column and K edges; all
    epilogues; the same bits every time and whichever CTA adds up."""
    from oracle_engine_b200.csrc import ops_tc
    with ops_tc.knobs(gemm_schedule=(0, 1, -1, -1)):
        a, w = _rand(M, K, dtype=torch.bfloat16, scale=0.5, seed=1), _rand(N, K, dtype=torch.bfloat16, scale=0.5, seed=2)
        want = a.double() @ w.double().T
        tol = 2e-6 * K + 1e-5
        out32 = torch.full((M, N), 9.0, device=DEV)
        ops_tc.gemm(out32, a, w, kernel="tcgen05")
        assert (out32.double() - want).abs().max() < tol
        for _ in range(3):
            again = torch.empty(M, N, device=DEV)
            ops_tc.gemm(again, a, w, kernel="tcgen05")
            assert torch.equal(again, out32)
        out16 = torch.full((M, N), 9.0, dtype=torch.bfloat16, device=DEV)
        ops_tc.gemm(out16, a, w, kernel="tcgen05")
        assert (out16.double() - want).abs().max() < 0.005 * want.abs().max() + tol
        base = _rand(M, N, seed=3)
        acc = base.clone()
        ops_tc.gemm(acc, a, w, accumulate=True, kernel="tcgen05")
        assert (acc.double() - (base.double() + want)).abs().max() < tol
        act = torch.full((M, N // 2), 9.0, dtype=torch.bfloat16, device=DEV)
        ops_tc.gemm(act, a, w, swiglu=True, kernel="tcgen05")
        gate, up = want[:, 0::2], want[:, 1::2]
        ref = gate / (1 + torch.exp(-gate)) * up
        assert (act.double() - ref).abs().max() < 0.005 * ref.abs().max() + 10 * tol
        # whole tiles give the same sums up to the order of the pieces
        with ops_tc.knobs(gemm_schedule=(0, 0, -1, -1)):
            whole = torch.empty(M, N, device=DEV)
            ops_tc.gemm(whole, a, w, kernel="tcgen05")
        assert (whole.double() - out32.double()).abs().max() < tol
        assert ops_tc.device_error() == 0


@pytest.mark.parametrize("M,N,K", [(64, 3072, 3072), (17, 640, 1024), (100, 520, 4096), (128, 264, 8192), (33, 1000, 328)])
@pytest.mark.parametrize("cluster", [-1, 0])
def test_gemm_few_tokens_split_k(M, N, K, cluster):
    """Up to 128 tokens, swap-AB with K split: the splits of a tile add up inside a cluster
    (2 to 8 CTAs, shares of rows that are not equal, a last weight tile that is partly empty)
    or through the workspace; all epilogues; the same bits every time."""
    from oracle_engine_b200.csrc import ops_tc
    with ops_tc.knobs(gemm_schedule=(0, -1, cluster, 0)):
        a, w = _rand(M, K, dtype=torch.bfloat16, scale=0.5, seed=1), _rand(N, K, dtype=torch.bfloat16, scale=0.5, seed=2)
        want = a.double() @ w.double().T
        tol = 2e-6 * K + 1e-5
        out32 = torch.full((M, N), 9.0, device=DEV)
        ops_tc.gemm(out32, a, w, kernel="tcgen05")
        assert (out32.double() - want).abs().max() < tol
        for _ in range(3):
            again = torch.empty(M, N, device=DEV)
            ops_tc.gemm(again, a, w, kernel="tcgen05")
            assert torch.equal(again, out32)
        out16 = torch.full((M, N), 9.0, dtype=torch.bfloat16, device=DEV)
        ops_tc.gemm(out16, a, w, kernel="tcgen05")
        assert (out16.double() - want).abs().max() < 0.005 * want.abs().max() + tol
        base = _rand(M, N, seed=3)
        acc = base.clone()
        ops_tc.gemm(acc, a, w, accumulate=True, kernel="tcgen05")
        assert (acc.double() - (base.double() + want)).abs().max() < tol
        act = torch.full((M, N // 2), 9.0, dtype=torch.bfloat16, device=DEV)
        ops_tc.gemm(act, a, w, swiglu=True, kernel="tcgen05")
        gate, up = want[:, 0::2], want[:, 1::2]
        ref = gate / (1 + torch.exp(-gate)) * up
        assert (act.double() - ref).abs().max() < 0.005 * ref.abs().max() + 10 * tol
        assert ops_tc.device_error() == 0


def _paged(k, v, lens, dtype, extra_pages=3, seed=0):
    """Dense per-sequence K/V [len, KVH, hd] -> one cache entry [pages, 2, KVH, 64, hd] with
    shuffled pages, and the page tables."""
    KVH, hd = k[0].shape[1], k[0].shape[2]
    need = [(n + 63) // 64 for n in lens]
    total = sum(need) + extra_pages
    rng = np.random.RandomState(seed)
    order = rng.permutation(total).tolist()
    cache = torch.full((total, 2, KVH, 64, hd), 1e4, dtype=dtype)      # stale values must never be read
    tables = np.full((len(lens), max(need) + 1), -1, dtype=np.int32)
    for b, n in enumerate(lens):
        for p in range(need[b]):
            page = order.pop()
            tables[b, p] = page
            rows = slice(p * 64, min(n, p * 64 + 64))
            cnt = rows.stop - rows.start
            cache[page, 0, :, :cnt] = k[b][rows].transpose(0, 1).to(dtype)
            cache[page, 1, :, :cnt] = v[b][rows].transpose(0, 1).to(dtype)
    return cache.to(DEV), torch.from_numpy(tables).to(DEV)


def _attn_case(H, KVH, hd, lens, qlens, dtype, seed):
    """Queries for the last qlen tokens of each sequence; returns tensors and the plain result."""
    g = torch.Generator().manual_seed(seed)
    k = [torch.randn(n, KVH, hd, generator=g) for n in lens]
    v = [torch.randn(n, KVH, hd, generator=g) for n in lens]
    q = [torch.randn(n, H, hd, generator=g) * 2.0 for n in lens]
    rd = (lambda t: t.to(dtype).double())
    want = []
    return k, v, q, rd


@pytest.mark.parametrize("dtype,kernel", [(torch.float32, "paged"), (torch.bfloat16, "paged"),
                                          (torch.bfloat16, "mma"), (torch.bfloat16, "tcgen05")])
@pytest.mark.parametrize("H,KVH,hd,window", [(4, 2, 16, 0), (6, 2, 32, 0), (5, 1, 48, 0), (8, 8, 64, 0),
                                             (24, 8, 128, 0), (6, 3, 32, 70), (4, 4, 16, 5), (10, 2, 64, 70),
                                             (3, 1, 128, 129)])
def test_attention_kernels(pin, dtype, kernel, H, KVH, hd, window):
    """Ragged prompts and decoded tokens over a shuffled paged cache with stale pages."""
    from types import SimpleNamespace
    from oracle_engine_b200.csrc import ops, ops_tc
    if kernel == "tcgen05" and hd not in ops_tc.TCGEN05_ATTENTION_HEAD_DIMS:
        pytest.skip("the tcgen05 prompt kernel is built for head_dim 64 and 128")
    pin(prompt_kernel="tcgen05" if kernel == "tcgen05" else "mma")
    lens = [1, 64, 65, 200, 130, 17]
    g = torch.Generator().manual_seed(H * 100 + hd)
    k = [torch.randn(n, KVH, hd, generator=g) for n in lens]
    v = [torch.randn(n, KVH, hd, generator=g) for n in lens]
    q = [torch.randn(n, H, hd, generator=g) * 1.5 for n in lens]
    cache, tables = _paged(k, v, lens, dtype)
    rd = lambda t: t.to(dtype).double()                                  # noqa: E731
    full = [pl.causal_attention(rd(q[b]), rd(k[b]), rd(v[b]), window or None) for b in range(len(lens))]
    tol = 1e-5 if dtype == torch.float32 else 2.5e-2
    for mode, qlens in (("prompt", [1, 64, 30, 200, 67, 17]), ("decode", [1] * len(lens))):
        tok_seq, tok_pos, rows_q, want = [], [], [], []
        cu, starts = [0], []
        for b, (n, ql) in enumerate(zip(lens, qlens)):
            starts.append(n - ql)
            for i in range(n - ql, n):
                tok_seq.append(b)
                tok_pos.append(i)
                rows_q.append(q[b][i].reshape(-1))
                want.append(full[b][i])
            cu.append(len(tok_seq))
        # a padding row and a padding sequence at the end
        tok_seq.append(-1)
        tok_pos.append(0)
        rows_q.append(torch.zeros(H * hd))
        T = len(tok_seq)
        # queries live in a wider buffer (as in the fused qkv projection)
        qbuf = torch.zeros(T, H * hd + 2 * KVH * hd)
        qbuf[:, :H * hd] = torch.stack(rows_q)
        qbuf = qbuf.to(dtype).to(DEV)
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)    # noqa: E731
        out = torch.full((T, H * hd), 7.0, dtype=dtype, device=DEV)
        tab = torch.cat([tables, torch.full((1, tables.shape[1]), -1, dtype=torch.int32, device=DEV)])
        if kernel == "paged":
            ops.attn_paged(out, qbuf, cache, tab, i32(tok_seq), i32(tok_pos), H, KVH, hd, window, 1 / math.sqrt(hd))
        else:
            ctx = SimpleNamespace(cu_q=i32(cu + [cu[-1]]), seq_start=i32(starts + [0]), seq_qlen=i32(qlens + [0]),
                                  tok_seq=i32(tok_seq), n_seqs=len(lens) + 1, max_qlen=max(qlens),
                                  all_decode=(mode == "decode"))
            ops_tc.attention(out, qbuf, cache, tab, ctx, H, KVH, hd, window, 1 / math.sqrt(hd))
        got = out[:T - 1].double().cpu()
        err = (got - torch.stack(want)).abs().max().item()
        assert err < tol, f"{kernel} {mode}: {err}"
    assert ops_tc.device_error() == 0


@pytest.mark.parametrize("kernel", ["mma", "tcgen05"])
@pytest.mark.parametrize("hd,step", [(64, 12.0), (128, 4.0), (128, -6.0)])
def test_attention_moving_maximum(pin, kernel, hd, step):
    """Scores that climb (or fall) by `step` from one block of 64 keys to the next: the running maximum
    moves at every block (12), at every second or third block (4: in between, probabilities above 1
    are summed against an older maximum), or never (falling: the first block outweighs all later ones)."""
    from types import SimpleNamespace
    from oracle_engine_b200.csrc import ops_tc
    pin(prompt_kernel=kernel)
    H, KVH, n = 4, 2, 700
    g = torch.Generator().manual_seed(int(hd + step))
    u = torch.randn(hd, generator=g)
    u = u / u.norm()
    k = torch.randn(n, KVH, hd, generator=g) * 0.5
    q = torch.randn(n, H, hd, generator=g) * 0.5
    v = torch.randn(n, KVH, hd, generator=g)
    # q . k / sqrt(hd) gains `step` per block along u
    q = q + u * math.sqrt(math.sqrt(hd) * 8.0)
    k = k + u * (torch.arange(n) // 64).reshape(n, 1, 1) * (step / 8.0) * math.sqrt(math.sqrt(hd) * 8.0)
    rd = lambda t: t.to(torch.bfloat16).double()                          # noqa: E731
    want = pl.causal_attention(rd(q), rd(k), rd(v), None)
    cache, tables = _paged([k], [v], [n], torch.bfloat16)
    qbuf = torch.zeros(n, (H + 2 * KVH) * hd)
    qbuf[:, :H * hd] = q.reshape(n, -1)
    qbuf = qbuf.to(torch.bfloat16).to(DEV)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)        # noqa: E731
    out = torch.full((n, H * hd), 7.0, dtype=torch.bfloat16, device=DEV)
    ctx = SimpleNamespace(cu_q=i32([0, n]), seq_start=i32([0]), seq_qlen=i32([n]), tok_seq=i32([0] * n), n_seqs=1,
                          max_qlen=n, all_decode=False)
    ops_tc.attention(out, qbuf, cache, tables, ctx, H, KVH, hd, 0, 1 / math.sqrt(hd))
    err = (out.double().cpu() - want.reshape(n, -1)).abs().max().item()
    assert err < 2.5e-2, err
    assert ops_tc.device_error() == 0


@pytest.mark.parametrize("hd,window", [(128, 0), (64, 1000)])
def test_attention_long_prompt(hd, window):
    """A prompt of 36 key blocks through the tensor-memory kernel (every row checked), with and
    without a window that spans many blocks, and the same sequence continued from a cached prefix."""
    from types import SimpleNamespace
    from oracle_engine_b200.csrc import ops_tc
    H, KVH, n = 2, 1, 2300
    g = torch.Generator().manual_seed(hd + window)
    k = torch.randn(n, KVH, hd, generator=g)
    v = torch.randn(n, KVH, hd, generator=g)
    q = torch.randn(n, H, hd, generator=g) * 1.5
    rd = lambda t: t.to(torch.bfloat16).double()                          # noqa: E731
    want = pl.causal_attention(rd(q), rd(k), rd(v), window or None)
    cache, tables = _paged([k], [v], [n], torch.bfloat16)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)        # noqa: E731
    for start in (0, 1111):                                               # whole, and the last tokens over a cached prefix
        m = n - start
        qbuf = torch.zeros(m, (H + 2 * KVH) * hd)
        qbuf[:, :H * hd] = q[start:].reshape(m, -1)
        qbuf = qbuf.to(torch.bfloat16).to(DEV)
        out = torch.full((m, H * hd), 7.0, dtype=torch.bfloat16, device=DEV)
        ctx = SimpleNamespace(cu_q=i32([0, m]), seq_start=i32([start]), seq_qlen=i32([m]), tok_seq=i32([0] * m), n_seqs=1,
                              max_qlen=m, all_decode=False)
        ops_tc.attention(out, qbuf, cache, tables, ctx, H, KVH, hd, window, 1 / math.sqrt(hd))
        err = (out.double().cpu() - want[start:]).abs().max().item()
        assert err < 2.5e-2, (start, err)
    assert ops_tc.device_error() == 0


def test_rope_kv_write():
    from oracle_engine_b200.csrc import ops
    from oracle_engine_b200.parts.positions import rotary_inv_freq
    H, KVH, hd, T = 3, 2, 24, 6
    for dtype in (torch.float32, torch.bfloat16):
        inv = rotary_inv_freq(hd, 10000.0, {"factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                            "original_max_position_embeddings": 16})
        assert torch.allclose(inv, pl.rope_inv_freq(hd, 10000.0, {"rope_type": "llama3", "factor": 4.0,
                              "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                              "original_max_position_embeddings": 16}), rtol=0, atol=0)
        ang = torch.arange(300, dtype=torch.float64)[:, None] * inv[None]
        cos, sin = torch.cos(ang).float().to(DEV), torch.sin(ang).float().to(DEV)
        qkv = _rand(T, (H + 2 * KVH) * hd, dtype=dtype, seed=9)
        orig = qkv.clone()
        cache = torch.zeros(5, 2, KVH, 64, hd, dtype=dtype, device=DEV)
        tables = torch.tensor([[3, 1, -1], [4, -1, -1]], dtype=torch.int32, device=DEV)
        tok_seq = torch.tensor([0, 0, 1, -1, 0, 1], dtype=torch.int32, device=DEV)
        tok_pos = torch.tensor([63, 64, 0, 0, 127, 1], dtype=torch.int32, device=DEV)
        ops.rope_kv_write(qkv, cos, sin, cache, tables, tok_seq, tok_pos, H, KVH, hd, True)
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        for t in range(T):
            if tok_seq[t] < 0:
                assert torch.equal(qkv[t], orig[t])
                continue
            p = torch.tensor([int(tok_pos[t])])
            o = orig[t].double().cpu()
            qw = pl.rope_rotate(o[:H * hd].reshape(1, H, hd), p, inv)
            kw = pl.rope_rotate(o[H * hd:(H + KVH) * hd].reshape(1, KVH, hd), p, inv)
            assert (qkv[t, :H * hd].double().cpu() - qw.reshape(-1)).abs().max() < tol
            page = int(tables[int(tok_seq[t]), int(tok_pos[t]) // 64])
            r = int(tok_pos[t]) % 64
            assert (cache[page, 0, :, r].double().cpu() - kw[0]).abs().max() < tol
            assert torch.equal(cache[page, 1, :, r].cpu(), orig[t, (H + KVH) * hd:].reshape(KVH, hd).cpu())
        assert cache[0].abs().max() == 0 and cache[2].abs().max() == 0          # unmapped pages untouched
        # no rotation (a mixer without position encoding), queries only
        q_only = orig[:, :H * hd].clone()
        ops.rope_kv_write(q_only, None, None, None, tables, tok_seq, tok_pos, H, KVH, hd, False)
        assert torch.equal(q_only, orig[:, :H * hd])


@pytest.mark.parametrize("H,KVH,hd", [(3, 2, 32), (40, 8, 128), (5, 1, 48)])
def test_rope_kv_write_many_tokens(H, KVH, hd):
    """From 512 tokens on the rows are staged in shared memory, 4, 2 or 1 tokens to a block: the same bits as the
    kernel for few tokens (the same step in pieces of under 512 tokens), with a token count that is no multiple
    of 4, padding tokens in between, three sequences at different places, and with and without rotation."""
    from oracle_engine_b200.csrc import ops
    T, B, pages_per_seq = 771, 3, 8
    g = torch.Generator().manual_seed(hd)
    tok_seq = torch.randint(0, B, (T,), generator=g, dtype=torch.int32)
    tok_seq[torch.randperm(T, generator=g)[:40]] = -1                     # padding tokens
    tok_seq[T - 1] = 2
    tok_pos = torch.zeros(T, dtype=torch.int32)
    nxt = [5, 64, 200]
    for t in range(T):
        b = int(tok_seq[t])
        if b >= 0:
            tok_pos[t] = nxt[b]
            nxt[b] += 1
    assert max(nxt) <= pages_per_seq * 64
    tables = torch.randperm(B * pages_per_seq, generator=g).reshape(B, pages_per_seq).to(torch.int32)
    ang = torch.arange(pages_per_seq * 64, dtype=torch.float64)[:, None] * (10000.0 ** (-torch.arange(hd // 2, dtype=torch.float64) / (hd // 2)))[None]
    cos, sin = torch.cos(ang).float().to(DEV), torch.sin(ang).float().to(DEV)
    tok_seq, tok_pos, tables = tok_seq.to(DEV), tok_pos.to(DEV), tables.to(DEV)
    for dtype in (torch.bfloat16, torch.float32):
        for rotate in (True, False):
            orig = _rand(T, (H + 2 * KVH) * hd, dtype=dtype, seed=4)
            outs = []
            for pieces in ((T,), (300, 300, 171)):
                qkv = orig.clone()
                cache = torch.zeros(B * pages_per_seq, 2, KVH, 64, hd, dtype=dtype, device=DEV)
                at = 0
                for n in pieces:
                    ops.rope_kv_write(qkv[at:at + n], cos if rotate else None, sin if rotate else None, cache, tables,
                                      tok_seq[at:at + n], tok_pos[at:at + n], H, KVH, hd, True)
                    at += n
                outs.append((qkv, cache))
            assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1]), (dtype, rotate)
            if rotate:
                assert not torch.equal(outs[0][0][:, :H * hd], orig[:, :H * hd])
                pad = (tok_seq < 0)
                assert torch.equal(outs[0][0][pad], orig[pad])
            else:
                assert torch.equal(outs[0][0], orig)


def test_argmax_and_sampling():
    from oracle_engine_b200.csrc import ops
    V, R = 1003, 6
    g = torch.Generator().manual_seed(5)
    logits = (torch.randn(R, V, generator=g) * 3).to(DEV)
    logits[2, 100] = logits[2, 900] = 50.0                      # a tie: the first maximum wins
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    ops.argmax_rows(logits, out)
    assert out.tolist() == [pl.greedy(logits[r].cpu()) for r in range(R)] and out[2].item() == 100

    wide = (torch.randn(5, 20011, generator=g) * 3).to(DEV)       # the two-stage kernel for wide rows
    wide[1, 7] = wide[1, 20000] = 60.0
    wide[3, 20010] = 70.0
    out5 = torch.empty(5, dtype=torch.int32, device=DEV)
    ops.argmax_rows(wide, out5)
    assert out5.tolist() == wide.argmax(dim=1).tolist() and out5[1].item() == 7 and out5[3].item() == 20010

    n_slots = 8
    seeds = torch.arange(100, 100 + n_slots, dtype=torch.int64, device=DEV)
    row_slot = torch.tensor([5, 0, 7, 2, 3, 1], dtype=torch.int32, device=DEV)
    cases = [dict(temperature=0.8, top_k=0, top_p=1.0, penalty=1.0), dict(temperature=1.0, top_k=40, top_p=0.9, penalty=1.15),
             dict(temperature=0.7, top_k=5, top_p=1.0, penalty=1.0), dict(temperature=1.3, top_k=0, top_p=0.5, penalty=1.0),
             dict(temperature=0.0, top_k=40, top_p=0.9, penalty=1.5)]
    for c in cases:
        counters = torch.zeros(n_slots, dtype=torch.int32, device=DEV)
        hist = torch.zeros(n_slots, 16, dtype=torch.int32, device=DEV)
        hist_count = torch.zeros(n_slots, dtype=torch.int32, device=DEV)
        history = {int(s): [] for s in row_slot.tolist()}
        for s in history:                                           # some recorded tokens, with a repeat
            toks = [(s * 37 + j * 11) % V for j in range(5)] + [int(logits[row_slot.tolist().index(s)].argmax())] * 2
            history[s] = toks
            for j, t in enumerate(toks):
                hist[s, j % 16] = t
            hist_count[s] = len(toks)
        for draw in range(3):
            work = logits.clone()
            ops.sample_rows(work, out, row_slot, c["temperature"], c["top_k"], c["top_p"], c["penalty"], 6, seeds,
                            counters, hist, hist_count, record=True)
            got = out.tolist()
            for r, s in enumerate(row_slot.tolist()):
                u = pl.uniform_from_counter(100 + s, draw)
                want = pl.sample(logits[r].cpu(), c["temperature"], c["top_k"], c["top_p"], u, history[s],
                                 c["penalty"], 6)
                assert got[r] == want, f"{c} draw {draw} row {r}: {got[r]} vs {want}"
                history[s].append(got[r])
        assert counters[5].item() == (3 if c["temperature"] > 0 else 0) and hist_count[5].item() == 10


@pytest.mark.parametrize("kernel", ["fused", "warps", "warps 4x3", "warps 2x3", "warps 1x3", "warps 3x2",
                                    "warps 6x2x2", "warps 6x2x4", "warps 2x3x2", "warps 1x3x8"])
@pytest.mark.parametrize("H,KVH,hd,window,rotate", [(24, 8, 128, 0, True), (6, 2, 32, 0, True), (8, 8, 64, 100, False),
                                                     (4, 1, 32, 0, True), (16, 1, 64, 300, True)])
def test_attention_decode_fused(H, KVH, hd, window, rotate, kernel):
    """One kernel for rotation, cache write, attention and merge (the keys split over CTAs, or over
    the warps of one CTA, in every form of that kernel: warps x tiles in a warp's ring, alone or
    several CTAs of a cluster sharing the keys), against
    the plain parts."""
    import functools
    from types import SimpleNamespace
    from oracle_engine_b200.csrc import ops_tc
    decode = ops_tc.attention_decode_fused if kernel == "fused" else ops_tc.attention_decode_warps
    if " " in kernel:                      # warps x ring [x CTAs of a cluster that share a (sequence, KV head)]
        form = tuple(int(v) for v in kernel.split()[1].split("x"))
        decode = functools.partial(decode, shape=form[:2], cluster=form[2] if len(form) > 2 else 1)
    lens = [1, 64, 65, 200, 130, 17, 128, 33, 600, 2100]       # length including the new token
    B = len(lens)
    g = torch.Generator().manual_seed(hd + H)
    bf = lambda t: t.to(torch.bfloat16)                       # noqa: E731
    inv = pl.rope_inv_freq(hd, 10000.0, None)
    ang = torch.arange(4096, dtype=torch.float64)[:, None] * inv[None]
    cos, sin = torch.cos(ang).float().to(DEV), torch.sin(ang).float().to(DEV)
    k_old = [bf(torch.randn(n - 1, KVH, hd, generator=g)) for n in lens]        # already rotated, in the cache
    v_old = [bf(torch.randn(n - 1, KVH, hd, generator=g)) for n in lens]
    qkv = bf(torch.randn(B, (H + 2 * KVH) * hd, generator=g) * 1.2)
    # cache pages hold the old keys; the page of the new token exists but its row is stale
    pad = lambda t: torch.cat([t, torch.full((1, KVH, hd), 77.0, dtype=t.dtype)])          # noqa: E731
    cache, tables = _paged([pad(k) for k in k_old], [pad(v) for v in v_old], lens, torch.bfloat16, seed=3)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)                           # noqa: E731
    # a padding sequence at the end
    tab = torch.cat([tables, torch.full((1, tables.shape[1]), -1, dtype=torch.int32, device=DEV)])
    ctx = SimpleNamespace(cu_q=i32(list(range(B + 1)) + [B]), seq_start=i32([n - 1 for n in lens] + [0]),
                          seq_qlen=i32([1] * B + [0]), n_seqs=B + 1)
    out = torch.full((B + 1, H * hd), 5.0, dtype=torch.bfloat16, device=DEV)
    qkv_dev = torch.cat([qkv, torch.zeros(1, qkv.shape[1], dtype=torch.bfloat16)]).to(DEV)
    decode(out, qkv_dev, cos if rotate else None, sin if rotate else None, cache, tab, ctx, H, KVH,
           hd, window, 1 / math.sqrt(hd), True)
    for b, n in enumerate(lens):
        q = qkv[b, :H * hd].double().reshape(1, H, hd)
        k = qkv[b, H * hd:(H + KVH) * hd].double().reshape(1, KVH, hd)
        v = qkv[b, (H + KVH) * hd:].double().reshape(1, KVH, hd)
        if rotate:
            p = torch.tensor([n - 1])
            q, k = pl.rope_rotate(q, p, inv), pl.rope_rotate(k, p, inv)
        k_new = bf(k).double()
        k_all = torch.cat([k_old[b].double(), k_new])
        v_all = torch.cat([v_old[b].double(), v])
        qq = torch.zeros(n, H, hd, dtype=torch.float64)
        qq[-1] = bf(q).double()[0]
        want = pl.causal_attention(qq, k_all, v_all, window or None)[-1]
        err = (out[b].double().cpu() - want).abs().max().item()
        assert err < 2.5e-2, f"sequence {b} (len {n}): {err}"
        page = int(tables[b, (n - 1) // 64])
        assert torch.equal(cache[page, 0, :, (n - 1) % 64].cpu(), bf(k_new)[0])            # the new key and value are stored
        assert torch.equal(cache[page, 1, :, (n - 1) % 64].cpu(), bf(v)[0])
    # an entry that reads another entry's cache: queries only, nothing stored
    out2 = torch.full_like(out, 5.0)
    q_only = qkv_dev[:, :H * hd].contiguous()
    decode(out2, q_only, cos if rotate else None, sin if rotate else None, cache, tab, ctx, H, KVH,
           hd, window, 1 / math.sqrt(hd), False)
    assert torch.equal(out2[:B], out[:B])


def test_gemm_wait_that_runs_out_returns_and_reports():
    """A wait inside the tensor-core product that nothing ends: with the epilogues told to withhold
    their accumulators and a limit of 2 ms, the waits for each CTA's third tile run out; the
    kernel must come back by itself, report the wait's code through oe_gemm_tc_error(), leave the
    tensor memory free, and the next ordinary product must be right."""
    import time
    from oracle_engine_b200.csrc import ops_tc
    M, N, K = 300, 2048, 256
    a, w = _rand(M, K, dtype=torch.bfloat16, scale=0.5, seed=1), _rand(N, K, dtype=torch.bfloat16, scale=0.5, seed=2)
    want = a.double() @ w.double().T
    out = torch.zeros(M, N, device=DEV)
    assert ops_tc.device_error() == 0
    with ops_tc.knobs(sm_count=4, gemm_waits=(2_000_000, 1)):          # 24 tiles on 4 CTAs: 6 each
        t0 = time.time()
        ops_tc.gemm(out, a, w, kernel="tcgen05", split_k=False)
        torch.cuda.synchronize()
        took = time.time() - t0
    assert took < 1.0, f"the kernel took {took:.2f} s to give up"
    # the MMA role's wait for an accumulator (4), the epilogue's wait for the next sums (3) or the TMA role's wait
    # for a free stage (1): all three start within microseconds of each other, whichever ran out first
    assert ops_tc.device_error() in (1, 3, 4)
    assert ops_tc.device_error() == 0                                   # reading the flag clears it
    for _ in range(2):                                                  # tensor memory and barriers are as new
        good = torch.zeros(M, N, device=DEV)
        ops_tc.gemm(good, a, w, kernel="tcgen05", split_k=False)
        assert (good.double() - want).abs().max() < 2e-6 * K + 1e-5
    assert ops_tc.device_error() == 0
