"""The attention entry point that allocates nothing (csrc/attention_noalloc.h), called
through its exported C symbol and checked against the ordinary entry point.

It serves callers that cannot call cudaMalloc while a step runs (fixed-memory control
loops, plugins inside someone else's memory pool): the split-key scratch lives in a fixed
array inside the library.  The array is shared by all calls and keeps the last call's
contents, so the check is made on two different calls in a row."""
import math
from ctypes import c_char_p, c_float, c_int, c_longlong, c_void_p
from types import SimpleNamespace

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SCRATCH_TOO_SMALL = 100002


def _case(seed, lens, H, KVH, hd):
    """One decoded token per sequence over a shuffled paged cache, and the plain model's attention
    for it (tests/plain_llama.py, float64 on the values the kernel reads)."""
    import plain_llama as pl
    from test_gpu_kernels import _paged
    g = torch.Generator().manual_seed(seed)
    k = [torch.randn(n, KVH, hd, generator=g) for n in lens]
    v = [torch.randn(n, KVH, hd, generator=g) for n in lens]
    cache, tables = _paged(k, v, lens, torch.bfloat16, seed=seed)
    B = len(lens)
    q = (torch.randn(B, H * hd, generator=g) * 1.5).to(torch.bfloat16)
    rd = lambda t: t.to(torch.bfloat16).double()                           # noqa: E731
    plain = []
    for b, n in enumerate(lens):
        qq = torch.zeros(n, H, hd, dtype=torch.float64)
        qq[-1] = q[b].double().reshape(H, hd)
        plain.append(pl.causal_attention(qq, rd(k[b]), rd(v[b]), None)[-1])
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)       # noqa: E731
    ctx = SimpleNamespace(cu_q=i32(list(range(B + 1))), seq_start=i32([n - 1 for n in lens]), seq_qlen=i32([1] * B),
                          tok_seq=i32(list(range(B))), n_seqs=B, max_qlen=1, all_decode=True)
    return q.to(DEV), cache, tables, ctx, torch.stack(plain)


def _entry(hd):
    from oracle_engine_b200.csrc import build
    lib = build.load("attention_tc", {"OE_HD": hd})
    fn = lib.oe_attn_mma_bf16_noalloc
    fn.argtypes = [c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                   c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p]
    fn.restype = c_int
    lib.oe_attn_mma_error_string.argtypes = [c_int]
    lib.oe_attn_mma_error_string.restype = c_char_p
    return lib, fn


def _call(fn, out, q, cache, tables, ctx, n_tokens, H, KVH, scale, n_splits):
    return fn(out.data_ptr(), q.data_ptr(), q.stride(0), cache.data_ptr(), tables.data_ptr(), tables.shape[1],
              ctx.cu_q.data_ptr(), ctx.seq_start.data_ptr(), ctx.seq_qlen.data_ptr(), ctx.tok_seq.data_ptr(),
              ctx.n_seqs, n_tokens, 1, H, KVH, 0, scale, n_splits, torch.cuda.current_stream().cuda_stream)


def test_no_alloc_entry_point_matches_the_ordinary_one():
    from oracle_engine_b200.csrc import ops_tc
    H, KVH, hd = 6, 2, 64
    lib, fn = _entry(hd)
    scale = 1 / math.sqrt(hd)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    for seed, lens in ((1, [300, 65, 1, 129]), (2, [64, 500, 17, 200])):          # two calls in a row
        q, cache, tables, ctx, plain = _case(seed, lens, H, KVH, hd)
        want = torch.empty(len(lens), H * hd, dtype=torch.bfloat16, device=DEV)
        ops_tc.attention(want, q, cache, tables, ctx, H, KVH, hd, 0, scale)      # the existing entry point
        n_splits = ops_tc.decode_splits(ctx.n_seqs, KVH, sms, tables.shape[1])
        assert n_splits > 1                                                        # the scratch is in use
        got = torch.full_like(want, 3.0)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        code = _call(fn, got, q, cache, tables, ctx, len(lens), H, KVH, scale, n_splits)
        assert code == 0, lib.oe_attn_mma_error_string(code).decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        # same kernels, same split order: within the tolerance the kernel tests use (here: equal)
        assert (got.float() - want.float()).abs().max().item() < 2.5e-2
        assert torch.equal(got, want)
        # and on its own feet: against the plain attention, with the kernel tests' tolerance
        assert (got.double().cpu() - plain).abs().max().item() < 2.5e-2
        # one CTA per (sequence, KV head), no split: the scratch is not touched, the result stands
        one = torch.full_like(want, 3.0)
        assert _call(fn, one, q, cache, tables, ctx, len(lens), H, KVH, scale, 1) == 0
        torch.cuda.synchronize()
        assert (one.double().cpu() - plain).abs().max().item() < 2.5e-2
    # a call that needs more scratch than the fixed array is refused before any launch
    code = _call(fn, got, q, cache, tables, ctx, 1 << 20, H, KVH, scale, 32)
    assert code == SCRATCH_TOO_SMALL and b"scratch" in lib.oe_attn_mma_error_string(code)
    torch.cuda.synchronize()


def test_no_alloc_entry_point_at_its_limit():
    """The largest call the fixed array takes (2 Mi floats: with heads of 64, 31,775 x 66 floats =
    41 tokens x 25 heads x 31 splits) runs and is right; one token more is refused."""
    H, KVH, hd, splits = 25, 5, 64, 31
    lib, fn = _entry(hd)
    lib.oe_attn_mma_partial_floats.argtypes = [c_int, c_int, c_int]
    lib.oe_attn_mma_partial_floats.restype = c_longlong
    limit = 2 << 20
    assert lib.oe_attn_mma_partial_floats(41, H, splits) <= limit < lib.oe_attn_mma_partial_floats(42, H, splits)
    lens = [splits * 64 + 5 * i for i in range(42)]                 # at least one page per split
    q, cache, tables, ctx, plain = _case(7, lens, H, KVH, hd)
    scale = 1 / math.sqrt(hd)
    got = torch.full((42, H * hd), 3.0, dtype=torch.bfloat16, device=DEV)
    ctx41 = SimpleNamespace(**{**vars(ctx), "n_seqs": 41})
    assert _call(fn, got, q, cache, tables, ctx41, 41, H, KVH, scale, splits) == 0
    torch.cuda.synchronize()
    assert (got[:41].double().cpu() - plain[:41]).abs().max().item() < 2.5e-2
    assert (got[41] == 3.0).all()                                    # the row beyond the call is untouched
    code = _call(fn, got, q, cache, tables, ctx, 42, H, KVH, scale, splits)
    assert code == SCRATCH_TOO_SMALL
