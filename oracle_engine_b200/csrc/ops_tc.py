"""Entry points of the tensor-core kernels of the bfloat16 serving path.

`gemm`: csrc/gemm_tcgen05.cu (tcgen05.mma + TMA).  Shapes the kernel cannot take (rows
not 16-byte aligned: K or the row stride not a multiple of 8) are reported by
`gemm_supported`, and the caller uses the CUDA-core kernel for them; that choice depends
on shapes only.
"""
from __future__ import annotations

import contextlib
from ctypes import c_int, c_longlong, c_void_p

import torch

from . import build as _build
from . import ops
from .ops import KernelError

_state: dict = {}


class _Knobs:
    """Choices that measurements and tests may pin; the defaults are what serving uses.
    They are set only through `knobs(...)`, which puts the old values back when its block ends."""
    prompt_kernel = "tcgen05"      # "tcgen05" or "mma": the prompt attention kernel for head sizes 64 / 128
    decode_kernel = "auto"         # "auto", "warps", "split": the decode attention kernel
    decode_splits = 0              # > 0: this many CTAs per (sequence, KV head) instead of the rule's
    decode_warps_shape = None      # (warps, ring depth) of the kernel whose warps split the keys, instead of the rule's
    decode_warps_cluster = 0       # > 0: this many CTAs of that kernel share a (sequence, KV head), instead of the rule's
    pair_max_tile = 0              # > 0: an upper limit for the two-SM product's tile width
    sm_count = 0                   # > 0: the products plan their grids for this many SMs
    gemm_schedule = (0, -1, -1, -1, -1)     # one-SM tcgen05 product: tile width, stream-K, cluster, narrow, atoms (see knobs)
    gemm_waits = (0, 0)            # one-SM tcgen05 product: the limit of its waits in ns (0: 2 s), and whether its
                                   # epilogues withhold their accumulators (the test of a wait that runs out)


KNOBS = _Knobs()


@contextlib.contextmanager
def knobs(**kw):
    """with knobs(prompt_kernel="mma", decode_splits=4): ...   pins choices inside the block.
    (A CUDA graph keeps the choices its kernels were captured with: pin them around the engine's whole
    life, or use an engine without graphs.)

    gemm_schedule = (n_tile, stream_k, cluster, narrow[, atoms]) of the one-SM tcgen05 product: its tile
    width for many tokens (0: chosen by the shape), its schedule (1: stream-K wherever the tiles
    leave a remainder, 0: whole tiles, -1: by the shape); for up to 128 tokens whether the K
    splits of a tile may be the CTAs of a cluster (0: never, they add up through the workspace)
    and whether narrow tiles without a split (1) or swap-AB with split K (0) are used (-1: by
    the shape), and how many 64-deep swizzle atoms a k-block of those products holds (1, 2; -1: by
    the shape)."""
    old = {}
    for k, v in kw.items():
        if not hasattr(_Knobs, k):
            raise KeyError(f"unknown knob {k!r}")
        old[k] = getattr(KNOBS, k)
    try:
        for k, v in kw.items():
            setattr(KNOBS, k, (tuple(v) + (-1,) * 5)[:5] if k == "gemm_schedule" else v)
        if "gemm_schedule" in kw:
            _lib().oe_gemm_tc_force(*[int(x) for x in KNOBS.gemm_schedule])
        if "gemm_waits" in kw:
            _lib().oe_gemm_tc_waits(c_longlong(int(KNOBS.gemm_waits[0])), int(KNOBS.gemm_waits[1]))
        yield KNOBS
    finally:
        for k, v in old.items():
            setattr(KNOBS, k, v)
        if "gemm_schedule" in old:
            _lib().oe_gemm_tc_force(*[int(x) for x in KNOBS.gemm_schedule])
        if "gemm_waits" in old:
            _lib().oe_gemm_tc_waits(c_longlong(int(KNOBS.gemm_waits[0])), int(KNOBS.gemm_waits[1]))


def _lib():
    lib = _state.get("gemm")
    if lib is None:
        lib = _build.load("gemm_tc")
        lib.oe_gemm_tc_supported.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_longlong]
        lib.oe_gemm_tc_supported.restype = c_int
        lib.oe_gemm_tc_bf16.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong,
                                        c_int, c_void_p, c_longlong, c_void_p, c_int, c_int, c_void_p]
        lib.oe_gemm_tc_bf16.restype = c_int
        lib.oe_gemm_tc_prefetch.argtypes = [c_void_p, c_longlong]
        lib.oe_gemm_tc_prefetch.restype = None
        lib.oe_gemm_tc_error.argtypes = []
        lib.oe_gemm_tc_error.restype = c_int
        lib.oe_gemm_tc_workspace_bytes.restype = c_longlong
        lib.oe_gemm_tc_counters.restype = c_int
        _state["gemm"] = lib
    return lib


def _scratch(device):
    """Split-K workspace and tile counters of `device` (allocated once, zeroed once)."""
    key = ("scratch", device.index)
    sc = _state.get(key)
    if sc is None:
        lib = _lib()
        ws = torch.empty(lib.oe_gemm_tc_workspace_bytes() // 4, dtype=torch.float32, device=device)
        counters = torch.zeros(lib.oe_gemm_tc_counters(), dtype=torch.int32, device=device)
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        sc = (ws, counters, sms)
        _state[key] = sc
    return sc


def gemm_supported(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        return False
    K = a.shape[1]
    return (K % 8 == 0 and a.stride(0) % 8 == 0 and a.stride(1) == 1 and w.is_contiguous()
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and out.stride(1) == 1)


SKINNY_MAX_TOKENS = 16      # up to here every product goes to the weight-streaming kernel (gemm_skinny.cu).  Alone, the
                            # tcgen05 kernel is the faster one for the large weights from 9 tokens on (us at 16 tokens,
                            # 3072->16384 with SwiGLU, 8192->3072, 3072->5120, 3072->3072; weight-streaming / tcgen05:
                            # 23.8 15.2 12.0 7.2 / 19.9 13.7 10.1 9.2), but a decode step is a chain of kernels that
                            # overlap, and in the chain the weight-streaming kernels with the flags of parts/linear.py
                            # win: 16 sequences of the 3B shape 2.11 ms a step against 2.38 with tcgen05 for the large
                            # weights (12 sequences 2.06 / 2.36); the 1B shape lost 5 % with tcgen05 there as well


def uses_skinny(M: int, N: int, K: int, kind: int) -> bool:
    """Whether a product of M tokens with an [N, K] weight goes to the weight-streaming kernel
    (kind: the epilogue, 1 = float32 store, the logits)."""
    return M <= SKINNY_MAX_TOKENS


PAIR_MIN_TOKENS = 129       # from here on the two-SM kernel (gemm_tcgen05_pair.cu), except where the one-SM kernel can
                            # split K four ways or more over the CTAs of a cluster (few tiles, see uses_pair).  Measured
                            # alone (us; pair / one-SM): 192 tokens 3072->5120 16.0 / 17.0, 3072->16384 SwiGLU 29.8 / 34.1,
                            # 8192->3072 30.8 / 21.5, 3072->3072 15.6 / 14.7; 384 tokens 8192->3072 33.4 / 26.4, 3072->3072
                            # 16.7 / 16.1; 512 tokens 34.2 / 33.4 and 17.4 / 18.6; 2,048 tokens 3072->16384 132 / 149,
                            # 8192->3072 74 / 91


def uses_pair(M: int, N: int, K: int, sm_count: int | None = None) -> bool:
    """Whether a product of M tokens with an [N, K] weight goes to the two-SM kernel."""
    if M < PAIR_MIN_TOKENS or N < 32:
        return False
    if M <= 384 and N >= 256 and K >= 2048:
        tiles = -(-M // 128) * -(-N // 256)              # tiles of 128 x 256 of the one-SM kernel
        if tiles * 4 <= (sm_count or _sm_count()):       # it splits K over a cluster of 4 to 8 CTAs per tile
            return False
    return True


def _pair():
    lib = _state.get("pair")
    if lib is None:
        lib = _build.load("gemm_pair")
        lib.oe_gemm_pair_bf16.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong,
                                          c_int, c_int, c_void_p]
        lib.oe_gemm_pair_bf16.restype = c_int
        lib.oe_gemm_pair_error.restype = c_int
        _state["pair"] = lib
    return lib


def _skinny():
    lib = _state.get("skinny")
    if lib is None:
        lib = _build.load("gemm_skinny")
        lib.oe_gemm_skinny_bf16.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong,
                                            c_int, c_int, c_void_p]
        lib.oe_gemm_skinny_bf16.restype = c_int
        _state["skinny"] = lib
    return lib


NEXT_WEIGHTS_L2_BYTES = 8 << 20     # see gemm(then=)


def gemm(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, accumulate: bool = False, split_k: bool = True,
         swiglu: bool = False, kernel: str = "auto", early: int = 0, then: torch.Tensor | None = None) -> None:
    """out (+)= a @ w.T, a [M, K] and w [N, K] bfloat16; out bfloat16 or float32 [M, N].

    swiglu: w's rows alternate gate and up rows (g0, u0, g1, u1, ...) and out [M, N/2]
    bfloat16 receives silu(gate) * up, computed in float32 in the epilogue.
    kernel: "auto" (weight-streaming kernel for a handful of rows, see uses_skinny, the two-SM tcgen05
    kernel from PAIR_MIN_TOKENS rows, the one-SM tcgen05 kernel otherwise),
    "tcgen05", "pair" or "skinny".
    early (weight-streaming kernel only): bit 0, it may start while the kernel before it drains;
    bit 1, the kernel after it is released only when its CTAs have streamed their weights.
    then (one-SM tcgen05 kernel with up to 128 tokens only): the weight matrix of the product that runs
    after this one; when this kernel's own loads are out it asks the first 8 MB of it into the L2, so that the
    memory does not idle through its epilogue and the next kernel's set-up (decode step of the 28-layer 3B shape,
    ms, without / 4 / 8 / 12 / 32 MB: 32 sequences 2.62 / 2.57 / 2.56 / 2.56 / 2.63, 64: 2.96 / 2.91 / 2.89 / 2.89 / 3.01)."""
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N // 2 if swiglu else N):
        raise KernelError(f"gemm: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)} do not agree")
    if not gemm_supported(a, w, out):
        raise KernelError("gemm: the tensor-core kernel needs bfloat16 operands with 16-byte aligned rows")
    if swiglu:
        if out.dtype != torch.bfloat16 or accumulate or N % 2:
            raise KernelError("gemm: the swiglu epilogue writes bfloat16 and needs an even number of weight rows")
        kind = 3
    elif accumulate:
        if out.dtype != torch.float32:
            raise KernelError("gemm: accumulate needs a float32 output")
        kind = 2
    elif out.dtype == torch.bfloat16:
        kind = 0
    elif out.dtype == torch.float32:
        kind = 1
    else:
        raise KernelError("gemm: output must be bfloat16 or float32")
    if kernel == "skinny" or (kernel == "auto" and uses_skinny(M, N, K, kind)):
        code = _skinny().oe_gemm_skinny_bf16(out.data_ptr(), a.data_ptr(), w.data_ptr(), M, N, K, a.stride(0),
                                             out.stride(0), kind, int(early), ops._stream())
        ops._check(code, "gemm_skinny", (M, N, K))
        return
    if kernel == "pair" or (kernel == "auto" and uses_pair(M, N, K, KNOBS.sm_count or None)):
        code = _pair().oe_gemm_pair_bf16(out.data_ptr(), a.data_ptr(), w.data_ptr(), M, N, K, a.stride(0), out.stride(0),
                                         kind, int(KNOBS.pair_max_tile), ops._stream())
        ops._check(code, "gemm_pair", (M, N, K))
        return
    ws, counters, sms = _scratch(a.device)
    sms = KNOBS.sm_count or sms
    if then is not None and M <= 128 and then.is_cuda and NEXT_WEIGHTS_L2_BYTES > 0:
        _lib().oe_gemm_tc_prefetch(then.data_ptr(), min(NEXT_WEIGHTS_L2_BYTES, then.numel() * then.element_size()))
    code = _lib().oe_gemm_tc_bf16(out.data_ptr(), a.data_ptr(), w.data_ptr(), M, N, K, a.stride(0), out.stride(0), kind,
                                  ws.data_ptr() if split_k else None, ws.numel() * 4,
                                  counters.data_ptr() if split_k else None, counters.numel(), sms,
                                  ops._stream())
    ops._check(code, "gemm_tc", (M, N, K))


def device_error() -> int:
    """The code of a bounded wait that ran out inside a tensor-core kernel since the last
    call (0 = none).  Synchronises the device."""
    code = 0
    if "gemm" in _state:
        code = int(_lib().oe_gemm_tc_error())
    if "pair" in _state:
        code = code or int(_state["pair"].oe_gemm_pair_error())
    for key, lib in list(_state.items()):
        if isinstance(key, tuple) and key[0] == "attn_tc5":
            code = code or int(lib.oe_attn_tc_error())
    return code


# ----------------------------------------------------------------------------------------
# attention (csrc/attention_mma.cu, one library per head size)
# ----------------------------------------------------------------------------------------
from ctypes import c_float  # noqa: E402


def attention_supported(head_dim: int, n_heads: int, n_kv_heads: int) -> bool:
    return head_dim % 16 == 0 and 16 <= head_dim <= 256 and n_heads % n_kv_heads == 0 \
        and n_heads // n_kv_heads <= 64


def _attn_lib(head_dim: int):
    key = ("attn", head_dim)
    lib = _state.get(key)
    if lib is None:
        lib = _build.load("attention_tc", {"OE_HD": head_dim})
        lib.oe_attn_mma_bf16.argtypes = [c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                         c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                                         c_void_p, c_void_p]
        lib.oe_attn_mma_bf16.restype = c_int
        lib.oe_attn_decode_fused_bf16.argtypes = [c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int,
                                                  c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                                  c_int, c_float, c_int, c_void_p, c_void_p, c_void_p]
        lib.oe_attn_decode_fused_bf16.restype = c_int
        lib.oe_attn_decode_warps_bf16.argtypes = [c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int,
                                                  c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                                  c_int, c_float, c_int, c_int, c_void_p]
        lib.oe_attn_decode_warps_bf16.restype = c_int
        lib.oe_attn_mma_partial_floats.argtypes = [c_int, c_int, c_int]
        lib.oe_attn_mma_partial_floats.restype = c_longlong
        _state[key] = lib
    return lib


TCGEN05_ATTENTION_HEAD_DIMS = (64, 128)


def _attn_tc5_lib(head_dim: int):
    key = ("attn_tc5", head_dim)
    lib = _state.get(key)
    if lib is None:
        lib = _build.load("attention_tc5", {"OE_HD": head_dim})
        lib.oe_attn_tc_bf16.argtypes = [c_void_p, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_int, c_void_p,
                                        c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p]
        lib.oe_attn_tc_bf16.restype = c_int
        lib.oe_attn_tc_error.argtypes = []
        lib.oe_attn_tc_error.restype = c_int
        _state[key] = lib
    return lib


# Context classes (engine/batch.py: the longest sequence of a step is up to 768, 1,536, 4,096 tokens, or longer)
MID_CONTEXT, LONG_CONTEXT, VERY_LONG_CONTEXT = 1, 2, 3


def decode_splits(n_seqs: int, n_kv_heads: int, sm_count: int, max_pages: int, context_class: int = 0,
                  ctas_per_sm: int = 3) -> int:
    """How many CTAs share one (sequence, KV head) of a decode step, never more than the pages a
    sequence can have.  Depends on the batch size, the step's context class and the cache
    geometry only, so a captured graph stays valid.
    Short contexts: enough CTAs to occupy the GPU about twice.  Long contexts, where the time is
    the keys' bytes: the fewest splits that fill the last round of resident CTAs (ctas_per_sm x SMs)
    to 85 %, else the best-filled; measured at 8,000 keys (us): 8 sequences 5 / 6 splits 57 / 50,
    32 sequences 2 / 3 splits 246 / 175, 40 sequences 1 / 4 splits 362 / 206."""
    if KNOBS.decode_splits > 0:
        return max(1, min(max_pages, 32, KNOBS.decode_splits))
    ctas = max(1, n_seqs * n_kv_heads)
    cap = max(1, min(max_pages, 32))
    if context_class < LONG_CONTEXT:
        return max(1, min(cap, (2 * sm_count + ctas - 1) // ctas))
    resident = max(1, ctas_per_sm) * sm_count
    best, best_fill = 1, 0.0
    for s in range(1, cap + 1):
        rounds = (ctas * s + resident - 1) // resident
        fill = ctas * s / (rounds * resident)
        if fill >= 0.85:
            return s
        if fill > best_fill + 1e-9:
            best, best_fill = s, fill
    return best


def decode_splits_for(n_seqs: int, n_kv_heads: int, tables, context_class: int = 0, head_dim: int = 0) -> int:
    sms = torch.cuda.get_device_properties(tables.device).multi_processor_count
    per_sm = _decode_ctas_per_sm(head_dim) if head_dim and context_class >= LONG_CONTEXT else 3
    return decode_splits(n_seqs, n_kv_heads, sms, tables.shape[1], context_class, per_sm)


def _decode_ctas_per_sm(head_dim: int) -> int:
    key = ("decode_ctas_per_sm", head_dim)
    if key not in _state:
        n = int(_attn_lib(head_dim).oe_attn_mma_decode_ctas_per_sm())
        if n <= 0:
            raise KernelError("attention: the decode kernel does not fit an SM")
        _state[key] = n
    return _state[key]


def attention(out, qkv, cache, tables, ctx, n_heads: int, n_kv_heads: int, head_dim: int, window: int,
              scale: float) -> None:
    """out[t] = attention of the step's tokens over their sequences' paged cache (bfloat16).

    qkv [T, >= H hd] (queries first), out [T, H hd], cache [pages, 2, KVH, PAGE, hd]."""
    T = out.shape[0]
    if out.dtype != torch.bfloat16 or qkv.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16:
        raise KernelError("attention: bfloat16 tensors expected")
    if not out.is_contiguous() or out.shape[1] != n_heads * head_dim or qkv.stride(1) != 1 or not cache.is_contiguous():
        raise KernelError("attention: out must be contiguous [T, H hd]; cache contiguous")
    if tuple(cache.shape[1:]) != (2, n_kv_heads, ops.PAGE, head_dim):
        raise KernelError("attention: cache entry must be [pages, 2, KVH, PAGE, head_dim]")
    group = n_heads // n_kv_heads
    if (KNOBS.prompt_kernel == "tcgen05" and head_dim in TCGEN05_ATTENTION_HEAD_DIMS and ctx.max_qlen * group > 64
            and group <= 128 and qkv.stride(0) % 8 == 0 and qkv.data_ptr() % 16 == 0):
        # prompts: S and O_blk in tensor memory (csrc/attention_tcgen05.cu)
        code = _attn_tc5_lib(head_dim).oe_attn_tc_bf16(
            out.data_ptr(), qkv.data_ptr(), qkv.stride(0), cache.data_ptr(), cache.shape[0], tables.data_ptr(),
            tables.shape[1], ctx.cu_q.data_ptr(), ctx.seq_start.data_ptr(), ctx.seq_qlen.data_ptr(), ctx.n_seqs, T,
            ctx.max_qlen, n_heads, n_kv_heads, int(window), float(scale), ops._stream())
        ops._check(code, "attention_tcgen05")
        return
    lib = _attn_lib(head_dim)
    n_splits, partial = 1, None
    if ctx.all_decode and group <= 16:
        n_splits = decode_splits_for(ctx.n_seqs, n_kv_heads, tables, getattr(ctx, "context_class", 0), head_dim)
        if n_splits > 1:
            partial = torch.empty(lib.oe_attn_mma_partial_floats(T, n_heads, n_splits), dtype=torch.float32,
                                  device=out.device)
    code = lib.oe_attn_mma_bf16(out.data_ptr(), qkv.data_ptr(), qkv.stride(0), cache.data_ptr(), tables.data_ptr(),
                                tables.shape[1], ctx.cu_q.data_ptr(), ctx.seq_start.data_ptr(),
                                ctx.seq_qlen.data_ptr(), ctx.tok_seq.data_ptr(), ctx.n_seqs, T, max(1, ctx.max_qlen),
                                n_heads, n_kv_heads, int(window), float(scale), n_splits,
                                None if partial is None else partial.data_ptr(),
                                ops._stream())
    ops._check(code, "attention_mma", {"splits": n_splits})
    if n_splits > 1:
        ops.LAUNCHES[0] += 1


def decode_fused_supported(head_dim: int, n_heads: int, n_kv_heads: int) -> bool:
    return attention_supported(head_dim, n_heads, n_kv_heads) and head_dim % 32 == 0


DECODE_WARPS_FORMS = ((6, 2), (2, 3), (1, 3))    # (warps, tiles in a warp's ring) the rule picks from (csrc/attention_mma.cu)
SM_SHARED_BYTES = 227 * 1024   # what the CTAs resident on an SM share, each with 1 KB of the system's on top


def decode_warps_supported(head_dim: int, n_heads: int, n_kv_heads: int) -> bool:
    return decode_fused_supported(head_dim, n_heads, n_kv_heads) and n_heads // n_kv_heads <= 16


def decode_uses_warps(n_seqs: int, context_class: int, head_dim: int, n_heads: int, n_kv_heads: int,
                      sm_count: int | None = None) -> bool:
    """Whether a decode step goes to the kernel whose warps split the keys (one launch, no
    scratch) rather than to CTAs that split the keys plus a merge.  Depends on the batch size and
    the step's context class (engine/batch.py) only; a captured graph is kept per class.
    It is used wherever it can be (groups of up to 16 heads, head sizes that are multiples of 32).
    Alone, the split kernels are faster for few long sequences (us, 24 heads over 8 KV heads of 128;
    warps / split: 2,048 keys, 1 sequence 20 / 12; 8,000 keys, 1: 63 / 18, 8: 66 / 56), but inside the
    decode step their three launches cost the overlap with the products around them (ms a step of the
    28-layer model, split / warps: 2,048-token contexts, 1 sequence 2.50 / 1.93, 8: 3.17 / 2.05; 6,000
    tokens, 1: 2.60 / 2.74, 16: 4.40 / 4.03), and with a cluster per pair (`decode_warps_cluster`) the
    warps kernel wins there too (1 sequence at 6,000 tokens: 1.80)."""
    if KNOBS.decode_kernel == "split" or not decode_warps_supported(head_dim, n_heads, n_kv_heads):
        return False
    return True


def decode_warps_per_sm(shape: tuple, head_dim: int) -> int:
    """How many CTAs of a form of the warps kernel an SM holds (0: the form does not fit)."""
    smem = shape[0] * shape[1] * 2 * 32 * (head_dim * 2 + 16)      # K and V tiles of 32 padded rows
    return 0 if smem > 220 * 1024 else SM_SHARED_BYTES // (smem + 1024)


def decode_warps_shape(n_seqs: int, context_class: int, head_dim: int, n_kv_heads: int,
                       sm_count: int | None = None) -> tuple:
    """(warps, tiles in each warp's ring) for the kernel whose warps split the keys.

    What an SM streams is its bytes in flight over the memory latency, and a CTA's start and
    merge hide only behind another CTA of the same SM.  So: the form with the most warps whose
    CTAs are all resident at once (at head size 128 one CTA an SM for up to 148 pairs, then two,
    then four); with more pairs than that, short contexts take the smallest CTAs.  Long contexts
    leave the one-warp form out (a lone warp's arithmetic shows there) and, past one round, take
    the form whose last round of CTAs is fullest.  Measured (us; 24 heads over 8 KV heads of 128; 6x2 / 2x3 /
    1x3 / the one-warp kernel with one staged page):
    600 keys:   16 sequences 10.5 / 14.0 / 20.6 / -,  24: 19.2 / 15.0 / 22.8 / -,  32: 21.2 / 16.1 / 24.2 / -,
                48: 31.5 / 31.4 / 24.9 / 35.2,  64: 41.9 / 33.1 / 31.3 / 37.8,  128: 74.1 / 64.1 / 55.3 / 74.2
    2,100 keys: 24: 46.0 / 40.0 / 67.3,  32: 48.3 / 49.0 / 70.5,  48: 71.9 / 83.8 / 73.9,  64: 95.1 / 87.2 / 96.4,
                96: 139 / 132 / 155,  128: 182 / 174 / 169;   8,000 keys, 64: 314 / 309 / 349."""
    if KNOBS.decode_warps_shape is not None:
        return tuple(KNOBS.decode_warps_shape)
    sms = sm_count or _sm_count()
    pairs = max(1, n_seqs * n_kv_heads)
    forms, seen = [], set()
    for shape in DECODE_WARPS_FORMS:                # most warps first; one form for each number of CTAs an SM holds
        per_sm = decode_warps_per_sm(shape, head_dim)
        if per_sm > 0 and per_sm not in seen:
            seen.add(per_sm)
            forms.append((shape, per_sm * sms))
    if not forms:
        raise KernelError(f"attention_decode_warps: no form of the kernel fits an SM at head size {head_dim}")
    if context_class >= LONG_CONTEXT and len(forms) > 1:
        forms = forms[:-1]
    for shape, slots in forms:
        if pairs <= slots:
            return shape
    if context_class < LONG_CONTEXT:
        return forms[-1][0]
    best, best_fill = forms[0][0], 0.0
    for shape, slots in forms:
        fill = pairs / (-(-pairs // slots) * slots)
        if fill >= best_fill - 1e-9:                 # equal fill: the smaller CTAs, whose tail is shorter
            best, best_fill = shape, fill
    return best


def decode_warps_cluster(n_seqs: int, context_class: int, n_kv_heads: int, sm_count: int | None = None) -> int:
    """How many CTAs (a thread-block cluster) of the warps kernel share one (sequence, KV head).

    One where the context is short or the pairs alone fill the SMs.  Past 768 keys, few sequences are
    streamed by 2 or 4 CTAs each (8 for a single sequence past 4,096 keys), which add up through the
    cluster's shared memory, as long as all clusters are resident at once (ms a step of the 28-layer model
    with 1 / 2 / 4 CTAs per pair at 1,400 tokens: 1 sequence 1.79 / 1.68 / 1.64, 4 sequences 1.85 / 1.77 / 2.56;
    at 512 tokens 1.595 / 1.578 / 1.582 and 1.66 / 1.67 / 2.53, at 128 tokens 1.51 / 1.54 / 1.57).  Measured alone (us; 24 heads over
    8 KV heads of 128, six warps x two tiles; 1 / 2 / 4 / 8 CTAs, and the split kernels + merge):
    2,100 keys: 1 sequence 18.4 / 12.5 / 8.8 / 9.6 (12), 4: 19.0 / 13.3 / 12.3 / 29 , 8: 19.5 / 16.1 / 23.8 / 51 (22);
    8,000 keys: 1: 61 / 34 / 21 / 15.6 (18), 2: 62 / 35 / 21.5 / 30, 4: 63 / 36 / 27.5 / 46, 8: 64 / 44.8 / 52 / 80 (56),
    16: 88 / 85 / 101 / 149 (90).  530 keys, 8 sequences: 7.0 / 9.0 / 15.4 / 41."""
    if KNOBS.decode_warps_cluster > 0:
        return int(KNOBS.decode_warps_cluster)
    if context_class < MID_CONTEXT:
        return 1
    # Inside the decode step the attention's CTAs (a whole SM's shared memory and two thirds of its
    # registers each) must leave SMs to the products before and after it, which overlap it: with more than
    # about 64 of them on 148 SMs the step loses more than the attention gains (ms a step of the 28-layer
    # model, 1 / 2 / 4 CTAs per pair; 2,048-token contexts: 1 sequence 1.93 / 1.76 / 1.69, 4: 1.98 / 1.85 /
    # 2.62, 8: 2.05 / 2.93 / 3.13; 6,000 tokens: 2: 2.77 / 2.20 / 1.95, 4: 2.82 / 2.27 / 2.93, 8: 2.88 / 3.49 / 3.68).
    budget = (sm_count or _sm_count()) * 7 // 16
    pairs = max(1, n_seqs * n_kv_heads)
    for cr in ((8, 4, 2) if context_class >= VERY_LONG_CONTEXT else (4, 2)):
        if pairs * cr <= budget:
            return cr
    return 1


def _sm_count() -> int:
    if "sms" not in _state:
        _state["sms"] = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return _state["sms"]


def attention_decode_warps(out, qkv, cos, sin, cache, tables, ctx, n_heads: int, n_kv_heads: int, head_dim: int,
                           window: int, scale: float, has_kv: bool, shape: tuple | None = None,
                           cluster: int | None = None) -> None:
    """The decode step's mixer core (rotation, cache write, attention) in one launch: one CTA per
    (sequence, KV head), whose warps split the keys (csrc/attention_mma.cu).  Same arguments as
    attention_decode_fused; shape = (warps, tiles in each warp's ring), None: `decode_warps_shape`;
    cluster = CTAs that share one (sequence, KV head), None: `decode_warps_cluster`."""
    if out.dtype != torch.bfloat16 or qkv.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16:
        raise KernelError("attention_decode_warps: bfloat16 tensors expected")
    width = (n_heads + (2 * n_kv_heads if has_kv else 0)) * head_dim
    if qkv.shape[1] != width or qkv.stride(1) != 1 or not out.is_contiguous() or not cache.is_contiguous():
        raise KernelError(f"attention_decode_warps: qkv must be [B, {width}], out and cache contiguous")
    if tuple(cache.shape[1:]) != (2, n_kv_heads, ops.PAGE, head_dim):
        raise KernelError("attention_decode_warps: cache entry must be [pages, 2, KVH, PAGE, head_dim]")
    lib = _attn_lib(head_dim)
    if shape is None:
        shape = decode_warps_shape(ctx.n_seqs, getattr(ctx, "context_class", 0), head_dim, n_kv_heads)
    if cluster is None:
        cluster = decode_warps_cluster(ctx.n_seqs, getattr(ctx, "context_class", 0), n_kv_heads)
    code = lib.oe_attn_decode_warps_bf16(
        out.data_ptr(), qkv.data_ptr(), qkv.stride(0), None if cos is None else cos.data_ptr(),
        None if sin is None else sin.data_ptr(), cache.data_ptr(), int(has_kv), tables.data_ptr(), tables.shape[1],
        ctx.cu_q.data_ptr(), ctx.seq_start.data_ptr(), ctx.seq_qlen.data_ptr(), ctx.n_seqs, n_heads, n_kv_heads,
        int(window), float(scale), shape[0] * 16 + shape[1], int(cluster), ops._stream())
    ops._check(code, "attention_decode_warps", {"warps": shape[0], "ring": shape[1], "cluster": int(cluster)})


def _attn_counters(device):
    key = ("attn_counters", device.index)
    c = _state.get(key)
    if c is None:
        c = torch.zeros(1 << 16, dtype=torch.int32, device=device)
        _state[key] = c
    return c


def attention_decode_fused(out, qkv, cos, sin, cache, tables, ctx, n_heads: int, n_kv_heads: int, head_dim: int,
                           window: int, scale: float, has_kv: bool, n_splits: int | None = None) -> None:
    """One kernel for a decode step's mixer core: rotates q and the new k, stores k and v
    in the cache (has_kv), attends over the sequence's pages split across CTAs and merges.
    n_splits: CTAs per (sequence, KV head); None: the rule of `decode_splits_for` for the step's
    context class (the caller that chose this kernel by that rule passes what it got).

    qkv [B, (H + 2 KVH) hd] (or [B, H hd] when has_kv is false) before rotation; cos/sin
    float32 [max_pos, hd/2] or None; every sequence of the step brings exactly one token."""
    B = out.shape[0]
    if out.dtype != torch.bfloat16 or qkv.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16:
        raise KernelError("attention_decode_fused: bfloat16 tensors expected")
    width = (n_heads + (2 * n_kv_heads if has_kv else 0)) * head_dim
    if qkv.shape[1] != width or qkv.stride(1) != 1 or not out.is_contiguous() or not cache.is_contiguous():
        raise KernelError(f"attention_decode_fused: qkv must be [B, {width}], out and cache contiguous")
    if tuple(cache.shape[1:]) != (2, n_kv_heads, ops.PAGE, head_dim):
        raise KernelError("attention_decode_fused: cache entry must be [pages, 2, KVH, PAGE, head_dim]")
    if ctx.n_seqs * n_kv_heads > (1 << 16):
        raise KernelError("attention_decode_fused: too many sequences for the merge counters")
    lib = _attn_lib(head_dim)
    if n_splits is None:
        n_splits = decode_splits_for(ctx.n_seqs, n_kv_heads, tables, getattr(ctx, "context_class", 0), head_dim)
    partial = None
    if n_splits > 1:
        partial = torch.empty(lib.oe_attn_mma_partial_floats(B, n_heads, n_splits), dtype=torch.float32,
                              device=out.device)
    code = lib.oe_attn_decode_fused_bf16(
        out.data_ptr(), qkv.data_ptr(), qkv.stride(0), None if cos is None else cos.data_ptr(),
        None if sin is None else sin.data_ptr(), cache.data_ptr(), int(has_kv), tables.data_ptr(), tables.shape[1],
        ctx.cu_q.data_ptr(), ctx.seq_start.data_ptr(), ctx.seq_qlen.data_ptr(), ctx.n_seqs, n_heads, n_kv_heads,
        int(window), float(scale), n_splits, None if partial is None else partial.data_ptr(),
        _attn_counters(out.device).data_ptr(), ops._stream())
    ops._check(code, "attention_decode_fused", {"splits": n_splits})
