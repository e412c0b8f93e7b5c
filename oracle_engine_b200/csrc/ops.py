"""Typed Python entry points of the CUDA kernels (ctypes over the libraries of build.py).

Every function takes CUDA tensors, checks what the kernel assumes (device, dtype,
contiguity, shapes), launches on torch's current stream and raises `KernelError` if the
kernel refuses the sizes or the launch fails.  Nothing here computes on the host, and
nothing falls back to a library when the extension is missing.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_float, c_longlong, c_void_p

import torch

from . import build as _build

ERR_UNSUPPORTED = 100001
PAGE = 64            # tokens per cache page; must equal OE_PAGE of common.cuh
MAX_HEAD_DIM = 256   # the largest head size the attention kernels take; must equal MAX_HD of attention.cu


class KernelError(RuntimeError):
    pass


def require_cuda() -> None:
    if not torch.cuda.is_available():
        raise KernelError("oracle_engine_b200 needs a CUDA device (B200, sm_100a): there is no CPU path")


_SUFFIX = {torch.float32: "f32", torch.bfloat16: "bf16"}

_P, _I, _F, _L = c_void_p, c_int, c_float, c_longlong
_SIGNATURES = {
    "elementwise": {
        "oe_embed_gather": [_P, _P, _P, _I, _I, _I, _P, _P],
        "oe_rmsnorm": [_P, _P, _P, _I, _I, _F, _P],
        "oe_rope_kv_write": [_P, _I, _P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _P],
        "oe_swiglu": [_P, _P, _I, _I, _P],
        "oe_gather_rows_f32": [_P, _P, _P, _I, _I, _P],
    },
    "gemm_simple": {
        "oe_gemm_simple": [_P, _P, _P, _I, _I, _I, _L, _L, _I, _P],
    },
    "attention": {
        "oe_attn_paged": [_P, _P, _I, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _P],
    },
    "sampling": {
        "oe_argmax_rows": [_P, _P, _I, _I, _P],
        "oe_argmax_rows_wide": [_P, _P, _P, _P, _I, _I, _P],
        "oe_sample_rows": [_P, _P, _P, _I, _I, _F, _I, _F, _F, _I, _P, _P, _P, _P, _I, _I, _P],
    },
}
_TYPED = {"oe_embed_gather", "oe_rmsnorm", "oe_rope_kv_write", "oe_swiglu", "oe_gemm_simple", "oe_attn_paged"}
_fn_cache: dict[str, object] = {}


def _fn(lib: str, name: str, dtype=None):
    full = f"{name}_{_SUFFIX[dtype]}" if name in _TYPED else name
    f = _fn_cache.get(full)
    if f is None:
        f = getattr(_build.load(lib), full)
        f.argtypes = _SIGNATURES[lib][name]
        f.restype = c_int
        _fn_cache[full] = f
    return f


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current CUDA stream's handle.  torch.cuda.current_stream() builds a Python object on
    every call (about 17 us); the raw query is what a kernel launch per few microseconds needs."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


LAUNCHES = [0]          # kernels launched through this module (or captured into a graph)
OBSERVER = [None]       # engine/profile.py: an object whose mark(what, detail) hears of every launch


def _check(code: int, what: str, detail=None) -> None:
    if code == 0:
        LAUNCHES[0] += 1
        if OBSERVER[0] is not None:
            OBSERVER[0].mark(what, detail)
        return
    if code == ERR_UNSUPPORTED:
        raise KernelError(f"{what}: sizes outside what this kernel takes")
    raise KernelError(f"{what}: CUDA error {code} at launch ({torch.cuda.get_device_name()})")


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _dev(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel arguments must be CUDA tensors")


def _i32(t: torch.Tensor, name: str) -> None:
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{name} must be a contiguous int32 tensor")


# ----------------------------------------------------------------------------------------

def embed_gather(x: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, err: torch.Tensor | None) -> None:
    """x[t] = table[ids[t]] as float32; ids outside the table set err[0] = 1 and give zeros."""
    _dev(x, table, ids, err)
    _i32(ids, "ids")
    n, D = x.shape
    if x.dtype != torch.float32 or not x.is_contiguous() or not table.is_contiguous() or table.shape[1] != D:
        raise KernelError("embed_gather: x must be float32 [n, D] and table [V, D], contiguous")
    if ids.numel() < n:
        raise KernelError("embed_gather: fewer ids than rows")
    _check(_fn("elementwise", "oe_embed_gather", table.dtype)(
        _ptr(x), _ptr(table), _ptr(ids), n, D, table.shape[0], _ptr(err), _stream()), "embed_gather")


def rmsnorm(y: torch.Tensor, x: torch.Tensor, w: torch.Tensor, eps: float) -> None:
    """y = (x / sqrt(mean(x^2) + eps)) * w, x float32 [rows, D], w float32 [D]."""
    _dev(y, x, w)
    rows, D = x.shape
    if x.dtype != torch.float32 or w.dtype != torch.float32 or w.numel() != D or y.shape != x.shape:
        raise KernelError("rmsnorm: x and w must be float32, y of x's shape")
    if not (x.is_contiguous() and y.is_contiguous() and w.is_contiguous()):
        raise KernelError("rmsnorm: tensors must be contiguous")
    _check(_fn("elementwise", "oe_rmsnorm", y.dtype)(_ptr(y), _ptr(x), _ptr(w), rows, D, float(eps), _stream()),
           "rmsnorm")


def rope_kv_write(qkv: torch.Tensor, cos: torch.Tensor | None, sin: torch.Tensor | None,
                  cache: torch.Tensor | None, tables: torch.Tensor, tok_seq: torch.Tensor,
                  tok_pos: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, has_kv: bool) -> None:
    """Rotates q (in place) and k at each token's position and writes k, v to the paged cache.

    qkv [T, (H + 2 KVH) hd] (or [T, H hd] when has_kv is false); cos/sin float32
    [max_pos, hd/2] or None for no rotation; cache one entry [pages, 2, KVH, PAGE, hd];
    tables int32 [B, max_pages]; tok_seq / tok_pos int32 [T] (tok_seq < 0: padding row)."""
    _dev(qkv, cos, sin, cache, tables, tok_seq, tok_pos)
    for t, n in ((tables, "tables"), (tok_seq, "tok_seq"), (tok_pos, "tok_pos")):
        _i32(t, n)
    T = qkv.shape[0]
    width = (n_heads + (2 * n_kv_heads if has_kv else 0)) * head_dim
    if qkv.shape[1] != width or qkv.stride(1) != 1:
        raise KernelError(f"rope_kv_write: qkv must be [T, {width}]")
    rotate = cos is not None
    if rotate and (cos.dtype != torch.float32 or cos.shape[1] != head_dim // 2 or not cos.is_contiguous()
                   or sin.shape != cos.shape or not sin.is_contiguous()):
        raise KernelError("rope_kv_write: cos/sin must be float32 [max_pos, head_dim/2]")
    if has_kv:
        if cache is None or cache.dtype != qkv.dtype or not cache.is_contiguous() or \
                tuple(cache.shape[1:]) != (2, n_kv_heads, PAGE, head_dim):
            raise KernelError("rope_kv_write: cache entry must be [pages, 2, KVH, PAGE, head_dim] of qkv's dtype")
    _check(_fn("elementwise", "oe_rope_kv_write", qkv.dtype)(
        _ptr(qkv), qkv.stride(0), _ptr(cos), _ptr(sin), _ptr(cache), _ptr(tables), tables.shape[1],
        _ptr(tok_seq), _ptr(tok_pos), T, n_heads, n_kv_heads, head_dim, int(has_kv), int(rotate), _stream()),
        "rope_kv_write")


def swiglu(out: torch.Tensor, gu: torch.Tensor) -> None:
    """out = silu(gu[:, :FF]) * gu[:, FF:]."""
    _dev(out, gu)
    rows, FF = out.shape
    if gu.shape != (rows, 2 * FF) or gu.dtype != out.dtype or not (gu.is_contiguous() and out.is_contiguous()):
        raise KernelError("swiglu: gu must be [rows, 2 FF] and out [rows, FF], same dtype, contiguous")
    _check(_fn("elementwise", "oe_swiglu", out.dtype)(_ptr(out), _ptr(gu), rows, FF, _stream()), "swiglu")


def gather_rows_f32(out: torch.Tensor, x: torch.Tensor, rows: torch.Tensor) -> None:
    _dev(out, x, rows)
    _i32(rows, "rows")
    if x.dtype != torch.float32 or out.dtype != torch.float32 or not (x.is_contiguous() and out.is_contiguous()):
        raise KernelError("gather_rows_f32: float32 contiguous tensors expected")
    _check(_fn("elementwise", "oe_gather_rows_f32")(_ptr(out), _ptr(x), _ptr(rows), out.shape[0], x.shape[1],
                                                    _stream()), "gather_rows_f32")


def gemm_simple(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, accumulate: bool = False) -> None:
    """out (+)= a @ w.T on the CUDA cores with float32 accumulation in k order.

    a [M, K] and w [N, K] of one dtype (float32 or bfloat16); out [M, N] of that dtype or
    float32; accumulate needs a float32 out."""
    _dev(out, a, w)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N) or a.dtype != w.dtype or not w.is_contiguous():
        raise KernelError(f"gemm: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)} do not agree")
    if a.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm: rows of a and out must be contiguous")
    if accumulate:
        if out.dtype != torch.float32:
            raise KernelError("gemm: accumulate needs a float32 output")
        kind = 2
    elif out.dtype == a.dtype:
        kind = 0
    elif out.dtype == torch.float32:
        kind = 1
    else:
        raise KernelError("gemm: output must have the inputs' dtype or float32")
    _check(_fn("gemm_simple", "oe_gemm_simple", a.dtype)(
        _ptr(out), _ptr(a), _ptr(w), M, N, K, a.stride(0), out.stride(0), kind, _stream()), "gemm_simple")


def attn_paged(out: torch.Tensor, q: torch.Tensor, cache: torch.Tensor, tables: torch.Tensor,
               tok_seq: torch.Tensor, tok_pos: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
               window: int, scale: float) -> None:
    """out[t] = attention of token t's query heads over keys (pos-window, pos] of its sequence.

    q [T, >= H hd] (row stride free, e.g. a view of the qkv buffer), out [T, H hd]."""
    _dev(out, q, cache, tables, tok_seq, tok_pos)
    for t, n in ((tables, "tables"), (tok_seq, "tok_seq"), (tok_pos, "tok_pos")):
        _i32(t, n)
    T = out.shape[0]
    if out.shape[1] != n_heads * head_dim or not out.is_contiguous() or q.stride(1) != 1 or q.dtype != out.dtype:
        raise KernelError("attn_paged: out must be contiguous [T, H hd] and q of its dtype")
    if cache.dtype != out.dtype or not cache.is_contiguous() or \
            tuple(cache.shape[1:]) != (2, n_kv_heads, PAGE, head_dim):
        raise KernelError("attn_paged: cache entry must be [pages, 2, KVH, PAGE, head_dim]")
    _check(_fn("attention", "oe_attn_paged", out.dtype)(
        _ptr(out), _ptr(q), q.stride(0), _ptr(cache), _ptr(tables), tables.shape[1], _ptr(tok_seq), _ptr(tok_pos),
        T, n_heads, n_kv_heads, head_dim, int(window), float(scale), _stream()), "attn_paged")


_argmax_scratch: dict = {}


def argmax_rows(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = index of the first maximum of row r (float32 logits)."""
    _dev(logits, out)
    _i32(out, "out")
    if logits.dtype != torch.float32 or not logits.is_contiguous():
        raise KernelError("argmax_rows: logits must be contiguous float32")
    rows, V = logits.shape
    if V >= 8192 and rows <= 4096:
        # wide vocabulary: slices of a row on different SMs, then one warp per row
        key = (logits.device.index, rows)
        sc = _argmax_scratch.get(key)
        if sc is None:
            sc = (torch.empty(rows * 32, dtype=torch.float32, device=logits.device),
                  torch.empty(rows * 32, dtype=torch.int32, device=logits.device))
            _argmax_scratch[key] = sc
        _check(_fn("sampling", "oe_argmax_rows_wide")(_ptr(logits), _ptr(out), _ptr(sc[0]), _ptr(sc[1]), rows, V,
                                                      _stream()), "argmax_rows")
        LAUNCHES[0] += 1
        return
    _check(_fn("sampling", "oe_argmax_rows")(_ptr(logits), _ptr(out), logits.shape[0], logits.shape[1], _stream()),
           "argmax_rows")


def sample_rows(logits: torch.Tensor, out: torch.Tensor, row_slot: torch.Tensor, temperature: float, top_k: int,
                top_p: float, repeat_penalty: float, repeat_last_n: int, rng_seed: torch.Tensor,
                rng_counter: torch.Tensor, hist: torch.Tensor | None, hist_count: torch.Tensor | None,
                record: bool = True) -> None:
    """One token per row of float32 logits (overwritten), by the reference's sampling chain."""
    _dev(logits, out, row_slot, rng_seed, rng_counter, hist, hist_count)
    _i32(out, "out")
    _i32(row_slot, "row_slot")
    _i32(rng_counter, "rng_counter")
    if rng_seed.dtype != torch.int64:
        raise KernelError("sample_rows: rng_seed must be int64")
    if logits.dtype != torch.float32 or not logits.is_contiguous():
        raise KernelError("sample_rows: logits must be contiguous float32")
    cap = 0
    if hist is not None:
        _i32(hist, "hist")
        _i32(hist_count, "hist_count")
        cap = hist.shape[1]
    _check(_fn("sampling", "oe_sample_rows")(
        _ptr(logits), _ptr(out), _ptr(row_slot), logits.shape[0], logits.shape[1], float(temperature), int(top_k),
        float(top_p), float(repeat_penalty), int(repeat_last_n), _ptr(rng_seed), _ptr(rng_counter), _ptr(hist),
        _ptr(hist_count), cap, int(record), _stream()), "sample_rows")
