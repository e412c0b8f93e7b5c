"""Isolated kernels: correctness against a float64 restatement, then time and roofline.

    python -m oracle_engine_b200.csrc.microbench gemm --m 8 --n 16384 --k 3072 [--out swiglu] [--kernel auto]
    python -m oracle_engine_b200.csrc.microbench attention --batch 8 --context 640 [--prompt 0]
    python -m oracle_engine_b200.csrc.microbench attention --batch 1 --prompt 2048
    python -m oracle_engine_b200.csrc.microbench attention --batch 8 --context 640 --decode warps
    python -m oracle_engine_b200.csrc.microbench norm --rows 2048 --width 3072
    python -m oracle_engine_b200.csrc.microbench rope --tokens 4096

In the manner of the reference's benchmark/micro_gemm.cpp (:97-128 correctness against a
scalar double-precision product, :130-151 GFLOP/s), for the CUDA kernels of this library.
Timing: the kernel is captured N times in a CUDA graph over operands that rotate through
more memory than the L2 holds, and one replay is timed with CUDA events.  `--once` runs
the kernel a few times without graph or timing (the form to put under a profiler).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
from types import SimpleNamespace

import torch

from ..engine.batch import context_class
from . import ops, ops_tc

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            raw = json.load(open(path))
            return float(raw["hbm_gbs"]), float(raw["bf16_tflops"]), "measured"
        except (KeyError, ValueError, OSError):
            pass
    return 6650.0, 1590.0, "fallback"


def timed(fn, iters, once):
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    if once:
        return None
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(iters):
            fn(i)
    g.replay()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    g.replay()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters * 1e3          # microseconds


def report(name, us, nbytes, flops, err, extra=""):
    hbm, tf, src = peaks()
    if us is None:
        print(f"{name}: ran (not timed); max error {err:.3g} {extra}")
        return
    gbs, tfs = nbytes / us / 1e3, flops / us / 1e6
    print(f"{name}: {us:.1f} us  {gbs:.0f} GB/s ({gbs / hbm:.2f} of {src} HBM)  {tfs:.1f} TFLOP/s "
          f"({tfs / tf:.2f} of {src} bf16 peak)  max error {err:.3g} {extra}")


def run_gemm(a):
    dev = torch.device("cuda:0")
    M, N, K = a.m, a.n, a.k
    copies = max(2, int(400e6 // (N * K * 2)) + 1)
    g = torch.Generator(device="cuda").manual_seed(0)
    ws = [(torch.randn(N, K, device=dev, generator=g) * 0.05).to(torch.bfloat16) for _ in range(copies)]
    x = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
    swiglu, acc = a.out == "swiglu", a.out == "accumulate"
    dtype = torch.float32 if a.out in ("float32", "accumulate") else torch.bfloat16
    out = torch.zeros(M, N // 2 if swiglu else N, device=dev, dtype=dtype)
    with ops_tc.knobs(gemm_schedule=(a.tile, a.stream_k, a.cluster, a.narrow, a.atoms), sm_count=a.sms):
        ops_tc.gemm(out, x, ws[0], accumulate=acc, swiglu=swiglu, kernel=a.kernel)
        ref = x[:64].double() @ ws[0].double().T
        if swiglu:
            ref = ref[:, 0::2] / (1 + torch.exp(-ref[:, 0::2])) * ref[:, 1::2]
        err = ((out[:64].double() - ref).abs().max() / ref.abs().max()).item()
        us = timed(lambda i: ops_tc.gemm(out, x, ws[i % copies], accumulate=acc, swiglu=swiglu, kernel=a.kernel),
                   a.iters, a.once)
    extra = "(relative)"
    if a.sms and us is not None:
        extra += f"  {N * K * 2 / us / 1e3 / a.sms:.1f} GB/s of weights per SM on {a.sms} SMs"
    report(f"gemm M={M} N={N} K={K} out={a.out} kernel={a.kernel}", us, N * K * 2 + M * K * 2 + out.numel() * out.element_size(),
           2.0 * M * N * K, err, extra)
    assert ops_tc.device_error() == 0


def run_attention(a):
    shape = tuple(int(v) for v in a.warps.split("x")) if a.warps else None
    with ops_tc.knobs(decode_splits=a.splits, decode_warps_shape=shape, decode_warps_cluster=a.cluster):
        _run_attention(a)


def _run_attention(a):
    dev = torch.device("cuda:0")
    H, KVH, hd, B = a.heads, a.kv_heads, a.head_dim, a.batch
    qlen = a.prompt if a.prompt else 1
    ctx_len = a.prompt if a.prompt else a.context
    pages = (ctx_len + 63) // 64
    g = torch.Generator(device="cuda").manual_seed(0)
    copies = max(1, int(300e6 // (B * pages * 2 * KVH * 64 * hd * 2)) + 1) if not a.prompt else 1
    caches = [torch.randn(B * pages, 2, KVH, 64, hd, device=dev, generator=g).to(torch.bfloat16) for _ in range(copies)]
    tables = torch.arange(B * pages, dtype=torch.int32, device=dev).reshape(B, pages).contiguous()
    T = B * qlen
    qkv = torch.randn(T, (H + 2 * KVH) * hd, device=dev, generator=g).to(torch.bfloat16)
    out = torch.empty(T, H * hd, device=dev, dtype=torch.bfloat16)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)          # noqa: E731
    ctx = SimpleNamespace(cu_q=i32([b * qlen for b in range(B + 1)]), seq_start=i32([ctx_len - qlen] * B),
                          seq_qlen=i32([qlen] * B), tok_seq=i32([b for b in range(B) for _ in range(qlen)]),
                          n_seqs=B, n_tokens=T, max_qlen=qlen, all_decode=(qlen == 1),
                          context_class=context_class(ctx_len))
    scale = 1 / math.sqrt(hd)
    if a.decode != "split" and not a.prompt:
        # the one-launch decode kernels: rotation, cache write, attention and merge together
        half = hd // 2
        ang = torch.arange(ctx_len, dtype=torch.float64)[:, None] * (10000.0 ** (-torch.arange(half, dtype=torch.float64) / half))[None]
        cos, sin = torch.cos(ang).float().to(dev), torch.sin(ang).float().to(dev)
        fn = ops_tc.attention_decode_warps if a.decode == "warps" else ops_tc.attention_decode_fused
        fn(out, qkv, cos, sin, caches[0], tables, ctx, H, KVH, hd, 0, scale, True)
        torch.cuda.synchronize()
        us = timed(lambda i: fn(out, qkv, cos, sin, caches[i % copies], tables, ctx, H, KVH, hd, 0, scale, True), a.iters, a.once)
        report(f"decode attention ({a.decode}) B={B} context={ctx_len} H={H} KVH={KVH} hd={hd}", us,
               B * ctx_len * 2 * KVH * hd * 2 + 2 * T * H * hd * 2, 4.0 * B * H * hd * ctx_len, float("nan"))
        return
    ops_tc.attention(out, qkv, caches[0], tables, ctx, H, KVH, hd, 0, scale)
    # correctness on the first sequence's last row, head 0
    kk = caches[0][:pages, 0, 0].reshape(-1, hd)[:ctx_len].double()
    vv = caches[0][:pages, 1, 0].reshape(-1, hd)[:ctx_len].double()
    qq = qkv[qlen - 1, :hd].double()
    p = torch.softmax((kk @ qq) * scale, 0)
    err = (out[qlen - 1, :hd].double() - p @ vv).abs().max().item()
    us = timed(lambda i: ops_tc.attention(out, qkv, caches[i % copies], tables, ctx, H, KVH, hd, 0, scale), a.iters, a.once)
    kv_bytes = B * ctx_len * 2 * KVH * hd * 2
    flops = 4.0 * B * H * hd * (qlen * (ctx_len - qlen) + qlen * (qlen + 1) / 2)
    report(f"attention B={B} q_len={qlen} context={ctx_len} H={H} KVH={KVH} hd={hd}", us, kv_bytes + 2 * T * H * hd * 2, flops, err)


def run_norm(a):
    dev = torch.device("cuda:0")
    rows, D = a.rows, a.width
    x = torch.randn(rows, D, device=dev)
    w = torch.rand(D, device=dev) + 0.5
    y = torch.empty(rows, D, device=dev, dtype=torch.bfloat16)
    ops.rmsnorm(y, x, w, 1e-5)
    ref = x.double() / torch.sqrt((x.double() ** 2).mean(-1, keepdim=True) + 1e-5) * w.double()
    err = (y.double() - ref).abs().max().item()
    us = timed(lambda i: ops.rmsnorm(y, x, w, 1e-5), a.iters, a.once)
    report(f"rmsnorm rows={rows} width={D}", us, rows * D * 6, 3.0 * rows * D, err)


def run_rope(a):
    """The rotation of q and k at each token's place and the write of k and v into the paged cache."""
    dev = torch.device("cuda:0")
    T, H, KVH, hd = a.tokens, a.heads, a.kv_heads, a.head_dim
    half = hd // 2
    width = (H + 2 * KVH) * hd
    pages = (T + ops.PAGE - 1) // ops.PAGE
    copies = max(2, (256 << 20) // (T * width * 2) + 1)
    qkvs = [torch.randn(T, width, device=dev).bfloat16() for _ in range(copies)]
    caches = [torch.zeros(pages, 2, KVH, ops.PAGE, hd, device=dev, dtype=torch.bfloat16) for _ in range(copies)]
    tables = torch.arange(pages, device=dev, dtype=torch.int32)[None].contiguous()
    tok_seq = torch.zeros(T, device=dev, dtype=torch.int32)
    tok_pos = torch.arange(T, device=dev, dtype=torch.int32)
    ang = torch.arange(T, dtype=torch.float64)[:, None] * (10000.0 ** (-torch.arange(half, dtype=torch.float64) / half))[None]
    cos, sin = torch.cos(ang).float().to(dev), torch.sin(ang).float().to(dev)
    # correctness: the last token's first query head and first key head
    before = qkvs[0][T - 1].double().clone()
    ops.rope_kv_write(qkvs[0], cos, sin, caches[0], tables, tok_seq, tok_pos, H, KVH, hd, True)
    c, s_ = cos[T - 1].double(), sin[T - 1].double()

    def rot(x):
        return torch.cat([x[:half] * c - x[half:] * s_, x[:half] * s_ + x[half:] * c])
    k_at = caches[0][(T - 1) // ops.PAGE, 0, 0, (T - 1) % ops.PAGE].double()
    err = max((qkvs[0][T - 1, :hd].double() - rot(before[:hd])).abs().max().item(),
              (k_at - rot(before[H * hd:(H + 1) * hd])).abs().max().item())
    us = timed(lambda i: ops.rope_kv_write(qkvs[i % copies], cos, sin, caches[i % copies], tables, tok_seq, tok_pos,
                                           H, KVH, hd, True), a.iters, a.once)
    # reads q, k, v; writes q in place and k, v to the cache
    report(f"rope_kv_write tokens={T} H={H} KVH={KVH} hd={hd}", us, T * (width + H * hd + 2 * KVH * hd) * 2,
           3.0 * T * (H + KVH) * hd, err)


def main(argv=None):
    ap = argparse.ArgumentParser(prog="microbench")
    sub = ap.add_subparsers(dest="what", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--m", type=int, default=8)
    g.add_argument("--n", type=int, default=16384)
    g.add_argument("--k", type=int, default=3072)
    g.add_argument("--out", default="bfloat16", choices=["bfloat16", "float32", "accumulate", "swiglu"])
    g.add_argument("--kernel", default="auto", choices=["auto", "tcgen05", "pair", "skinny"])
    g.add_argument("--tile", type=int, default=0, help="one-SM tcgen05 kernel, many tokens: this tile width (0: by the shape)")
    g.add_argument("--cluster", type=int, default=-1, choices=[-1, 0],
                   help="one-SM tcgen05 kernel, few tokens: 0 adds the K splits up through the workspace, never in a cluster")
    g.add_argument("--narrow", type=int, default=-1, choices=[-1, 0, 1],
                   help="one-SM tcgen05 kernel, up to 128 tokens: 1 narrow tiles without a split, 0 swap-AB with split K")
    g.add_argument("--stream-k", type=int, default=-1, choices=[-1, 0, 1],
                   help="one-SM tcgen05 kernel, many tokens: 1 stream-K wherever a remainder exists, 0 whole tiles, -1 by the shape")
    g.add_argument("--atoms", type=int, default=-1, choices=[-1, 1, 2],
                   help="one-SM tcgen05 kernel, up to 128 tokens: 64-deep swizzle atoms per k-block (-1: by the shape)")
    g.add_argument("--sms", type=int, default=0,
                   help="one-SM tcgen05 kernel: plan the grid for this many SMs (0: the device's); shows what one SM streams")
    at = sub.add_parser("attention")
    at.add_argument("--batch", type=int, default=8)
    at.add_argument("--context", type=int, default=640)
    at.add_argument("--prompt", type=int, default=0, help="tokens per sequence in the step (0: one decoded token)")
    at.add_argument("--heads", type=int, default=24)
    at.add_argument("--kv-heads", type=int, default=8)
    at.add_argument("--head-dim", type=int, default=128)
    at.add_argument("--splits", type=int, default=0, help="split kernel: CTAs per (sequence, KV head) (0: the rule's)")
    at.add_argument("--cluster", type=int, default=0, help="warps kernel: CTAs that share a (sequence, KV head) (0: the rule's)")
    at.add_argument("--warps", default="", help="warps kernel: WARPSxRING, e.g. 1x3 (default: the rule's)")
    at.add_argument("--decode", default="split", choices=["split", "warps", "fused"],
                    help="decode kernel: keys split over CTAs plus a merge (after a separate rotation kernel, not timed "
                         "here), over the warps of one CTA, or the one-warp fused kernel")
    n = sub.add_parser("norm")
    n.add_argument("--rows", type=int, default=2048)
    n.add_argument("--width", type=int, default=3072)
    r = sub.add_parser("rope")
    r.add_argument("--tokens", type=int, default=4096)
    r.add_argument("--heads", type=int, default=24)
    r.add_argument("--kv-heads", type=int, default=8)
    r.add_argument("--head-dim", type=int, default=128)
    for p in (g, at, n, r):
        p.add_argument("--iters", type=int, default=20)
        p.add_argument("--once", action="store_true", help="run without graph or timing (for a profiler)")
    a = ap.parse_args(argv)
    ops.require_cuda()
    {"gemm": run_gemm, "attention": run_attention, "norm": run_norm, "rope": run_rope}[a.what](a)
    return 0


if __name__ == "__main__":
    sys.exit(main())
