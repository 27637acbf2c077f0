"""Times one kernel of the library in isolation with CUDA events, on inputs larger than L2
where that matters, and prints what it achieved against the roofline that bounds it.

    python -m hfee_b200.kernels.microbench gemm_tcgen05 --m 2048 --n 16384 --k 2048 [--epilogue swiglu]
    python -m hfee_b200.kernels.microbench gemm_pair    --m 2048 --n 16384 --k 2048 --epilogue swiglu
    python -m hfee_b200.kernels.microbench gemm_stream  --m 8 --n 16384 --k 2048 [--epilogue swiglu]
    python -m hfee_b200.kernels.microbench gemm_ring    --m 8 --n 2048 --k 8192 --epilogue accum
    python -m hfee_b200.kernels.microbench gemm_skinny  --m 64 --n 2048 --k 8192 --epilogue accum
    python -m hfee_b200.kernels.microbench attention_decode  --batch 8 --context 2048 --heads 32 --kv-heads 8 --head-dim 64
    python -m hfee_b200.kernels.microbench attention_prefill --tokens 2048 --heads 32 --kv-heads 8 --head-dim 64

``--iters`` timed launches follow ``--warmup`` untimed ones; ``--rotate`` distinct weight
buffers are cycled so that a weight-streaming kernel never finds its weights in L2.  The
same command line under ``ncu`` gives the counters summarised in ``profiles/``.
"""
from __future__ import annotations

import argparse
import json
import math
import sys

import torch

from . import ops

DEV = "cuda:0"
EPI = {"store": ops.EPI_STORE, "accum": ops.EPI_ACCUM, "swiglu": ops.EPI_SWIGLU}


GRAPH = False


def _time(fn, warmup: int, iters: int) -> float:
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    if GRAPH:          # device time without host launch overhead: the timed launches replay from a CUDA graph
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(iters):
                fn(warmup + i)
        g.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / iters * 1e-3
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(iters):
        fn(warmup + i)
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters * 1e-3


def _gemm(args, kind: str) -> dict:
    m, n, k = args.m, args.n, args.k
    epi = EPI[args.epilogue]
    a = (torch.randn(m, k, device=DEV) * 0.5).to(torch.bfloat16)
    ws = [(torch.randn(n, k, device=DEV) * 0.05).to(torch.bfloat16) for _ in range(args.rotate)]
    if epi == ops.EPI_ACCUM:
        out = torch.zeros(m, n, dtype=torch.float32, device=DEV)
    elif epi == ops.EPI_SWIGLU:
        out = torch.empty(m, n // 2, dtype=torch.bfloat16, device=DEV)
    else:
        out = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    if kind == "gemm_tcgen05":
        fn = lambda i: ops.gemm_tcgen05(a, ws[i % len(ws)], out, epi, args.block_n)
    elif kind == "gemm_skinny":
        fn = lambda i: ops.gemm_skinny(a, ws[i % len(ws)], out, epi)
    elif kind == "gemm_pair":
        fn = lambda i: ops.gemm_tcgen05_pair(a, ws[i % len(ws)], out, epi)
    elif kind == "gemm_ring":
        fn = lambda i: ops.gemm_ring(a, ws[i % len(ws)], out, epi)
    else:
        fn = lambda i: ops.gemm_stream(a, ws[i % len(ws)], out, epi)
    sec = _time(fn, args.warmup, args.iters)
    ops.check_status()
    flops = 2.0 * m * n * k
    bytes_ = 2.0 * (n * k + m * k) + out.numel() * out.element_size()
    return {"kernel": kind, "m": m, "n": n, "k": k, "epilogue": args.epilogue, "us": round(sec * 1e6, 2),
            "tflops": round(flops / sec / 1e12, 1), "gbs": round(bytes_ / sec / 1e9, 1)}


class _Batch:
    pass


def _attention(args, decode: bool) -> dict:
    heads, kv, hd, page = args.heads, args.kv_heads, args.head_dim, args.page_size
    if decode:
        before, new = [args.context] * args.batch, [1] * args.batch
    else:
        before, new = [args.context_before], [args.tokens]
    r = len(before)
    total = [b + n for b, n in zip(before, new)]
    max_pages = max(-(-t // page) for t in total)
    n_pages = r * max_pages
    table = torch.randperm(n_pages).reshape(r, max_pages).to(torch.int32).to(DEV)
    kp = torch.randn(n_pages, kv, page, hd, device=DEV).to(torch.bfloat16)
    vp = torch.randn(n_pages, kv, page, hd, device=DEV).to(torch.bfloat16)
    n = sum(new)
    q = torch.randn(n, heads * hd, device=DEV).to(torch.bfloat16)
    out = torch.empty_like(q)
    b = _Batch()
    cu = [0]
    for x in new:
        cu.append(cu[-1] + x)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    b.cu_tokens, b.slots, b.context_before = i32(cu), i32(list(range(r))), i32(before)
    b.n, b.r, b.max_new, b.max_context = n, r, max(new), max(total)
    b.planning_context = b.max_context
    b.attention_splits = args.splits or None
    pos = i32([p for s, c in zip(before, new) for p in range(s, s + c)])
    sot = i32([i for i, c in enumerate(new) for _ in range(c)])
    scratch = torch.empty(r * heads * ops.MAX_SPLITS * (hd + 2), dtype=torch.float32, device=DEV) if decode else None
    scale = 1.0 / math.sqrt(hd)
    fn = lambda i: ops.paged_attention(q, kp, vp, table, page, pos, sot, out, heads, kv, hd, scale, 0, step=b, scratch=scratch)
    sec = _time(fn, args.warmup, args.iters)
    kv_bytes = sum(total) * kv * hd * 2 * 2
    flops = sum(4.0 * heads * hd * (c * s + c * (c + 1) / 2) for s, c in zip(before, new))
    return {"kernel": "attention_decode" if decode else "attention_prefill", "heads": heads, "kv_heads": kv,
            "head_dim": hd, "requests": r, "context": max(total), "us": round(sec * 1e6, 2),
            "kv_gbs": round(kv_bytes / sec / 1e9, 1), "tflops": round(flops / sec / 1e12, 1)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("kernel", choices=["gemm_tcgen05", "gemm_stream", "gemm_skinny", "gemm_ring", "gemm_pair", "attention_decode", "attention_prefill"])
    ap.add_argument("--m", type=int, default=2048)
    ap.add_argument("--n", type=int, default=16384)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--epilogue", default="store", choices=list(EPI))
    ap.add_argument("--block-n", type=int, default=None)
    ap.add_argument("--rotate", type=int, default=4, help="distinct weight buffers cycled between launches")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--context-before", type=int, default=0)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=64)
    ap.add_argument("--page-size", type=int, default=64)
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--tc-attention", action="store_true", help="attention_prefill: the tcgen05 kernel (the default)")
    ap.add_argument("--no-tc-attention", action="store_true", help="attention_prefill: the mma.sync kernel")
    ap.add_argument("--graph", action="store_true", help="replay the timed launches from a CUDA graph (no host launch cost)")
    args = ap.parse_args(argv)
    global GRAPH
    GRAPH = args.graph
    ops.USE_TC_ATTENTION = args.tc_attention or not args.no_tc_attention
    torch.manual_seed(0)
    if args.kernel.startswith("gemm"):
        res = _gemm(args, args.kernel)
    else:
        res = _attention(args, args.kernel == "attention_decode")
    print(json.dumps(res))
    return 0


if __name__ == "__main__":
    sys.exit(main())
