"""Micro-benchmarks of single kernels on synthetic inputs: device time with CUDA events and the achieved fraction
of the kernel's own roofline (bytes it must read / time, or flops / time).

    python -m cppvllm_b200.kernel_bench attn_decode  --batch 8 --context 4096
    python -m cppvllm_b200.kernel_bench attn_prefill --tokens 2048
    python -m cppvllm_b200.kernel_bench gemv --batch 8 --rows 4096 --cols 1024
    python -m cppvllm_b200.kernel_bench gemv_fused --form stream_norm --batch 8 --rows 4096 --cols 1024

Inputs are larger than the 126 MB L2 where the shape allows, or the buffers are rotated between iterations so
that no iteration finds its operands in L2.  This is also the small case that profiler captures run on.
"""
from __future__ import annotations

import argparse
import json
import math
import sys

import torch


def _time(fn, iters: int, warmup: int = 3) -> float:
    """Microseconds per call.  The `iters` calls are captured into one CUDA graph and the graph is timed, so the
    host's cost of making a call does not show; a short profiler run (--iters <= 3) launches eagerly instead."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if iters <= 3:
        e0.record()
        for i in range(iters):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters * 1e3
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(iters):
            fn(i)
    graph.replay()
    torch.cuda.synchronize()
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e3


def _paged_inputs(batch, context, q_len, H, KV, hd, page, copies, seed=0):
    d = torch.device("cuda:0")
    g = torch.Generator(device="cuda").manual_seed(seed)
    pages_per_seq = (context + page - 1) // page
    n_pages = batch * pages_per_seq
    caches = [torch.randn(n_pages + 1, 2, KV, page, hd, generator=g, device=d, dtype=torch.float32).to(torch.bfloat16)
              for _ in range(copies)]
    perm = torch.randperm(n_pages, generator=g, device=d).to(torch.int32)
    tables = perm.view(batch, pages_per_seq).contiguous()
    T = batch * q_len
    q = torch.randn(T, H * hd, generator=g, device=d, dtype=torch.float32).to(torch.bfloat16)
    cu = torch.arange(0, T + 1, q_len, dtype=torch.int32, device=d)
    pos = (torch.arange(T, device=d, dtype=torch.int32) % q_len) + (context - q_len)
    return caches, tables, q, cu, pos.contiguous()


def attn_decode(a) -> dict:
    from .csrc import ops
    H, KV, hd, page = a.heads, a.kv_heads, a.head_dim, a.page_size
    kv_bytes = a.batch * a.context * 2 * KV * hd * 2
    copies = 1 if a.warm else max(1, min(8, int(300e6 // kv_bytes) + 1))
    caches, tables, q, cu, pos = _paged_inputs(a.batch, a.context, 1, H, KV, hd, page, copies)
    out = torch.empty_like(q)
    splits = a.splits
    if not splits:                                       # the engine's choice (parts/attention.py: decode_splits)
        splits = 1
        while splits * 2 <= min(16, (a.context + 63) // 64) and a.batch * KV * splits * 2 <= 296:
            splits *= 2
        if splits == 16 and a.batch * KV * 16 > 128:
            splits = 8
    n = ops.attn_decode_scratch_floats(a.batch, KV, hd, splits)
    scratch = torch.empty(max(1, n), dtype=torch.float32, device=q.device)
    scale = 1 / math.sqrt(hd)

    def run(i):
        ops.attn_decode_bf16(out, q, caches[i % copies], tables, cu, pos, a.batch, H, KV, hd, page, scale, splits,
                             scratch if splits > 1 else None)
    us = _time(run, a.iters)
    ops.check_device_errors(q.device)
    return {"kernel": "attn_decode_bf16", "batch": a.batch, "context": a.context, "splits": splits, "us": round(us, 2),
            "GBps": round(kv_bytes / us / 1e3, 1), "bytes": kv_bytes}


def attn_prefill(a) -> dict:
    from .csrc import ops
    H, KV, hd, page = a.heads, a.kv_heads, a.head_dim, a.page_size
    caches, tables, q, cu, pos = _paged_inputs(a.batch, a.tokens + a.cached, a.tokens, H, KV, hd, page, 1)
    out = torch.empty_like(q)
    scale = 1 / math.sqrt(hd)
    if a.impl == "tcgen05":
        tiles = ops.prefill_tiles_tcgen05([a.tokens] * a.batch, H, KV)

        pieces = a.pieces if a.pieces else ops.prefill_pieces_tcgen05(tiles, KV)        # 0: the engine's choice
        scratch = counters = None
        if pieces > 1:
            scratch = torch.empty(ops.attn_prefill_tcgen05_scratch_floats(tiles, KV, hd, pieces), dtype=torch.float32, device=q.device)
            counters = torch.zeros(tiles * KV, dtype=torch.int32, device=q.device)

        def run(i):
            ops.attn_prefill_tcgen05(out, q, caches[0], tables, cu, pos, a.batch, tiles, H, KV, hd, page, scale,
                                     pieces=pieces, min_rounds=a.min_rounds, scratch=scratch, piece_counts=counters)
    else:
        tiles = ops.prefill_tiles([a.tokens] * a.batch, H, KV)

        def run(i):
            ops.attn_prefill_bf16(out, q, caches[0], tables, cu, pos, a.batch, tiles, H, KV, hd, page, scale)
    us = _time(run, a.iters)
    ops.check_device_errors(q.device)
    flops = a.batch * 4 * H * hd * (a.tokens * (a.tokens + 1) // 2 + a.tokens * a.cached)
    return {"kernel": f"attn_prefill ({a.impl})", "batch": a.batch, "tokens": a.tokens, "cached": a.cached, "pieces": pieces if a.impl == "tcgen05" else 1,
            "us": round(us, 2), "TFLOPs": round(flops / us / 1e6, 1), "flops": flops}


def gemv(a) -> dict:
    from .csrc import ops
    d = torch.device("cuda:0")
    copies = 1 if a.warm else max(1, min(64, int(300e6 // (a.rows * a.cols * 2)) + 1))
    ws = [torch.randn(a.rows, a.cols, device=d).to(torch.bfloat16) for _ in range(copies)]
    x = torch.randn(a.batch, a.cols, device=d).to(torch.bfloat16)
    out = torch.empty(a.batch, a.rows, device=d, dtype=torch.bfloat16)

    def run(i):
        ops.linear(x, ws[i % copies], out=out)
    us = _time(run, a.iters)
    nbytes = a.rows * a.cols * 2
    return {"kernel": "linear (library)", "batch": a.batch, "rows": a.rows, "cols": a.cols, "us": round(us, 2),
            "GBps": round(nbytes / us / 1e3, 1)}


def gemv_fused(a) -> dict:
    """The package's own weight-streaming product: plain, with the norm prologue, or with norm and SwiGLU."""
    from .csrc import ops
    d = torch.device("cuda:0")
    copies = 1 if a.warm else max(1, min(64, int(300e6 // (a.rows * a.cols * 2)) + 1))
    ws = [torch.randn(a.rows, a.cols, device=d).to(torch.bfloat16) for _ in range(copies)]
    x = torch.randn(a.batch, a.cols, device=d).to(torch.bfloat16)
    delta = torch.randn(a.batch, a.cols, device=d).to(torch.bfloat16)
    h2 = torch.empty_like(x)
    nw = torch.ones(a.cols, device=d)
    n_out = a.rows // 2 if a.form.endswith("swiglu") else a.rows
    out = torch.empty(a.batch, n_out, device=d, dtype=torch.bfloat16)

    def run(i):
        if a.form == "splitk":
            ops.gemv_splitk_bf16(out, x, ws[i % copies], a.batch)
        elif a.form == "ring":
            ops.gemv_ring_bf16(out, x, ws[i % copies], a.batch)
        elif a.form.startswith("stream"):
            kind = a.form[len("stream"):].lstrip("_")
            if kind == "":
                ops.gemv_stream_bf16(out, x, ws[i % copies], a.batch)
            else:
                ops.gemv_stream_bf16(out, x, ws[i % copies], a.batch, norm_weight=nw, eps=1e-6, delta=delta, resid_out=h2,
                                     swiglu=kind == "swiglu")
        elif a.form == "plain":
            ops.gemv_bf16(out, x, ws[i % copies], a.batch)
        else:
            ops.gemv_bf16(out, x, ws[i % copies], a.batch, norm_weight=nw, eps=1e-6, delta=delta, resid_out=h2,
                          swiglu=a.form == "swiglu")
    us = _time(run, a.iters)
    nbytes = a.rows * a.cols * 2
    return {"kernel": f"gemv_bf16 ({a.form})", "batch": a.batch, "rows": a.rows, "cols": a.cols, "us": round(us, 2),
            "GBps": round(nbytes / us / 1e3, 1)}


def gemm(a) -> dict:
    """Prefill-sized product: the package's tcgen05 kernel (plain or with the SwiGLU epilogue) and the library's."""
    from .csrc import ops
    d = torch.device("cuda:0")
    M, N, K = a.tokens, a.rows, a.cols
    w = (torch.randn(N, K, device=d) * 0.05).to(torch.bfloat16)
    x = torch.randn(M, K, device=d).to(torch.bfloat16)
    swiglu = a.form == "swiglu"
    out = torch.empty(M, N // 2 if swiglu else N, device=d, dtype=torch.bfloat16)
    lib_out = torch.empty(M, N, device=d, dtype=torch.bfloat16)
    act = torch.empty(M, N // 2, device=d, dtype=torch.bfloat16)

    def ours(i):
        ops.gemm_bf16_tcgen05(out, x, w, swiglu=swiglu, tile_n=a.tile_n)

    def library(i):
        ops.linear(x, w, out=lib_out)
        if swiglu:
            ops.swiglu(act, lib_out)
    us, us_lib = _time(ours, a.iters), _time(library, a.iters)
    ops.check_device_errors(d)
    flops = 2.0 * M * N * K
    return {"kernel": f"gemm_bf16_tcgen05 ({a.form})", "M": M, "N": N, "K": K, "us": round(us, 2), "TFLOPs": round(flops / us / 1e6, 1),
            "library_us": round(us_lib, 2), "library_TFLOPs": round(flops / us_lib / 1e6, 1)}


def elementwise(a) -> dict:
    """The memory-bound kernels of a prompt portion of --tokens tokens at the model's widths (--cols hidden, --rows
    intermediate): residual add + RMSNorm, SwiGLU, per-head norm + rotary + cache write.  Inputs stay in L2 between
    calls, as they do in the model, where the product before each of these kernels has just written them."""
    from .csrc import ops
    d = torch.device("cuda:0")
    T, D, I, H, KV, hd, page = a.tokens, a.cols, a.rows, a.heads, a.kv_heads, a.head_dim, a.page_size
    bf = torch.bfloat16
    x, resid, out = (torch.randn(T, D, device=d).to(bf) for _ in range(3))
    w = torch.ones(D, device=d)
    gu, act = torch.randn(T, 2 * I, device=d).to(bf), torch.empty(T, I, device=d, dtype=bf)
    qkv, q = torch.randn(T, (H + 2 * KV) * hd, device=d).to(bf), torch.empty(T, H * hd, device=d, dtype=bf)
    qw = torch.ones(hd, device=d)
    inv = 1.0 / (1e6 ** (torch.arange(0, hd, 2, dtype=torch.float64) / hd))
    ang = torch.arange(T + 8, dtype=torch.float64)[:, None] * inv[None, :]
    cos, sin = ang.cos().float().to(d), ang.sin().float().to(d)
    pos = torch.arange(T, dtype=torch.int32, device=d)
    n_pages = (T + page - 1) // page
    cache = torch.zeros(n_pages, 2, KV, page, hd, device=d, dtype=bf)
    slots = torch.randperm(n_pages * page, device=d)[:T].to(torch.int32)
    res = {"kernel": "elementwise", "tokens": T}
    for name, fn, nbytes in (
            ("add_rmsnorm", lambda i: ops.add_rmsnorm(out, resid, x, w, 1e-6), 4 * T * D * 2),
            ("swiglu", lambda i: ops.swiglu(act, gu), 3 * T * I * 2),
            ("qk_norm_rope_kv", lambda i: ops.qk_norm_rope_kv(q, qkv, qw, qw, cos, sin, pos, slots, cache, H, KV, hd, page, 1e-6),
             2 * T * (H + 2 * KV) * hd * 2)):
        us = _time(fn, a.iters)
        res[name] = {"us": round(us, 2), "GBps": round(nbytes / us / 1e3, 1)}
    ops.check_device_errors(d)
    return res


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="kernel_bench")
    p.add_argument("kernel", choices=["attn_decode", "attn_prefill", "gemv", "gemv_fused", "gemm", "elementwise"])
    p.add_argument("--tile-n", type=int, default=0)
    p.add_argument("--impl", default="tcgen05", choices=["tcgen05", "mma"])
    p.add_argument("--form", default="plain", choices=["plain", "norm", "swiglu", "splitk", "ring", "stream", "stream_norm", "stream_swiglu"])
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--context", type=int, default=4096)
    p.add_argument("--tokens", type=int, default=2048)
    p.add_argument("--cached", type=int, default=0)
    p.add_argument("--heads", type=int, default=16)
    p.add_argument("--kv-heads", type=int, default=8)
    p.add_argument("--head-dim", type=int, default=128)
    p.add_argument("--page-size", type=int, default=32)
    p.add_argument("--splits", type=int, default=0)
    p.add_argument("--pieces", type=int, default=0, help="attn_prefill: blocks per long query block (0: the engine's choice)")
    p.add_argument("--min-rounds", type=int, default=8, help="attn_prefill: the fewest key tiles of a piece")
    p.add_argument("--rows", type=int, default=4096)
    p.add_argument("--cols", type=int, default=1024)
    p.add_argument("--iters", type=int, default=20)
    p.add_argument("--warm", action="store_true", help="one weight buffer (gemv) or one cache (attn_decode), so that it stays in L2 where it fits")
    a = p.parse_args(argv)
    if a.kernel == "attn_prefill" and a.batch == 8 and "--batch" not in (argv or sys.argv):
        a.batch = 1
    res = {"attn_decode": attn_decode, "attn_prefill": attn_prefill, "gemv": gemv, "gemv_fused": gemv_fused, "gemm": gemm,
           "elementwise": elementwise}[a.kernel](a)
    print(json.dumps(res))
    return 0


if __name__ == "__main__":
    sys.exit(main())
