"""Python faces of the CUDA launchers: argument checks, pointer passing, status codes turned into errors.

Every function works on CUDA tensors only and launches on the current stream of PyTorch, so the launches
are ordered with PyTorch's own work and are captured by ``torch.cuda.graph``.  There is no CPU path: a
tensor that is not on a CUDA device, or a missing compiler, raises.
"""
from __future__ import annotations

import ctypes
import math
import os
import sys
from ctypes import c_int, c_int64, c_float, c_void_p
from typing import Dict, Optional

import torch

from .build import load_library

_ERRORS = {
    -1: "element type must be float32 or bfloat16",
    -2: "a size is zero, negative or beyond what the kernel takes",
    -3: "a pointer or a row length breaks the kernel's alignment rule",
    -4: "sizes are inconsistent with one another",
    -5: "this specialised kernel does not cover the configuration",
    -6: "scratch memory is missing or too small",
}

DEVICE_ERRORS = {
    1: "a token id lies outside the embedding table",
    2: "a cache slot lies outside the page pool",
    3: "a position lies outside the rotary tables (beyond max_position_embeddings)",
    4: "attention needed a key whose page is missing from the block table",
    5: "a bounded wait in a kernel ran out",
    6: "a kernel found its shared memory misaligned for swizzled tiles",
}


class KernelError(RuntimeError):
    pass


LAUNCHES = 0      # kernels of this package launched (or recorded into a graph being captured) so far


def launches() -> int:
    return LAUNCHES


def _check(status: int, what: str, kernels: int = 1) -> None:
    global LAUNCHES
    if status == 0:
        LAUNCHES += kernels
        return
    if status < 0:
        raise KernelError(f"{what}: refused: {_ERRORS.get(status, f'code {status}')}")
    raise KernelError(f"{what}: CUDA launch failed with cudaError {status}")


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return 0
    if dt == torch.bfloat16:
        return 1
    raise KernelError(f"element type must be float32 or bfloat16, got {dt}")


def _cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("the kernels run on CUDA tensors only; got a tensor on " + str(t.device))


def _contig(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_contiguous():
            raise KernelError("kernel arguments must be contiguous")


def _ptr(t: Optional[torch.Tensor]):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


_device_index = None


def _stream():
    """The current CUDA stream's handle.  Asked of torch's C layer directly: `torch.cuda.current_stream()` builds a
    Python object at every call and costs about 15 us, which a step of a few hundred launches feels."""
    global _device_index
    if _device_index is None:
        _device_index = torch.cuda.current_device()
    return c_void_p(torch._C._cuda_getCurrentRawStream(_device_index))


_core = None


def core():
    global _core
    if _core is None:
        lib = load_library("core")
        for name in ("cvb_embed", "cvb_rmsnorm", "cvb_add_rmsnorm", "cvb_add", "cvb_swiglu", "cvb_gather_rows",
                     "cvb_qk_norm_rope_kv", "cvb_paged_attention_general", "cvb_sample", "cvb_sample_chunked",
                     "cvb_feed_tokens"):
            getattr(lib, name).restype = c_int
        _core = lib
    return _core


_err_flags = {}


def error_flag(device) -> torch.Tensor:
    """One int32 per device that kernels set when they meet an index they refuse to follow."""
    device = torch.device(device)
    key = device.index if device.index is not None else torch.cuda.current_device()
    f = _err_flags.get(key)
    if f is None:
        f = torch.zeros(1, dtype=torch.int32, device=device)
        _err_flags[key] = f
    return f


def check_device_errors(device) -> None:
    """Read the device error flag (synchronises) and raise if a kernel recorded a refused index."""
    f = error_flag(device)
    v = int(f.item())
    if v != 0:
        f.zero_()
        raise KernelError(f"a kernel reported: {DEVICE_ERRORS.get(v, f'error {v}')}")


def selftest_wait_runs_out(limit_cycles: int = 2_000_000) -> int:
    """Launches a block that waits on a barrier nothing arrives on, with a limit of `limit_cycles` clock cycles (about a
    millisecond by default).  Returns 1 if the wait gave up and the kernel ran to its end; the device error word then
    holds 5 (check_device_errors raises "a bounded wait in a kernel ran out")."""
    lib = core()
    lib.cvb_selftest_wait_runs_out.restype = c_int
    dev = torch.device("cuda", torch.cuda.current_device())
    finished = torch.zeros(1, dtype=torch.int32, device=dev)
    _check(lib.cvb_selftest_wait_runs_out(_ptr(error_flag(dev)), _ptr(finished), ctypes.c_longlong(limit_cycles), _stream()),
           "selftest_wait_runs_out")
    return int(finished.item())


# ---- elementwise ------------------------------------------------------------------------------------------

def embed(out: torch.Tensor, table: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
    _cuda(out, table, tokens); _contig(out, table, tokens)
    T, D = out.shape
    if tokens.dtype != torch.int32 or tokens.numel() != T or table.shape[1] != D or table.dtype != out.dtype:
        raise KernelError("embed: tokens must be int32 [T]; table [V, D] and out [T, D] of one element type")
    _check(core().cvb_embed(_ptr(out), _ptr(table), _ptr(tokens), c_int(T), c_int(D), c_int(table.shape[0]),
                            c_int(dtype_code(out.dtype)), _ptr(error_flag(out.device)), _stream()), "embed")
    return out


def rmsnorm(out: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    _cuda(out, x, weight); _contig(out, x, weight)
    T, D = x.shape
    if weight.dtype != torch.float32 or weight.numel() != D or out.shape != x.shape or out.dtype != x.dtype:
        raise KernelError("rmsnorm: weight must be float32 [D]; out like x")
    _check(core().cvb_rmsnorm(_ptr(out), _ptr(x), _ptr(weight), c_int(T), c_int(D), c_float(eps),
                              c_int(dtype_code(x.dtype)), _stream()), "rmsnorm")
    return out


def add_rmsnorm(out: torch.Tensor, resid: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """resid <- T(resid + x) in place; out <- rmsnorm(resid)."""
    _cuda(out, resid, x, weight); _contig(out, resid, x, weight)
    T, D = x.shape
    if (weight.dtype != torch.float32 or weight.numel() != D or out.shape != x.shape or resid.shape != x.shape
            or out.dtype != x.dtype or resid.dtype != x.dtype):
        raise KernelError("add_rmsnorm: weight must be float32 [D]; out, resid like x")
    _check(core().cvb_add_rmsnorm(_ptr(out), _ptr(resid), _ptr(x), _ptr(weight), c_int(T), c_int(D), c_float(eps),
                                  c_int(dtype_code(x.dtype)), _stream()), "add_rmsnorm")
    return out


def add_(resid: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    _cuda(resid, x); _contig(resid, x)
    if resid.shape != x.shape or resid.dtype != x.dtype:
        raise KernelError("add_: operands must match")
    _check(core().cvb_add(_ptr(resid), _ptr(x), c_int64(x.numel()), c_int(dtype_code(x.dtype)), _stream()), "add_")
    return resid


def swiglu(out: torch.Tensor, gate_up: torch.Tensor) -> torch.Tensor:
    _cuda(out, gate_up); _contig(out, gate_up)
    T, I = out.shape
    if gate_up.shape != (T, 2 * I) or gate_up.dtype != out.dtype:
        raise KernelError("swiglu: gate_up must be [T, 2I] for out [T, I]")
    _check(core().cvb_swiglu(_ptr(out), _ptr(gate_up), c_int(T), c_int(I), c_int(dtype_code(out.dtype)), _stream()),
           "swiglu")
    return out


def gather_rows(out: torch.Tensor, src: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    _cuda(out, src, rows); _contig(out, src, rows)
    R, D = out.shape
    if rows.dtype != torch.int32 or rows.numel() < R or src.shape[1] != D or src.dtype != out.dtype:
        raise KernelError("gather_rows: rows must be int32 [R]; src [N, D], out [R, D] of one element type")
    _check(core().cvb_gather_rows(_ptr(out), _ptr(src), _ptr(rows), c_int(R), c_int(D), c_int(src.shape[0]),
                                  c_int(dtype_code(out.dtype)), _stream()), "gather_rows")
    return out


# ---- projection epilogue: per-head norm, rotary, cache write --------------------------------------------------

def qk_norm_rope_kv(q_out: torch.Tensor, qkv: torch.Tensor, q_weight: Optional[torch.Tensor],
                    k_weight: Optional[torch.Tensor], cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                    positions: Optional[torch.Tensor], slots: Optional[torch.Tensor],
                    cache: Optional[torch.Tensor], num_heads: int, num_kv_heads: int, head_dim: int,
                    page_size: int, eps: float, rotary_dim: Optional[int] = None, interleaved: bool = False) -> torch.Tensor:
    """q_out[T, H, hd] <- rotate(norm(q)); k -> rotate(norm(k)) and v into `cache` [pages, 2, KV, page, hd]."""
    _cuda(q_out, qkv, q_weight, k_weight, cos, sin, positions, slots, cache)
    _contig(q_out, qkv, q_weight, k_weight, cos, sin, positions, slots, cache)
    T = qkv.shape[0]
    H, KV, hd = num_heads, num_kv_heads, head_dim
    if qkv.shape[1] != (H + 2 * KV) * hd or q_out.numel() != T * H * hd or q_out.dtype != qkv.dtype:
        raise KernelError("qk_norm_rope_kv: qkv must be [T, (H + 2 KV) hd] and q_out [T, H, hd]")
    for w in (q_weight, k_weight):
        if w is not None and (w.dtype != torch.float32 or w.numel() != hd):
            raise KernelError("qk_norm_rope_kv: per-head norm weights must be float32 [hd]")
    rot = head_dim if rotary_dim is None else int(rotary_dim)
    max_pos = 0
    if cos is not None:
        if cos.dtype != torch.float32 or sin is None or sin.shape != cos.shape or cos.shape[1] != rot // 2:
            raise KernelError("qk_norm_rope_kv: cos/sin tables must be float32 [max_pos, rotary_dim / 2]")
        max_pos = cos.shape[0]
        if positions is None or positions.dtype != torch.int32 or positions.numel() < T:
            raise KernelError("qk_norm_rope_kv: positions must be int32 [T]")
    if slots is not None and (slots.dtype != torch.int32 or slots.numel() < T):
        raise KernelError("qk_norm_rope_kv: slots must be int32 [T]")
    cache_elems = 0
    if cache is not None:
        if cache.dtype != qkv.dtype:
            raise KernelError("qk_norm_rope_kv: cache pages must have the activations' element type")
        cache_elems = cache.numel()
    _check(core().cvb_qk_norm_rope_kv(
        _ptr(q_out), _ptr(qkv), _ptr(q_weight), _ptr(k_weight), _ptr(cos), _ptr(sin), _ptr(positions), _ptr(slots),
        _ptr(cache), c_int(T), c_int(H), c_int(KV), c_int(hd), c_int(rot), c_int(1 if interleaved else 0),
        c_int(page_size), c_int(max_pos), c_float(eps), c_int64(cache_elems), c_int(dtype_code(qkv.dtype)),
        _ptr(error_flag(qkv.device)), _stream()), "qk_norm_rope_kv")
    return q_out


# ---- attention ---------------------------------------------------------------------------------------------

def paged_attention_general(out: torch.Tensor, q: torch.Tensor, cache: torch.Tensor, block_tables: torch.Tensor,
                            seq_of_token: torch.Tensor, positions: torch.Tensor, num_heads: int, num_kv_heads: int,
                            head_dim: int, page_size: int, scale: float, window: int = 0,
                            num_tokens: Optional[int] = None) -> torch.Tensor:
    _cuda(out, q, cache, block_tables, seq_of_token, positions)
    _contig(out, q, cache, block_tables, seq_of_token, positions)
    T = q.shape[0] if num_tokens is None else num_tokens
    if q.dtype != cache.dtype or out.dtype != q.dtype:
        raise KernelError("paged_attention: q, out and the cache pages must share one element type")
    if block_tables.dtype != torch.int32 or block_tables.dim() != 2:
        raise KernelError("paged_attention: block_tables must be int32 [S, W]")
    if seq_of_token.dtype != torch.int32 or positions.dtype != torch.int32:
        raise KernelError("paged_attention: seq_of_token and positions must be int32")
    if num_heads % num_kv_heads:
        raise KernelError(f"paged_attention: {num_heads} query heads are not a multiple of {num_kv_heads} kv heads")
    page_elems = 2 * num_kv_heads * page_size * head_dim
    num_pages = cache.numel() // page_elems
    _check(core().cvb_paged_attention_general(
        _ptr(out), _ptr(q), _ptr(cache), _ptr(block_tables), c_int(block_tables.shape[1]), _ptr(seq_of_token),
        _ptr(positions), c_int(T), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(page_size),
        c_int(window), c_float(scale), c_int(num_pages), c_int(dtype_code(q.dtype)),
        _ptr(error_flag(q.device)), _stream()), "paged_attention_general")
    return out


_attn = None


def attn_bf16():
    global _attn
    if _attn is None:
        lib = load_library("attn_bf16")
        lib.cvb_attn_prefill_bf16.restype = c_int
        lib.cvb_attn_decode_bf16.restype = c_int
        lib.cvb_attn_decode_scratch_floats.restype = c_int64
        _attn = lib
    return _attn


def fast_attention_supported(dtype: torch.dtype, num_heads: int, num_kv_heads: int, head_dim: int,
                             page_size: int = 16) -> bool:
    """The tensor-core kernels cover bf16, head sizes 64 and 128, up to 16 query heads per kv head and pages of
    16, 32, 64, ... tokens (a power of two)."""
    return (dtype == torch.bfloat16 and head_dim in (64, 128) and num_heads % num_kv_heads == 0
            and num_heads // num_kv_heads <= 16 and page_size >= 16 and page_size & (page_size - 1) == 0)


def prefill_tiles(q_lens, num_heads: int, num_kv_heads: int, skip_single: bool = True) -> int:
    """Tiles the prefill kernel's grid needs: per request ceil(tokens / (64 / group))."""
    tpt = 64 // (num_heads // num_kv_heads)
    return sum((n + tpt - 1) // tpt for n in q_lens if not (skip_single and n == 1))


def _attn_common_checks(out, q, cache, block_tables, cu_seqlens, positions):
    _cuda(out, q, cache, block_tables, cu_seqlens, positions)
    _contig(out, q, cache, block_tables, cu_seqlens, positions)
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("tensor-core attention takes bf16 queries, pages and output")
    if block_tables.dtype != torch.int32 or block_tables.dim() != 2 or cu_seqlens.dtype != torch.int32 \
            or positions.dtype != torch.int32:
        raise KernelError("tensor-core attention: block_tables [S, W], cu_seqlens and positions must be int32")


def attn_prefill_bf16(out, q, cache, block_tables, cu_seqlens, positions, num_seqs: int, num_tiles: int,
                      num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, scale: float,
                      window: int = 0, skip_single: bool = True):
    _attn_common_checks(out, q, cache, block_tables, cu_seqlens, positions)
    num_pages = cache.numel() // (2 * num_kv_heads * page_size * head_dim)
    _check(attn_bf16().cvb_attn_prefill_bf16(
        _ptr(out), _ptr(q), _ptr(cache), _ptr(block_tables), c_int(block_tables.shape[1]), _ptr(cu_seqlens),
        _ptr(positions), c_int(num_seqs), c_int(num_tiles), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim),
        c_int(page_size), c_int(window), c_float(scale), c_int(num_pages), c_int(1 if skip_single else 0),
        _ptr(error_flag(q.device)), _stream()), "attn_prefill_bf16")
    return out


_attn_tc = None


def prefill_tiles_tcgen05(q_lens, num_heads: int, num_kv_heads: int, skip_single: bool = True) -> int:
    """Blocks the tcgen05 prefill kernel's grid needs: per request ceil(tokens / (2 * (128 // group)))."""
    tpt = (128 // (num_heads // num_kv_heads)) * 2
    return sum((n + tpt - 1) // tpt for n in q_lens if not (skip_single and n == 1))


def _attn_tc_lib():
    global _attn_tc
    if _attn_tc is None:
        lib = load_library("attn_tcgen05")
        lib.cvb_attn_prefill_tcgen05.restype = c_int
        lib.cvb_attn_prefill_tcgen05_scratch_floats.restype = c_int64
        _attn_tc = lib
    return _attn_tc


# The tcgen05 prefill kernel shares the key tiles of a long query block out among several blocks when its grid leaves
# most SMs idle: a portion of 512 tokens behind 8,192 cached ones is 32 blocks (8 kv heads) of 68 key tiles each, 128 us
# as they are and 52 us in four pieces.  Pieces are taken only while all blocks can run at once (a second wave costs
# what the cut saves), and a piece has at least PREFILL_MIN_ROUNDS tiles: what a block costs outside its tiles, and
# adding the shares up, is worth about six tiles.
PREFILL_SMS = 148
PREFILL_MAX_PIECES = 8
PREFILL_MIN_ROUNDS = 8


def prefill_pieces_tcgen05(num_tiles: int, num_kv_heads: int, max_kv_len: int = 1 << 30) -> int:
    """Into how many pieces the kernel may cut a query block's keys; 1 if no request of the step is long enough for two
    pieces (the kernel that adds the shares up is then not launched)."""
    if max_kv_len < 2 * PREFILL_MIN_ROUNDS * 128:
        return 1
    blocks = max(1, num_tiles * num_kv_heads)
    return max(1, min(PREFILL_MAX_PIECES, PREFILL_SMS // blocks))


def attn_prefill_tcgen05_scratch_floats(num_tiles: int, num_kv_heads: int, head_dim: int, pieces: int) -> int:
    return int(_attn_tc_lib().cvb_attn_prefill_tcgen05_scratch_floats(c_int(num_tiles), c_int(num_kv_heads), c_int(head_dim),
                                                                      c_int(pieces)))


def attn_prefill_tcgen05(out, q, cache, block_tables, cu_seqlens, positions, num_seqs: int, num_tiles: int,
                         num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, scale: float,
                         window: int = 0, skip_single: bool = True, pieces: int = 1, min_rounds: int = PREFILL_MIN_ROUNDS,
                         scratch=None, piece_counts=None):
    """Flash attention of prompt portions on the tcgen05 tensor cores (same contract as attn_prefill_bf16).
    ``pieces`` > 1: a query block with at least 2 * min_rounds key tiles is worked on by up to ``pieces`` blocks;
    ``scratch`` (float32, attn_prefill_tcgen05_scratch_floats elements) and ``piece_counts`` (int32, num_tiles * kv heads)
    are then required, and a second kernel adds the pieces' shares up."""
    lib = _attn_tc_lib()
    _attn_common_checks(out, q, cache, block_tables, cu_seqlens, positions)
    num_pages = cache.numel() // (2 * num_kv_heads * page_size * head_dim)
    if pieces > 1:
        if scratch is None or piece_counts is None:
            raise ValueError("attn_prefill_tcgen05 with pieces > 1 needs scratch and piece_counts")
        if scratch.dtype != torch.float32 or piece_counts.dtype != torch.int32 or piece_counts.numel() < num_tiles * num_kv_heads:
            raise ValueError("attn_prefill_tcgen05: scratch must be float32 and piece_counts int32 with one entry per "
                             "(query block, kv head)")
    _check(lib.cvb_attn_prefill_tcgen05(
        _ptr(out), _ptr(q), _ptr(cache), _ptr(block_tables), c_int(block_tables.shape[1]), _ptr(cu_seqlens),
        _ptr(positions), c_int(num_seqs), c_int(num_tiles), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim),
        c_int(page_size), c_int(window), c_float(scale), c_int(num_pages), c_int(1 if skip_single else 0),
        c_int(pieces), c_int(min_rounds), _ptr(scratch), c_int64(scratch.numel() if scratch is not None else 0), _ptr(piece_counts),
        _ptr(error_flag(q.device)), _stream()), "attn_prefill_tcgen05", kernels=2 if pieces > 1 else 1)
    return out


def attn_decode_scratch_floats(num_seqs: int, num_kv_heads: int, head_dim: int, splits: int) -> int:
    return int(attn_bf16().cvb_attn_decode_scratch_floats(c_int(num_seqs), c_int(num_kv_heads), c_int(head_dim), c_int(splits)))


def attn_decode_bf16(out, q, cache, block_tables, cu_seqlens, positions, num_seqs: int, num_heads: int,
                     num_kv_heads: int, head_dim: int, page_size: int, scale: float, splits: int,
                     scratch: Optional[torch.Tensor], window: int = 0, cluster_merge: bool = True):
    """Split-KV attention of single decoded tokens.  With `cluster_merge` (and up to 16 splits) the splits of a request
    and kv head run as one thread-block cluster and merge their parts through distributed shared memory; otherwise the
    parts go through `scratch` and a second kernel merges them."""
    _attn_common_checks(out, q, cache, block_tables, cu_seqlens, positions)
    if scratch is not None and (scratch.dtype != torch.float32 or not scratch.is_cuda or not scratch.is_contiguous()):
        raise KernelError("attn_decode_bf16: scratch must be a contiguous float32 CUDA tensor")
    num_pages = cache.numel() // (2 * num_kv_heads * page_size * head_dim)
    _check(attn_bf16().cvb_attn_decode_bf16(
        _ptr(out), _ptr(q), _ptr(cache), _ptr(block_tables), c_int(block_tables.shape[1]), _ptr(cu_seqlens),
        _ptr(positions), c_int(num_seqs), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(page_size),
        c_int(window), c_float(scale), c_int(num_pages), c_int(splits), _ptr(scratch),
        c_int64(scratch.numel() if scratch is not None else 0), c_int(1 if cluster_merge else 0),
        _ptr(error_flag(q.device)), _stream()), "attn_decode_bf16",
        kernels=2 if splits > 1 and not (cluster_merge and splits <= 16) else 1)
    return out


DECODE_CLUSTER_SPLITS = 16      # up to this many splits merge inside a thread-block cluster and need no scratch


def attn_decode_fused_bf16(out, qkv, cache, block_tables, cu_seqlens, positions, slots, num_seqs: int, num_heads: int,
                           num_kv_heads: int, head_dim: int, page_size: int, scale: float, splits: int,
                           scratch: Optional[torch.Tensor], q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
                           qk_eps: float, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], window: int = 0):
    """Attention of single decoded tokens from the projection's raw output qkv [T, (H + 2 KV) hd]: per-head norm and
    rotation of queries and of the new key, the cache write of the new key and value, and the attention, one kernel."""
    _attn_common_checks(out, qkv, cache, block_tables, cu_seqlens, positions)
    _cuda(slots, q_weight, k_weight, cos, sin, scratch)
    _contig(slots, q_weight, k_weight, cos, sin, scratch)
    T = qkv.shape[0]
    if T != num_seqs:
        raise KernelError("attn_decode_fused_bf16: every request brings exactly one token (qkv has one row per request)")
    if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim or out.shape != (T, num_heads * head_dim):
        raise KernelError("attn_decode_fused_bf16: qkv must be [T, (H + 2 KV) hd] and out [T, H hd]")
    if slots.dtype != torch.int32 or slots.numel() < T:
        raise KernelError("attn_decode_fused_bf16: slots must be int32 [T]")
    for w in (q_weight, k_weight):
        if w is not None and (w.dtype != torch.float32 or w.numel() != head_dim):
            raise KernelError("attn_decode_fused_bf16: norm weights must be float32 [head_dim]")
    max_pos = 0
    if cos is not None:
        if sin is None or cos.dtype != torch.float32 or sin.dtype != torch.float32 or cos.shape != sin.shape \
                or cos.dim() != 2 or cos.shape[1] != head_dim // 2:
            raise KernelError("attn_decode_fused_bf16: cos and sin must be float32 [max_pos, head_dim / 2]")
        max_pos = cos.shape[0]
    if scratch is not None and scratch.dtype != torch.float32:
        raise KernelError("attn_decode_fused_bf16: scratch must be float32")
    num_pages = cache.numel() // (2 * num_kv_heads * page_size * head_dim)
    lib = attn_bf16()
    lib.cvb_attn_decode_fused_bf16.restype = c_int
    _check(lib.cvb_attn_decode_fused_bf16(
        _ptr(out), _ptr(qkv), _ptr(cache), _ptr(block_tables), c_int(block_tables.shape[1]), _ptr(cu_seqlens),
        _ptr(positions), _ptr(slots), c_int(num_seqs), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim),
        c_int(page_size), c_int(window), c_float(scale), c_int(num_pages), c_int(splits), _ptr(scratch),
        c_int64(scratch.numel() if scratch is not None else 0), _ptr(q_weight), _ptr(k_weight), c_float(qk_eps),
        _ptr(cos), _ptr(sin), c_int(max_pos), _ptr(error_flag(qkv.device)), _stream()), "attn_decode_fused_bf16",
        kernels=2 if splits > 16 else 1)
    return out


_gemv = None

SPLITK_MIN_BYTES = 16 << 20
GEMV_MAX_ROWS = 16           # the weight-streaming product: one or two groups of eight activation rows
SPLITK_MAX_ROWS = 8          # its split-K form: one group


def gemv_supported(x_dtype: torch.dtype, weight: torch.Tensor, rows: int) -> bool:
    """The weight-streaming product covers bf16 operands, up to 16 rows, and inner sizes that are multiples of 8 and whose
    staged rows (8 or 16 of them) fit into shared memory.  More than 8 rows against a large weight are left to the
    library: the split-K form takes 8 rows, and the plain form is slower than the library there."""
    staged = 8 if rows <= 8 else 16
    return (x_dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and 0 < rows <= GEMV_MAX_ROWS
            and weight.shape[1] % 8 == 0 and weight.shape[1] * staged * 2 + 32 * 1024 <= 200 * 1024
            and (rows <= 8 or weight.numel() * 2 < SPLITK_MIN_BYTES))


def gemv_bf16(out: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, rows: int, norm_weight: Optional[torch.Tensor] = None,
              eps: float = 0.0, delta: Optional[torch.Tensor] = None, resid_out: Optional[torch.Tensor] = None,
              swiglu: bool = False) -> torch.Tensor:
    """out[:rows] = x[:rows] @ weight^T for a few rows.  With `norm_weight`, x is the residual stream: `delta` (if given)
    is added first and the sum written to `resid_out`, then the RMSNorm with `norm_weight` is applied before the
    product.  With `swiglu`, weight holds gate rows over up rows and out receives silu(gate) * up."""
    _gemv_lib()
    _cuda(out, x, weight, norm_weight, delta, resid_out)
    _contig(out, x, weight, norm_weight, delta, resid_out)
    N, K = weight.shape
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or x.shape[1] != K:
        raise KernelError("gemv_bf16: x [M, K], weight [N, K] and out must be bf16")
    if out.shape[1] != (N // 2 if swiglu else N) or out.shape[0] < rows or x.shape[0] < rows:
        raise KernelError("gemv_bf16: out must be [M, N] (or [M, N / 2] with swiglu)")
    if swiglu and norm_weight is None:
        raise KernelError("gemv_bf16: the SwiGLU form comes with the norm prologue")
    if norm_weight is not None and (norm_weight.dtype != torch.float32 or norm_weight.numel() != K):
        raise KernelError("gemv_bf16: norm_weight must be float32 [K]")
    if delta is not None and (norm_weight is None or resid_out is None or delta.dtype != torch.bfloat16
                              or resid_out.dtype != torch.bfloat16 or resid_out.data_ptr() == x.data_ptr()):
        raise KernelError("gemv_bf16: delta needs the norm prologue and a resid_out buffer other than x")
    mode = 0 if norm_weight is None else (2 if swiglu else 1)
    _check(_gemv.cvb_gemv_bf16(_ptr(out), _ptr(x), _ptr(delta), _ptr(resid_out), _ptr(norm_weight), _ptr(weight), c_int(rows),
                               c_int(N), c_int(K), c_float(eps), c_int(mode), _stream()), "gemv_bf16")
    return out


def _gemv_lib():
    global _gemv
    if _gemv is None:
        lib = load_library("gemv_bf16")
        for name in ("cvb_gemv_bf16", "cvb_gemv_splitk_bf16", "cvb_gemv_splitk_counters", "cvb_gemv_stream_bf16",
                     "cvb_gemv_stream_supported", "cvb_gemv_ring_bf16"):
            getattr(lib, name).restype = c_int
        lib.cvb_gemv_splitk_scratch_floats.restype = c_int64
        _gemv = lib
    return _gemv


STREAM_MAX_ROWS = 16
_stream_ok: Dict[tuple, bool] = {}


def gemv_stream_supported(x_dtype: torch.dtype, weight: torch.Tensor, rows: int, swiglu: bool = False) -> bool:
    """The product that runs one block per SM and fetches the block's whole share of the weight ahead of its dependency
    covers bf16 operands, up to 16 rows, and weights whose share per SM (rows / #SMs, whole rows) fits into about half an
    SM's shared memory beside the staged activations (all of it from nine rows on): matrices of a few megabytes."""
    if not (x_dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.dim() == 2 and 0 < rows <= STREAM_MAX_ROWS):
        return False
    key = (weight.shape[0], weight.shape[1], swiglu, rows > 8)
    ok = _stream_ok.get(key)
    if ok is None:
        ok = bool(_gemv_lib().cvb_gemv_stream_supported(c_int(key[0]), c_int(key[1]), c_int(2 if swiglu else 0), c_int(rows)))
        _stream_ok[key] = ok
    return ok


def gemv_stream_bf16(out: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, rows: int, norm_weight: Optional[torch.Tensor] = None,
                     eps: float = 0.0, delta: Optional[torch.Tensor] = None, resid_out: Optional[torch.Tensor] = None,
                     swiglu: bool = False, prefetch: Optional[torch.Tensor] = None, late_trigger: bool = False,
                     dependent: bool = True, add_to: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Same contract as gemv_bf16 for shapes that gemv_stream_supported accepts.  `prefetch`: a tensor that a later kernel
    will stream (asked into the L2 by this kernel).  `late_trigger`: the next kernel on the stream may start only when
    this one's products are done (for successors whose blocks should find the SMs free).  `dependent=False` launches
    without the programmatic-dependent-launch attribute.  `add_to` (plain form only): out = rnd(add_to + rnd(x @ weight^T)),
    the residual sum folded into the product's store; `add_to` may be `out` itself."""
    lib = _gemv_lib()
    _cuda(out, x, weight, norm_weight, delta, resid_out, prefetch, add_to)
    _contig(out, x, weight, norm_weight, delta, resid_out, prefetch, add_to)
    if add_to is not None and (norm_weight is not None or add_to.dtype != torch.bfloat16 or add_to.shape != out.shape):
        raise KernelError("gemv_stream_bf16: add_to goes with the plain form and must be bf16, shaped like out")
    N, K = weight.shape
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or x.shape[1] != K:
        raise KernelError("gemv_stream_bf16: x [M, K], weight [N, K] and out must be bf16")
    if out.shape[1] != (N // 2 if swiglu else N) or out.shape[0] < rows or x.shape[0] < rows:
        raise KernelError("gemv_stream_bf16: out must be [M, N] (or [M, N / 2] with swiglu)")
    if swiglu and norm_weight is None:
        raise KernelError("gemv_stream_bf16: the SwiGLU form comes with the norm prologue")
    if norm_weight is not None and (norm_weight.dtype != torch.float32 or norm_weight.numel() != K):
        raise KernelError("gemv_stream_bf16: norm_weight must be float32 [K]")
    if delta is not None and (norm_weight is None or resid_out is None or delta.dtype != torch.bfloat16
                              or resid_out.dtype != torch.bfloat16 or resid_out.data_ptr() == x.data_ptr()):
        raise KernelError("gemv_stream_bf16: delta needs the norm prologue and a resid_out buffer other than x")
    mode = 0 if norm_weight is None else (2 if swiglu else 1)
    _check(lib.cvb_gemv_stream_bf16(_ptr(out), _ptr(x), _ptr(delta), _ptr(resid_out), _ptr(norm_weight), _ptr(weight), c_int(rows),
                                    c_int(N), c_int(K), c_float(eps), c_int(mode), _ptr(add_to), _ptr(prefetch),
                                    ctypes.c_longlong(prefetch.numel() * prefetch.element_size() if prefetch is not None else 0),
                                    c_int(1 if late_trigger else 0), c_int(1 if dependent else 0),
                                    _ptr(error_flag(x.device)), _stream()), "gemv_stream_bf16")
    return out


_splitk_buffers: Dict[int, list] = {}


def gemv_splitk_preferred(x_dtype: torch.dtype, weight: torch.Tensor, rows: int) -> bool:
    """Weights of 16 MB and more go through the kernel that splits the inner dimension over blocks as well."""
    return (x_dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and 0 < rows <= SPLITK_MAX_ROWS
            and weight.dim() == 2 and weight.shape[1] % 8 == 0 and weight.numel() * 2 >= SPLITK_MIN_BYTES)


def gemv_splitk_bf16(out: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, rows: int) -> torch.Tensor:
    """out[:rows] = x[:rows] @ weight^T for up to 8 rows and a large weight.  The scratch for the partial sums and the
    counters belong to the device and grow with the largest weight seen; they are made at the first call with a weight
    (a warm-up before any graph capture, as the runner does, sizes them)."""
    _gemv_lib()
    _cuda(out, x, weight)
    _contig(out, x, weight)
    N, K = weight.shape
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or x.shape[1] != K:
        raise KernelError("gemv_splitk_bf16: x [M, K], weight [N, K] and out must be bf16")
    if out.shape[1] != N or out.shape[0] < rows or x.shape[0] < rows:
        raise KernelError("gemv_splitk_bf16: out must be [M, N]")
    need_f = int(_gemv.cvb_gemv_splitk_scratch_floats(c_int(N), c_int(K)))
    need_c = int(_gemv.cvb_gemv_splitk_counters(c_int(N)))
    idx = x.device.index if x.device.index is not None else torch.cuda.current_device()
    buf = _splitk_buffers.get(idx)
    if buf is None or buf[0].numel() < need_f or buf[1].numel() < need_c:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("gemv_splitk_bf16: its scratch has to grow; run the shape once before capturing it")
        buf = [torch.empty(max(need_f, buf[0].numel() if buf else 0), dtype=torch.float32, device=x.device),
               torch.zeros(max(need_c, buf[1].numel() if buf else 0, 1024), dtype=torch.int32, device=x.device)]
        _splitk_buffers[idx] = buf
    _check(_gemv.cvb_gemv_splitk_bf16(_ptr(out), _ptr(x), _ptr(weight), c_int(rows), c_int(N), c_int(K), _ptr(buf[0]),
                                      c_int64(buf[0].numel()), _ptr(buf[1]), _stream()), "gemv_splitk_bf16")
    return out


RING_MAX_ROWS = 8


def gemv_ring_supported(x_dtype: torch.dtype, weight: torch.Tensor, rows: int) -> bool:
    """The ring-buffered streaming product covers bf16 operands, up to 8 rows, any weight whose rows are multiples of 16
    bytes; it is meant for weights too large for the decode chain's product."""
    return (x_dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.dim() == 2 and 0 < rows <= RING_MAX_ROWS
            and weight.shape[1] % 8 == 0)


def gemv_ring_bf16(out: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, rows: int, dependent: bool = False) -> torch.Tensor:
    """out[:rows] = x[:rows] @ weight^T for up to 8 rows: one block per SM streams its share of the weight's rows through a
    ring of shared-memory stages filled by bulk copies."""
    lib = _gemv_lib()
    _cuda(out, x, weight)
    _contig(out, x, weight)
    N, K = weight.shape
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or x.shape[1] != K:
        raise KernelError("gemv_ring_bf16: x [M, K], weight [N, K] and out must be bf16")
    if out.shape[1] != N or out.shape[0] < rows or x.shape[0] < rows:
        raise KernelError("gemv_ring_bf16: out must be [M, N]")
    _check(lib.cvb_gemv_ring_bf16(_ptr(out), _ptr(x), _ptr(weight), c_int(rows), c_int(N), c_int(K), c_int(1 if dependent else 0),
                                  _ptr(error_flag(x.device)), _stream()), "gemv_ring_bf16")
    return out


_project_choice: Dict[tuple, str] = {}
_flush_buffers: Dict[int, torch.Tensor] = {}


def _project_candidates(x: torch.Tensor, weight: torch.Tensor, rows: int):
    names = []
    if gemv_supported(x.dtype, weight, rows):
        names.append("gemv")
    if (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and 0 < rows <= SPLITK_MAX_ROWS and weight.dim() == 2
            and weight.shape[1] % 8 == 0 and weight.numel() * 2 >= (1 << 20)):
        names.append("splitk")
    if gemv_ring_supported(x.dtype, weight, rows) and weight.numel() * 2 >= (1 << 20):
        names.append("ring")
    names.append("library")
    return names


def _project_with(name: str, x, weight, out, rows, dependent: bool = False):
    if name == "gemv":
        return gemv_bf16(out, x, weight, rows)
    if name == "splitk":
        return gemv_splitk_bf16(out, x, weight, rows)
    if name == "ring":
        return gemv_ring_bf16(out, x, weight, rows, dependent=dependent)
    return linear(x, weight, out=out)


def _measure_projection(name: str, x, weight, out, rows) -> float:
    """Microseconds of four calls, each with the weight out of the L2 (a buffer larger than the L2 is written before every
    call), replayed from a captured graph so that the host's launch cost does not blur the comparison.  The writes of
    the buffer take the same time for every candidate."""
    idx = x.device.index if x.device.index is not None else torch.cuda.current_device()
    flush = _flush_buffers.get(idx)
    if flush is None:
        flush = torch.empty(256 << 20, dtype=torch.int8, device=x.device)
        _flush_buffers[idx] = flush
    _project_with(name, x, weight, out, rows)                 # sizes its scratch, loads its code
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(4):
            flush.zero_()
            _project_with(name, x, weight, out, rows)
    graph.replay()
    best = float("inf")
    for _ in range(3):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) * 1e3)
    return best


def project_rows(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, rows: int, dependent: bool = True) -> torch.Tensor:
    """out = x @ weight^T by the kernel that suits the step.  A weight whose share per SM fits into shared memory goes
    through the product made for chains of dependent launches (`dependent=False` keeps that kernel behind its
    predecessor's end instead of letting it start early and fetch its weights meanwhile).  Otherwise the candidates for a
    few bf16 rows (the weight-streaming product, its split-K form, the ring-buffered product, the library's product) are timed once per shape, with
    the weight out of the L2, the first time the shape is seen outside a graph capture, and the fastest is kept; during
    a capture an unseen shape takes the split-K form for large weights, the weight-streaming product for small ones.
    CVB_PROJECT=gemv|splitk|ring|library in the environment fixes the choice."""
    if gemv_stream_supported(x.dtype, weight, rows):
        return gemv_stream_bf16(out, x, weight, rows, dependent=dependent)
    if rows > GEMV_MAX_ROWS or x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        return linear(x, weight, out=out)
    key = (weight.shape[0], weight.shape[1], rows if rows <= 2 else (8 if rows <= 8 else 16))
    choice = _project_choice.get(key)
    if choice is None:
        names = _project_candidates(x, weight, rows)
        forced = os.environ.get("CVB_PROJECT")
        if forced in names:
            choice = forced
        elif len(names) == 1:
            choice = names[0]
        elif torch.cuda.is_current_stream_capturing():
            fallback = "splitk" if gemv_splitk_preferred(x.dtype, weight, rows) else ("gemv" if "gemv" in names else "library")
            return _project_with(fallback, x, weight, out, rows)
        else:
            timed = {n: _measure_projection(n, x, weight, out, rows) for n in names}
            choice = min(timed, key=timed.get)
            if os.environ.get("CVB_PROJECT_VERBOSE"):
                print(f"[cppvllm_b200] projection {key}: " + ", ".join(f"{n} {t:.1f} us" for n, t in timed.items()) + f" -> {choice}",
                      file=sys.stderr, flush=True)
        _project_choice[key] = choice
    return _project_with(choice, x, weight, out, rows, dependent)


_gemm = None


def gemm_tcgen05_supported(x_dtype: torch.dtype, weight: torch.Tensor, swiglu: bool = False) -> bool:
    """The tcgen05 product covers bf16 operands with inner sizes that are multiples of 8 and output widths that are
    multiples of 8."""
    n_out = weight.shape[0] // 2 if swiglu else weight.shape[0]
    return (x_dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.shape[1] % 8 == 0 and n_out % 8 == 0
            and (not swiglu or weight.shape[0] % 2 == 0))


def gemm_bf16_tcgen05(out: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, swiglu: bool = False, tile_n: int = 0,
                      resid: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = x @ weight^T on the tcgen05 tensor cores; with `swiglu`, weight holds gate rows over up rows and
    out = silu(x @ gate^T) * (x @ up^T); with `resid` (which may be `out`), out = round(x @ weight^T) + resid.
    `tile_n` (128 or 256) picks the tile width; 0 chooses by the number of tiles it gives."""
    global _gemm
    if _gemm is None:
        lib = load_library("gemm_bf16")
        lib.cvb_gemm_bf16_tcgen05.restype = c_int
        _gemm = lib
    _cuda(out, x, weight, resid); _contig(out, x, weight, resid)
    M, K = x.shape
    N = weight.shape[0]
    n_out = N // 2 if swiglu else N
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or weight.shape[1] != K \
            or out.shape != (M, n_out) or (swiglu and resid is not None) \
            or (resid is not None and (resid.dtype != torch.bfloat16 or resid.shape != out.shape)):
        raise KernelError("gemm_bf16_tcgen05: x [M, K], weight [N, K], out [M, N] (or [M, N / 2] with swiglu), resid like out, "
                          "all bf16")
    if tile_n == 0:
        # tiles of 256 columns halve the traffic of A; take them when they still fill the SMs
        tiles_256 = ((M + 127) // 128) * ((N + 255) // 256)
        tile_n = 256 if tiles_256 >= 120 else 128
    mode = 1 if swiglu else (2 if resid is not None else 0)
    _check(_gemm.cvb_gemm_bf16_tcgen05(_ptr(out), _ptr(x), _ptr(weight), _ptr(resid), c_int(M), c_int(N), c_int(K), c_int(mode),
                                       c_int(tile_n), _ptr(error_flag(x.device)), _stream()), "gemm_bf16_tcgen05")
    return out


GATED_MIN_ROWS = 1024
GATED_SMS = 148


def gated_product_fused(x_dtype: torch.dtype, weight: torch.Tensor, rows: int) -> bool:
    """Whether the gate/up product of `rows` tokens goes through the tcgen05 kernel with the SwiGLU epilogue instead of the
    library's product followed by the SwiGLU kernel.  The fused kernel wins where its tiles of 128 rows by 128 outputs
    fill the SMs at least twice over with little left over in the last round (measured on a B200, against the library
    product plus the SwiGLU kernel: 2,048 x 6,144 x 1,024: 25 us against 30; 4,096 rows: 43 against 57; 2,048 x 24,576 x
    4,096: 281 against 302; 1,024 rows or fewer: the library wins by 2 to 35 %).  CVB_GATED=fused|library fixes it."""
    forced = os.environ.get("CVB_GATED", "")
    ok = (x_dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.dim() == 2 and weight.shape[1] % 8 == 0
          and weight.shape[0] % 16 == 0)
    if not ok or forced == "library":
        return False
    if forced == "fused":
        return True
    if rows < GATED_MIN_ROWS:
        return False
    tiles = ((rows + 127) // 128) * ((weight.shape[0] // 2 + 127) // 128)
    rounds = tiles / GATED_SMS
    return rounds >= 2 and rounds / math.ceil(rounds) >= 0.8


# ---- sampling ----------------------------------------------------------------------------------------------

def sample(out: torch.Tensor, logits: torch.Tensor, rows: Optional[torch.Tensor], temps: torch.Tensor,
           seeds: torch.Tensor, out_positions: torch.Tensor, num_rows: Optional[int] = None,
           scratch: Optional[torch.Tensor] = None, chunks: int = 0) -> torch.Tensor:
    """With `scratch` (any dtype, at least rows * chunks * 8 bytes) and `chunks` > 1 the vocabulary of every row is
    searched by `chunks` blocks in parallel; the token is the same as with one block per row."""
    _cuda(out, logits, rows, temps, seeds, out_positions); _contig(out, logits, rows, temps, seeds, out_positions)
    R = out.numel() if num_rows is None else num_rows
    if (logits.dtype != torch.float32 or logits.dim() != 2 or out.dtype != torch.int32 or temps.dtype != torch.float32
            or seeds.dtype != torch.int64 or out_positions.dtype != torch.int32
            or (rows is not None and rows.dtype != torch.int32)):
        raise KernelError("sample: logits float32 [N, V]; out, rows, out_positions int32; temps float32; seeds int64")
    if scratch is not None and chunks > 1:
        _cuda(scratch); _contig(scratch)
        _check(core().cvb_sample_chunked(_ptr(out), _ptr(logits), _ptr(rows), _ptr(temps), _ptr(seeds), _ptr(out_positions),
                                         c_int(R), c_int(logits.shape[1]), c_int(logits.shape[0]), c_int(chunks), _ptr(scratch),
                                         c_int64(scratch.numel() * scratch.element_size()), _stream()), "sample", kernels=2)
        return out
    _check(core().cvb_sample(_ptr(out), _ptr(logits), _ptr(rows), _ptr(temps), _ptr(seeds), _ptr(out_positions),
                             c_int(R), c_int(logits.shape[1]), c_int(logits.shape[0]), _stream()), "sample")
    return out


def feed_tokens(tokens: torch.Tensor, src: torch.Tensor, sampled: torch.Tensor, n: int) -> torch.Tensor:
    _cuda(tokens, src, sampled); _contig(tokens, src, sampled)
    if tokens.dtype != torch.int32 or src.dtype != torch.int32 or sampled.dtype != torch.int32:
        raise KernelError("feed_tokens: all arguments must be int32")
    _check(core().cvb_feed_tokens(_ptr(tokens), _ptr(src), _ptr(sampled), c_int(n), c_int(sampled.numel()), _stream()),
           "feed_tokens")
    return tokens


# ---- library matrix products ---------------------------------------------------------------------------------

def linear(x: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """y = x @ weight^T through cuBLAS, as the reference does with at::linear (model_architecture.cpp:155,178,
    182,185,224).  float32 operands use full float32 arithmetic (no TF32); bf16 operands accumulate in
    float32.  `out_dtype=torch.float32` with bf16 operands returns the float32 accumulators unrounded."""
    _cuda(x, weight)
    if x.dtype != weight.dtype:
        if weight.dtype == torch.float32 and x.dtype == torch.bfloat16:
            # a weight stored in 32-bit stays so: the product runs in float32 and is rounded once at the end
            y = torch.mm(x.float(), weight.t())
            want = out_dtype or x.dtype
            if out is not None:
                out.copy_(y)
                return out
            return y.to(want)
        raise KernelError(f"linear: activations are {x.dtype} but the weight is {weight.dtype}")
    if out_dtype is not None and out_dtype != x.dtype:
        if out is not None:
            return torch.mm(x, weight.t(), out_dtype=out_dtype, out=out)
        return torch.mm(x, weight.t(), out_dtype=out_dtype)
    if out is not None:
        return torch.mm(x, weight.t(), out=out)
    return torch.mm(x, weight.t())


def configure_library_matmul() -> None:
    """Pin cuBLAS to exact modes: float32 products in true float32 (no TF32), bf16 products with float32
    accumulation and no reduced-precision split-K reduction."""
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    try:
        torch.backends.cuda.matmul.fp32_precision = "ieee"
    except (AttributeError, RuntimeError):
        torch.backends.cuda.matmul.allow_tf32 = False
