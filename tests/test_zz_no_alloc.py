"""The decode attention entry point that allocates nothing (cvb_attn_decode_bf16_static).

Some callers of the attention library cannot allocate device memory while they run: a loop that is forbidden to
call cudaMalloc, or a plug-in whose host owns all of the device's memory.  For them the library keeps the scratch
of the split-KV kernel in a static device array.  This test calls that entry point through its exported C symbol,
twice in a row with different inputs (the array keeps the first call's contents), and checks each output against
the ordinary entry point, which takes its scratch from the caller, and against a plain float32 restatement of the
attention; with and without a window.  It runs in a file that pytest collects last, and must pass alone in a fresh
process as well as after all other tests."""
import ctypes
import math
from ctypes import c_float, c_int, c_int64, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(seed, batch, context, H, KV, hd, page):
    d = torch.device("cuda:0")
    g = torch.Generator().manual_seed(seed)
    pages_per_seq = (context + page - 1) // page
    n_pages = batch * pages_per_seq
    cache = torch.randn(n_pages + 2, 2, KV, page, hd, generator=g).to(torch.bfloat16).to(d)
    tables = torch.randperm(n_pages, generator=g).to(torch.int32).view(batch, pages_per_seq).contiguous().to(d)
    q = (torch.randn(batch, H * hd, generator=g) * 1.5).to(torch.bfloat16).to(d)
    cu = torch.arange(0, batch + 1, dtype=torch.int32, device=d)
    lens = torch.randint(context // 2, context, (batch,), generator=g)
    pos = (lens - 1).to(torch.int32).to(d)
    return cache, tables, q, cu, pos


def _plain_attention(q, cache, tables, pos, H, KV, hd, page, scale, window):
    """softmax(scale q.k) v over the positions lo .. pos of every request, in float32, straight from the pages."""
    out = torch.zeros(q.shape[0], H, hd)
    cache, tables, q = cache.float().cpu(), tables.cpu(), q.float().cpu().view(-1, H, hd)
    for s in range(q.shape[0]):
        p = int(pos[s])
        lo = max(0, p - window + 1) if window > 0 else 0
        idx = torch.arange(lo, p + 1)
        pages, offs = tables[s, idx // page].long(), idx % page
        for h in range(H):
            g = h // (H // KV)
            k, v = cache[pages, 0, g, offs], cache[pages, 1, g, offs]
            out[s, h] = torch.softmax((k @ q[s, h]) * scale, 0) @ v
    return out.view(q.shape[0], H * hd)


def _call_static(lib, out, q, cache, tables, cu, pos, batch, H, KV, hd, page, scale, splits, err, window=0):
    stream = torch.cuda.current_stream().cuda_stream
    num_pages = cache.numel() // (2 * KV * page * hd)
    return lib.cvb_attn_decode_bf16_static(
        c_void_p(out.data_ptr()), c_void_p(q.data_ptr()), c_void_p(cache.data_ptr()), c_void_p(tables.data_ptr()),
        c_int(tables.shape[1]), c_void_p(cu.data_ptr()), c_void_p(pos.data_ptr()), c_int(batch), c_int(H), c_int(KV),
        c_int(hd), c_int(page), c_int(window), c_float(scale), c_int(num_pages), c_int(splits), c_void_p(err.data_ptr()),
        c_void_p(stream))


@pytest.mark.parametrize("H,KV,hd,page,window", [(16, 8, 128, 16, 0), (6, 2, 64, 32, 0), (8, 2, 128, 32, 200)])
def test_static_scratch_entry_point_matches_the_ordinary_one_twice_in_a_row(H, KV, hd, page, window):
    from cppvllm_b200.csrc import ops
    from cppvllm_b200.csrc.build import build_library
    lib = ctypes.CDLL(build_library("attn_bf16"))          # the exported C symbols, not the package's wrappers
    lib.cvb_attn_decode_bf16_static.restype = c_int
    lib.cvb_attn_decode_static_scratch_floats.restype = c_int64
    limit = lib.cvb_attn_decode_static_scratch_floats()
    assert limit == 1 << 21
    batch, scale = 5, 1 / math.sqrt(hd)
    err = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    for call, (seed, context, splits) in enumerate([(1, 700, 6), (2, 333, 3)]):
        cache, tables, q, cu, pos = _inputs(seed, batch, context, H, KV, hd, page)
        want = torch.zeros_like(q)
        n = ops.attn_decode_scratch_floats(batch, KV, hd, splits)
        assert n <= limit
        ops.attn_decode_bf16(want, q, cache, tables, cu, pos, batch, H, KV, hd, page, scale, splits,
                             torch.empty(n, dtype=torch.float32, device=q.device), window=window)
        got = torch.full_like(q, float("nan"))
        rc = _call_static(lib, got, q, cache, tables, cu, pos, batch, H, KV, hd, page, scale, splits, err, window)
        assert rc == 0, f"call {call}: status {rc}"
        torch.cuda.synchronize()
        assert int(err.item()) == 0
        torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2e-2)
        assert torch.isfinite(got.float()).all()
        plain = _plain_attention(q, cache, tables, pos.cpu(), H, KV, hd, page, scale, window)
        torch.testing.assert_close(got.float().cpu(), plain.to(torch.bfloat16).float(), atol=2e-2, rtol=2e-2)
    # one split needs no scratch at all and still works
    got1 = torch.zeros_like(q)
    assert _call_static(lib, got1, q, cache, tables, cu, pos, batch, H, KV, hd, page, scale, 1, err, window) == 0
    torch.cuda.synchronize()
    torch.testing.assert_close(got1.float(), want.float(), atol=2e-2, rtol=2e-2)


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from cppvllm_b200.csrc.build import build_library
    lib = ctypes.CDLL(build_library("attn_bf16"))
    lib.cvb_attn_decode_bf16_static.restype = c_int
    H, KV, hd, page, batch = 16, 8, 128, 16, 64
    cache, tables, q, cu, pos = _inputs(3, batch, 64, H, KV, hd, page)
    err = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    out = torch.zeros_like(q)
    # 64 requests * 8 kv heads * 32 splits * 16 rows * 130 floats = 34 M floats > 2 M
    assert _call_static(lib, out, q, cache, tables, cu, pos, batch, H, KV, hd, page, 0.1, 32, err) == -6
    torch.cuda.synchronize()
    assert out.abs().max() == 0 and int(err.item()) == 0    # nothing was launched
