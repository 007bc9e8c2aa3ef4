"""Each CUDA kernel alone against a plain PyTorch float32 restatement of the same formula, at sizes other than
the engine's tiny models (odd widths, head sizes in steps of 16, groups of 1, 3, 5 and 7, windows, page edges)."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def dev():
    return torch.device("cuda:0")


def rnd(x, dt):
    return x.to(dt).float()


def tol(dt):
    return dict(atol=2e-6, rtol=2e-6) if dt == torch.float32 else dict(atol=1e-2, rtol=1.6e-2)


@pytest.fixture(scope="module")
def ops():
    from cppvllm_b200.csrc import ops as o
    o.core()
    return o


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("T,D", [(1, 7), (5, 100), (33, 1000), (3, 4104)])
def test_rmsnorm_and_add_rmsnorm(ops, dt, T, D):
    g = torch.Generator(device="cpu").manual_seed(T * 1000 + D)
    x = (torch.randn(T, D, generator=g) * 3).to(dt).to(dev())
    r = torch.randn(T, D, generator=g).to(dt).to(dev())
    w = (1 + 0.3 * torch.randn(D, generator=g)).to(dev())
    eps = 3e-5
    out = torch.empty_like(x)
    ops.rmsnorm(out, x, w, eps)
    xf = x.float()
    ref = rnd(rnd(xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + eps), dt) * w, dt)
    torch.testing.assert_close(out.float(), ref, **tol(dt))
    res = r.clone()
    ops.add_rmsnorm(out, res, x, w, eps)
    s = rnd(r.float() + xf, dt)
    torch.testing.assert_close(res.float(), s, atol=0, rtol=0)
    ref = rnd(rnd(s * torch.rsqrt((s * s).mean(-1, keepdim=True) + eps), dt) * w, dt)
    torch.testing.assert_close(out.float(), ref, **tol(dt))
    ops.add_(res, x)
    torch.testing.assert_close(res.float(), rnd(s + xf, dt), atol=0, rtol=0)


@pytest.mark.parametrize("dt", DTYPES)
def test_swiglu_embed_gather(ops, dt):
    g = torch.Generator().manual_seed(0)
    gu = (torch.randn(9, 2 * 37, generator=g) * 4).to(dt).to(dev())
    out = torch.empty(9, 37, dtype=dt, device=dev())
    ops.swiglu(out, gu)
    gate, up = gu[:, :37].float(), gu[:, 37:].float()
    torch.testing.assert_close(out.float(), rnd(rnd(gate / (1 + torch.exp(-gate)), dt) * up, dt), **tol(dt))
    table = torch.randn(50, 13, generator=g).to(dt).to(dev())
    toks = torch.tensor([3, 49, 0, 3, 17], dtype=torch.int32, device=dev())
    e = torch.empty(5, 13, dtype=dt, device=dev())
    ops.embed(e, table, toks)
    assert torch.equal(e, table[toks.long()])
    rows = torch.tensor([4, 0, 0, 2], dtype=torch.int32, device=dev())
    o = torch.empty(4, 13, dtype=dt, device=dev())
    ops.gather_rows(o, e, rows)
    assert torch.equal(o, e[rows.long()])


def test_embed_reports_a_token_outside_the_table(ops):
    table = torch.randn(10, 4, device=dev())
    out = torch.empty(2, 4, device=dev())
    ops.embed(out, table, torch.tensor([1, 10], dtype=torch.int32, device=dev()))
    with pytest.raises(ops.KernelError, match="outside the embedding table"):
        ops.check_device_errors(dev())
    ops.check_device_errors(dev())          # the flag was cleared


def test_wrong_arguments_are_refused(ops):
    x = torch.randn(4, 8, device=dev())
    with pytest.raises(ops.KernelError, match="float32"):
        ops.rmsnorm(torch.empty_like(x), x, torch.ones(8, device=dev(), dtype=torch.bfloat16), 1e-6)
    with pytest.raises(ops.KernelError, match="CUDA tensors only"):
        ops.rmsnorm(torch.empty(4, 8), torch.randn(4, 8), torch.ones(8), 1e-6)
    with pytest.raises(ops.KernelError, match="float32 or bfloat16"):
        ops.rmsnorm(x.half(), x.half(), torch.ones(8, device=dev()), 1e-6)
    with pytest.raises(ops.KernelError, match="multiple"):
        ops.paged_attention_general(torch.empty(1, 5 * 16, device=dev()), torch.empty(1, 5 * 16, device=dev()),
                                    torch.zeros(2, 2, 2, 16, 16, device=dev()), torch.zeros(1, 1, dtype=torch.int32, device=dev()),
                                    torch.zeros(1, dtype=torch.int32, device=dev()), torch.zeros(1, dtype=torch.int32, device=dev()),
                                    5, 2, 16, 16, 0.25)


def rope_ref(n, cos, sin, pos, rot, interleaved):
    out = n.clone()
    half = rot // 2
    c, s = cos[pos][:, None, :], sin[pos][:, None, :]
    if interleaved:
        a, b = n[..., 0:rot:2], n[..., 1:rot:2]
        out[..., 0:rot:2] = a * c - b * s
        out[..., 1:rot:2] = b * c + a * s
    else:
        a, b = n[..., :half], n[..., half:rot]
        out[..., :half] = a * c - b * s
        out[..., half:rot] = b * c + a * s
    return out


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("H,KV,hd,rot,inter,norm", [(5, 5, 16, 16, False, True), (6, 2, 48, 48, False, True),
                                                    (7, 1, 80, 32, True, True), (3, 3, 144, 144, False, False),
                                                    (8, 4, 256, 128, False, True), (16, 8, 128, 128, False, True),
                                                    (3, 1, 64, 64, False, True), (4, 2, 32, 32, False, False),
                                                    (2, 2, 256, 256, False, True)])
def test_qk_norm_rope_kv_write(ops, dt, H, KV, hd, rot, inter, norm):
    T, page, pages, max_pos, eps = 23, 16, 9, 300, 2e-5
    g = torch.Generator().manual_seed(hd)
    qkv = torch.randn(T, (H + 2 * KV) * hd, generator=g).to(dt).to(dev())
    qw = (1 + 0.2 * torch.randn(hd, generator=g)).to(dev()) if norm else None
    kw = (1 + 0.2 * torch.randn(hd, generator=g)).to(dev()) if norm else None
    ang = torch.outer(torch.arange(max_pos, dtype=torch.float64), 1.0 / (5000.0 ** (torch.arange(0, rot, 2, dtype=torch.float64) / rot)))
    cos, sin = ang.cos().float().to(dev()), ang.sin().float().to(dev())
    pos = torch.randint(0, max_pos, (T,), generator=g).int().to(dev())
    slots = torch.randperm(pages * page, generator=g)[:T].int().to(dev())
    cache = torch.zeros(pages, 2, KV, page, hd, dtype=dt, device=dev())
    q = torch.empty(T, H * hd, dtype=dt, device=dev())
    ops.qk_norm_rope_kv(q, qkv, qw, kw, cos, sin, pos, slots, cache, H, KV, hd, page, eps, rotary_dim=rot, interleaved=inter)
    ops.check_device_errors(dev())
    x = qkv.float().view(T, H + 2 * KV, hd)
    def headnorm(v, w):
        if w is None:
            return v
        return rnd(rnd(v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps), dt) * w, dt)
    qr = rnd(rope_ref(headnorm(x[:, :H], qw), cos, sin, pos.long(), rot, inter), dt)
    kr = rnd(rope_ref(headnorm(x[:, H:H + KV], kw), cos, sin, pos.long(), rot, inter), dt)
    torch.testing.assert_close(q.float().view(T, H, hd), qr, **tol(dt))
    sl = slots.long()
    torch.testing.assert_close(cache[sl // page, 0, :, sl % page].float(), kr, **tol(dt))
    assert torch.equal(cache[sl // page, 1, :, sl % page], qkv.view(T, H + 2 * KV, hd)[:, H + KV:])
    untouched = torch.ones(pages * page, dtype=torch.bool)
    untouched[sl.cpu()] = False
    flat = cache.permute(0, 3, 1, 2, 4).reshape(pages * page, -1)
    assert flat[untouched.to(dev())].abs().max() == 0          # nothing but the step's slots was written
    # a layer that only reads another layer's cache writes nothing
    cache2 = torch.zeros_like(cache)
    q2 = torch.empty_like(q)
    ops.qk_norm_rope_kv(q2, qkv, qw, kw, cos, sin, pos, None, None, H, KV, hd, page, eps, rotary_dim=rot, interleaved=inter)
    assert torch.equal(q2, q) and cache2.abs().max() == 0


def attention_ref(q, k_all, v_all, kv_lens_per_token, positions, H, KV, hd, scale, window):
    """q: [T, H, hd]; k_all/v_all: list per token of that token's sequence keys [len, KV, hd]."""
    out = torch.zeros_like(q)
    for t in range(q.shape[0]):
        p = int(positions[t])
        lo = max(0, p - window + 1) if window > 0 else 0
        for h in range(H):
            g = h // (H // KV)
            k = k_all[t][lo:p + 1, g].float()
            v = v_all[t][lo:p + 1, g].float()
            s = (k @ q[t, h].float()) * scale
            out[t, h] = torch.softmax(s, 0) @ v
    return out


def build_paged(seqs_k, seqs_v, page, pages_total, KV, hd, dt, g):
    """Scatter per-sequence K/V [len, KV, hd] into shuffled pages; returns cache and block tables."""
    cache = torch.randn(pages_total, 2, KV, page, hd, generator=g).to(dt)       # garbage where nothing is stored
    perm = torch.randperm(pages_total, generator=g).tolist()
    W = max((k.shape[0] + page - 1) // page for k in seqs_k)
    tables = torch.full((len(seqs_k), W), -1, dtype=torch.int32)
    for s, (k, v) in enumerate(zip(seqs_k, seqs_v)):
        for i in range((k.shape[0] + page - 1) // page):
            pg = perm.pop()
            tables[s, i] = pg
            n = min(page, k.shape[0] - i * page)
            cache[pg, 0, :, :n] = k[i * page:i * page + n].transpose(0, 1)
            cache[pg, 1, :, :n] = v[i * page:i * page + n].transpose(0, 1)
    return cache, tables


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("H,KV,hd,page,window", [(4, 4, 16, 16, 0), (6, 2, 32, 32, 0), (5, 1, 64, 16, 0), (7, 7, 48, 16, 37),
                                                 (8, 2, 128, 64, 0), (3, 1, 160, 16, 130), (14, 2, 96, 16, 0)])
def test_paged_attention_general(ops, dt, H, KV, hd, page, window):
    g = torch.Generator().manual_seed(H * 100 + hd)
    lens = [1, 17, page, page + 1, 300, 129]
    seqs_k = [torch.randn(n, KV, hd, generator=g).to(dt) for n in lens]
    seqs_v = [torch.randn(n, KV, hd, generator=g).to(dt) for n in lens]
    cache, tables = build_paged(seqs_k, seqs_v, page, 64, KV, hd, dt, g)
    # queries: the last tokens of each sequence (a portion), plus some in the middle
    seq_of, positions = [], []
    for s, n in enumerate(lens):
        for p in sorted(set([0, n // 2, max(0, n - 3), max(0, n - 2), n - 1])):
            seq_of.append(s)
            positions.append(p)
    T = len(seq_of)
    q = (torch.randn(T, H, hd, generator=g) * 2).to(dt)
    scale = 1 / math.sqrt(hd)
    out = torch.empty(T, H * hd, dtype=dt, device=dev())
    ops.paged_attention_general(out, q.view(T, -1).to(dev()), cache.to(dev()), tables.to(dev()),
                                torch.tensor(seq_of, dtype=torch.int32, device=dev()),
                                torch.tensor(positions, dtype=torch.int32, device=dev()), H, KV, hd, page, scale, window=window)
    ops.check_device_errors(dev())
    ref = attention_ref(q, [seqs_k[s] for s in seq_of], [seqs_v[s] for s in seq_of], None, positions, H, KV, hd, scale, window)
    torch.testing.assert_close(out.float().cpu().view(T, H, hd), rnd(ref, dt), **tol(dt))


@pytest.mark.parametrize("dt", DTYPES)
def test_attention_finds_one_far_key_and_respects_the_window_edge(ops, dt):
    """One key far back among hundreds is made to dominate; the output must be its value.  With a window that
    just excludes it, the output must not contain it."""
    H = KV = 2
    hd, page, n = 32, 16, 700
    g = torch.Generator().manual_seed(1)
    k = torch.randn(n, KV, hd, generator=g) * 0.1
    v = torch.randn(n, KV, hd, generator=g)
    q = torch.randn(1, H, hd, generator=g)
    far = 37
    k[far] = q[0] * 4.0                                           # score ~ 4 |q|^2 / sqrt(hd): dominates the softmax
    cache, tables = build_paged([k.to(dt)], [v.to(dt)], page, 50, KV, hd, dt, g)
    args = (torch.zeros(1, dtype=torch.int32, device=dev()), torch.tensor([n - 1], dtype=torch.int32, device=dev()))
    out = torch.empty(1, H * hd, dtype=dt, device=dev())
    ops.paged_attention_general(out, q.view(1, -1).to(dt).to(dev()), cache.to(dev()), tables.to(dev()), *args,
                                H, KV, hd, page, 1 / math.sqrt(hd))
    torch.testing.assert_close(out.float().cpu().view(H, hd), v[far].to(dt).float(), atol=2e-2, rtol=2e-2)
    for window, sees in ((n - far, True), (n - far - 1, False)):      # the edge of the window, to the key
        ops.paged_attention_general(out, q.view(1, -1).to(dt).to(dev()), cache.to(dev()), tables.to(dev()), *args,
                                    H, KV, hd, page, 1 / math.sqrt(hd), window=window)
        close = torch.allclose(out.float().cpu().view(H, hd), v[far].to(dt).float(), atol=2e-2, rtol=2e-2)
        assert close == sees
    ops.check_device_errors(dev())


def test_attention_reports_a_missing_page(ops):
    cache = torch.zeros(4, 2, 1, 16, 16, device=dev())
    tables = torch.tensor([[0, -1]], dtype=torch.int32, device=dev())
    out = torch.empty(1, 16, device=dev())
    ops.paged_attention_general(out, torch.zeros(1, 16, device=dev()), cache, tables, torch.zeros(1, dtype=torch.int32, device=dev()),
                                torch.tensor([20], dtype=torch.int32, device=dev()), 1, 1, 16, 16, 0.25)
    with pytest.raises(ops.KernelError, match="page is missing"):
        ops.check_device_errors(dev())


# ---- sampling ----------------------------------------------------------------------------------------------

def philox(c, k):
    c = [np.uint32(x) for x in c]
    k = [np.uint32(k[0]), np.uint32(k[1])]
    for _ in range(10):
        p0 = np.uint64(0xD2511F53) * np.uint64(c[0])
        p1 = np.uint64(0xCD9E8D57) * np.uint64(c[2])
        c = [np.uint32(p1 >> np.uint64(32)) ^ c[1] ^ k[0], np.uint32(p1 & np.uint64(0xFFFFFFFF)),
             np.uint32(p0 >> np.uint64(32)) ^ c[3] ^ k[1], np.uint32(p0 & np.uint64(0xFFFFFFFF))]
        k = [np.uint32((int(k[0]) + 0x9E3779B9) & 0xFFFFFFFF), np.uint32((int(k[1]) + 0xBB67AE85) & 0xFFFFFFFF)]
    return c


def sample_ref(row, temp, seed, opos):
    if temp <= 0:
        return int(np.argmax(row))
    inv_t = np.float32(1.0) / max(np.float32(temp), np.float32(1e-5))
    best, best_i = -np.inf, -1
    for base in range(0, len(row), 4):
        r = philox([base >> 2, opos, 0x53414D50, 0], [seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF])
        for j in range(4):
            if base + j >= len(row):
                break
            u = (np.float32(int(r[j]) >> 8) + np.float32(0.5)) * np.float32(1.0 / 16777216.0)
            e = max(-np.log(u, dtype=np.float32), np.float32(1e-10))
            s = np.float32(row[base + j]) * inv_t - np.log(e, dtype=np.float32)
            if s > best:
                best, best_i = s, base + j
    return best_i


def test_sampling_matches_its_formula_and_does_not_depend_on_the_batch(ops):
    with np.errstate(over="ignore"):
        V, R = 1003, 6
        g = torch.Generator().manual_seed(3)
        logits = (torch.randn(R, V, generator=g) * 2).to(dev())
        logits[0, 500] = logits[0, 7] = 50.0                        # a tie: greedy takes the lower index
        temps = torch.tensor([0.0, 0.7, 1.0, 0.0, 0.3, 5.0], device=dev())
        seeds = torch.tensor([1, 2, 0x123456789ABCDEF, 4, 5, -7], dtype=torch.int64, device=dev())
        opos = torch.tensor([0, 3, 100, 1, 0, 9], dtype=torch.int32, device=dev())
        out = torch.zeros(R, dtype=torch.int32, device=dev())
        ops.sample(out, logits, None, temps, seeds, opos)
        got = out.tolist()
        assert got[0] == 7 and got[3] == int(logits[3].argmax())
        rows = logits.cpu().numpy()
        for r in (1, 2, 4, 5):
            sd = int(seeds[r]) & ((1 << 64) - 1)
            assert got[r] == sample_ref(rows[r], float(temps[r]), sd, int(opos[r]))
        # the same row alone, or at another place of another batch, draws the same token
        order = torch.tensor([4, 1, 5], dtype=torch.int32, device=dev())
        out2 = torch.zeros(3, dtype=torch.int32, device=dev())
        ops.sample(out2, logits, order, temps[order.long()].contiguous(), seeds[order.long()].contiguous(), opos[order.long()].contiguous())
        assert out2.tolist() == [got[4], got[1], got[5]]
        # other output positions and other seeds give other draws (with overwhelming probability over 20 tries)
        draws = set()
        for p in range(20):
            ops.sample(out, logits, None, temps, seeds, torch.full((R,), p, dtype=torch.int32, device=dev()))
            draws.add(out[5].item())
        assert len(draws) > 5


def test_chunked_sampling_returns_the_same_tokens(ops):
    V, R = 50021, 9
    g = torch.Generator().manual_seed(11)
    logits = (torch.randn(R, V, generator=g) * 3).to(dev())
    logits[3, 40000] = logits[3, 123] = 99.0          # a tie in a greedy row, in different chunks
    temps = torch.tensor([0.0, 0.6, 1.0, 0.0, 0.3, 2.0, 0.6, 0.6, 0.0], device=dev())
    seeds = torch.arange(R, dtype=torch.int64, device=dev()) * 977 + 5
    opos = torch.arange(R, dtype=torch.int32, device=dev())
    a = torch.zeros(R, dtype=torch.int32, device=dev())
    ops.sample(a, logits, None, temps, seeds, opos)
    for chunks in (2, 7, 32, 64):
        b = torch.full((R,), -1, dtype=torch.int32, device=dev())
        scratch = torch.empty(R * chunks * 2, dtype=torch.float32, device=dev())
        ops.sample(b, logits, None, temps, seeds, opos, scratch=scratch, chunks=chunks)
        assert b.tolist() == a.tolist()
    assert a[3].item() == 123


def test_temperature_sampling_follows_the_distribution(ops):
    V, N = 8, 4000
    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0, 0.5, -3.0, 1.5, 0.0]], device=dev()).repeat(N, 1).contiguous()
    out = torch.zeros(N, dtype=torch.int32, device=dev())
    ops.sample(out, logits, None, torch.full((N,), 0.8, device=dev()), torch.arange(N, dtype=torch.int64, device=dev()),
               torch.zeros(N, dtype=torch.int32, device=dev()))
    freq = torch.bincount(out.long(), minlength=V).float().cpu() / N
    p = torch.softmax(logits[0].cpu() / 0.8, 0)
    assert (freq - p).abs().max() < 0.03


def test_feed_tokens(ops):
    tokens = torch.tensor([5, 6, 7, 8], dtype=torch.int32, device=dev())
    src = torch.tensor([-1, 1, -1, 0], dtype=torch.int32, device=dev())
    sampled = torch.tensor([40, 41], dtype=torch.int32, device=dev())
    ops.feed_tokens(tokens, src, sampled, 4)
    assert tokens.tolist() == [5, 41, 7, 40]


# ---- tensor-core attention (bf16, head sizes 64 and 128) against the plain restatement -----------------------

@pytest.mark.parametrize("prefill", ["tcgen05", "mma"])
@pytest.mark.parametrize("H,KV,hd,page,window", [(4, 2, 128, 16, 0), (6, 2, 64, 16, 0), (8, 1, 128, 32, 0), (5, 5, 64, 64, 0),
                                                 (16, 8, 128, 16, 0), (14, 2, 128, 16, 150), (3, 1, 64, 16, 70), (32, 2, 64, 16, 0)])
def test_tensor_core_attention_mixed_portions_and_single_tokens(ops, H, KV, hd, page, window, prefill):
    dt = torch.bfloat16
    g = torch.Generator().manual_seed(H * 7 + hd + page)
    # (tokens already in the cache, tokens in this step): portions at the start, in the middle, crossing tile and page
    # edges, and single decoded tokens at short and long contexts
    reqs = [(0, 70), (0, 1), (130, 1), (63, 2), (64, 64), (500, 1), (17, 130), (255, 1), (256, 1), (0, 5), (1000, 3), (777, 1)]
    seqs_k = [torch.randn(c + n, KV, hd, generator=g).to(dt) for c, n in reqs]
    seqs_v = [torch.randn(c + n, KV, hd, generator=g).to(dt) for c, n in reqs]
    total_pages = sum((c + n + page - 1) // page for c, n in reqs) + 3
    cache, tables = build_paged(seqs_k, seqs_v, page, total_pages, KV, hd, dt, g)
    # what a former holder left behind a request's last key, in the same page: it has probability 0, and 0 times this
    # must not reach the output
    for s, (c, n) in enumerate(reqs):
        if (c + n) % page:
            cache[tables[s, (c + n - 1) // page], :, :, (c + n) % page:] = float("nan") if s % 2 else float("inf")
    if window > 0:
        # as in the engine: a request has given back the pages that lie wholly below its window (table entry -1), and
        # someone else may have left anything in them (here NaN): no kernel may look them up or read them
        for s, (c, n) in enumerate(reqs):
            for slot in range(max(0, c - window + 1) // page):
                cache[tables[s, slot]] = float("nan")
                tables[s, slot] = -1
    cu, positions, seq_of = [0], [], []
    for s, (c, n) in enumerate(reqs):
        cu.append(cu[-1] + n)
        positions += list(range(c, c + n))
        seq_of += [s] * n
    T = cu[-1]
    q = (torch.randn(T, H, hd, generator=g) * 1.5).to(dt)
    scale = 1 / math.sqrt(hd)
    d = dev()
    out = torch.zeros(T, H * hd, dtype=dt, device=d)
    q_lens = [n for _, n in reqs]
    cu_t = torch.tensor(cu, dtype=torch.int32, device=d)
    pos_t = torch.tensor(positions, dtype=torch.int32, device=d)
    if prefill == "tcgen05":
        ops.attn_prefill_tcgen05(out, q.view(T, -1).to(d), cache.to(d), tables.to(d), cu_t, pos_t, len(reqs),
                                 ops.prefill_tiles_tcgen05(q_lens, H, KV), H, KV, hd, page, scale, window=window)
    else:
        ops.attn_prefill_bf16(out, q.view(T, -1).to(d), cache.to(d), tables.to(d), cu_t, pos_t, len(reqs),
                              ops.prefill_tiles(q_lens, H, KV), H, KV, hd, page, scale, window=window)
    results = {}
    for splits, cluster in ((1, True), (3, True), (7, True), (7, False), (12, True), (20, True)):
        o2 = out.clone()
        n = ops.attn_decode_scratch_floats(len(reqs), KV, hd, splits)
        scratch = torch.full((max(n, 1),), float("nan"), device=d) if splits > 1 else None
        ops.attn_decode_bf16(o2, q.view(T, -1).to(d), cache.to(d), tables.to(d), cu_t, pos_t, len(reqs), H, KV, hd, page,
                             scale, splits, scratch, window=window, cluster_merge=cluster)
        results[(splits, cluster)] = o2.float().cpu().view(T, H, hd)
    ops.check_device_errors(d)
    ref = attention_ref(q, [seqs_k[s] for s in seq_of], [seqs_v[s] for s in seq_of], None, positions, H, KV, hd, scale, window)
    for _, got in results.items():
        torch.testing.assert_close(got, rnd(ref, dt), atol=2e-2, rtol=2e-2)
    # merged in the cluster's shared memory or by the second kernel: the same sums in the same order
    assert torch.equal(results[(7, True)], results[(7, False)])
    # and against the general kernel of the package
    gen = torch.empty_like(out)
    ops.paged_attention_general(gen, q.view(T, -1).to(d), cache.to(d), tables.to(d), torch.tensor(seq_of, dtype=torch.int32, device=d),
                                pos_t, H, KV, hd, page, scale, window=window)
    torch.testing.assert_close(results[(3, True)], gen.float().cpu().view(T, H, hd), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("H,KV,hd,page,window", [(4, 2, 128, 16, 0), (6, 1, 64, 32, 0), (6, 2, 128, 16, 300), (16, 8, 128, 32, 0)])
@pytest.mark.parametrize("pieces,min_rounds", [(2, 1), (3, 2), (8, 1), (5, 4)])
def test_tcgen05_prefill_shares_the_keys_of_long_query_blocks_among_blocks(ops, H, KV, hd, page, window, pieces, min_rounds):
    """Query blocks with many key tiles are worked on by several blocks, each with a range of the tiles, and a second
    kernel adds their shares up: the same rows as one block per query block gives, at contexts where the pieces' edges
    fall before, inside and after a query tile's own keys.  One early key of the longest request is made to stand out
    (its query and key are scaled), so a piece whose share went missing would show in every row that sees it."""
    dt = torch.bfloat16
    g = torch.Generator().manual_seed(H + 3 * hd + pieces)
    reqs = [(1000, 300), (0, 700), (2000, 40), (0, 3), (130, 1), (384, 129)]
    seqs_k = [torch.randn(c + n, KV, hd, generator=g).to(dt) for c, n in reqs]
    seqs_v = [torch.randn(c + n, KV, hd, generator=g).to(dt) for c, n in reqs]
    cu, positions, seq_of = [0], [], []
    for s, (c, n) in enumerate(reqs):
        cu.append(cu[-1] + n)
        positions += list(range(c, c + n))
        seq_of += [s] * n
    T = cu[-1]
    q = (torch.randn(T, H, hd, generator=g) * 1.5).to(dt)
    unit = torch.zeros(hd)
    unit[3] = 1.0
    seqs_k[1][37] = (unit * 12).to(dt)                    # key 37 of the request with 700 tokens ...
    q[cu[1] + 200:cu[1] + 700] += (unit * 12).to(dt)      # ... draws most of the weight of its later tokens
    total_pages = sum((c + n + page - 1) // page for c, n in reqs) + 3
    cache, tables = build_paged(seqs_k, seqs_v, page, total_pages, KV, hd, dt, g)
    for s, (c, n) in enumerate(reqs):                    # behind a request's last key: nothing that may reach the output
        if (c + n) % page:
            cache[tables[s, (c + n - 1) // page], :, :, (c + n) % page:] = float("nan")
    if window > 0:
        for s, (c, n) in enumerate(reqs):
            for slot in range(max(0, c - window + 1) // page):
                cache[tables[s, slot]] = float("nan")
                tables[s, slot] = -1
    scale = 1 / math.sqrt(hd)
    d = dev()
    q_lens = [n for _, n in reqs]
    cu_t = torch.tensor(cu, dtype=torch.int32, device=d)
    pos_t = torch.tensor(positions, dtype=torch.int32, device=d)
    tiles = ops.prefill_tiles_tcgen05(q_lens, H, KV)
    args = (q.view(T, -1).to(d), cache.to(d), tables.to(d), cu_t, pos_t, len(reqs), tiles, H, KV, hd, page, scale)
    whole = ops.attn_prefill_tcgen05(torch.zeros(T, H * hd, dtype=dt, device=d), *args, window=window)
    scratch = torch.full((ops.attn_prefill_tcgen05_scratch_floats(tiles, KV, hd, pieces),), float("nan"), device=d)
    counters = torch.full((tiles * KV,), -7, dtype=torch.int32, device=d)
    outs = []
    for _ in range(2):
        out = torch.full((T, H * hd), float("nan"), dtype=dt, device=d)
        ops.attn_prefill_tcgen05(out, *args, window=window, pieces=pieces, min_rounds=min_rounds, scratch=scratch, piece_counts=counters)
        outs.append(out)
    ops.check_device_errors(d)
    keep = torch.tensor([n > 1 for s, (c, n) in enumerate(reqs) for _ in range(n)])      # single tokens are the decode kernel's
    assert torch.equal(outs[0][keep.to(d)], outs[1][keep.to(d)])
    got = outs[0].float().cpu().view(T, H, hd)[keep]
    ref = attention_ref(q, [seqs_k[s] for s in seq_of], [seqs_v[s] for s in seq_of], None, positions, H, KV, hd, scale, window)[keep]
    torch.testing.assert_close(got, rnd(ref, dt), atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(got, whole.float().cpu().view(T, H, hd)[keep], atol=1e-2, rtol=1e-2)
    if window == 0:
        rows = slice(cu[1] + 300, cu[1] + 700)
        weight = torch.softmax((seqs_k[1][:, 0].float() @ q[cu[1] + 650, 0].float()) * scale, 0)[37]
        assert weight > 0.5, "the planted key does not stand out"
        assert torch.isfinite(got).all() and (got[rows] - rnd(ref, dt)[rows]).abs().max() < 2e-2


@pytest.mark.parametrize("seed", [0, 1, 2, 3, 4, 5])
def test_tcgen05_prefill_pieces_at_random_shapes(ops, seed):
    """Random requests (tokens in the cache, tokens in the step), heads, pages, windows, piece counts and piece lengths:
    the rows that come out of the pieces equal, within rounding, the rows of one block per query block."""
    import random
    rng = random.Random(seed)
    dt = torch.bfloat16
    g = torch.Generator().manual_seed(100 + seed)
    H, KV = rng.choice([(4, 2), (6, 1), (8, 8), (16, 8), (10, 2)])
    hd, page = rng.choice([64, 128]), rng.choice([16, 32, 64])
    window = rng.choice([0, 0, 400, 1100])
    pieces, min_rounds = rng.randint(2, 8), rng.randint(1, 3)
    reqs = [(rng.choice([0, rng.randint(1, 2500)]), rng.randint(2, 400)) for _ in range(rng.randint(2, 5))]
    seqs_k = [torch.randn(c + n, KV, hd, generator=g).to(dt) for c, n in reqs]
    seqs_v = [torch.randn(c + n, KV, hd, generator=g).to(dt) for c, n in reqs]
    cu, positions = [0], []
    for c, n in reqs:
        cu.append(cu[-1] + n)
        positions += list(range(c, c + n))
    T = cu[-1]
    q = (torch.randn(T, H, hd, generator=g) * 1.5).to(dt)
    total_pages = sum((c + n + page - 1) // page for c, n in reqs) + 3
    cache, tables = build_paged(seqs_k, seqs_v, page, total_pages, KV, hd, dt, g)
    for s, (c, n) in enumerate(reqs):
        if (c + n) % page:
            cache[tables[s, (c + n - 1) // page], :, :, (c + n) % page:] = float("nan")
        if window > 0:
            for slot in range(max(0, c - window + 1) // page):
                cache[tables[s, slot]] = float("nan")
                tables[s, slot] = -1
    d = dev()
    scale = 1 / math.sqrt(hd)
    q_lens = [n for _, n in reqs]
    tiles = ops.prefill_tiles_tcgen05(q_lens, H, KV)
    args = (q.view(T, -1).to(d), cache.to(d), tables.to(d), torch.tensor(cu, dtype=torch.int32, device=d),
            torch.tensor(positions, dtype=torch.int32, device=d), len(reqs), tiles, H, KV, hd, page, scale)
    whole = ops.attn_prefill_tcgen05(torch.full((T, H * hd), float("nan"), dtype=dt, device=d), *args, window=window)
    scratch = torch.full((ops.attn_prefill_tcgen05_scratch_floats(tiles, KV, hd, pieces),), float("nan"), device=d)
    counts = torch.full((tiles * KV,), -3, dtype=torch.int32, device=d)
    cut = ops.attn_prefill_tcgen05(torch.full((T, H * hd), float("nan"), dtype=dt, device=d), *args, window=window,
                                   pieces=pieces, min_rounds=min_rounds, scratch=scratch, piece_counts=counts)
    ops.check_device_errors(d)
    assert torch.isfinite(whole.float()).all() and torch.isfinite(cut.float()).all()
    torch.testing.assert_close(cut.float(), whole.float(), atol=1e-2, rtol=1e-2)
    assert int(counts.max()) <= pieces and int(counts.min()) >= 1


@pytest.mark.parametrize("H,KV,hd,page,window,norm,rope", [(16, 8, 128, 32, 0, True, True), (6, 2, 64, 16, 0, True, True),
                                                          (16, 1, 128, 16, 0, False, True), (4, 4, 64, 64, 70, True, False)])
def test_decode_attention_from_the_projection(ops, H, KV, hd, page, window, norm, rope):
    """Norm, rotation, cache write and attention of decoded tokens in one kernel against the three kernels it replaces:
    the same outputs and the same cache contents, at contexts that put the new token at the start, in the middle and at
    the end of a tile and of a page, for several split counts."""
    dt = torch.bfloat16
    g = torch.Generator().manual_seed(H + hd + page)
    ctxs = [0, 1, 15, 16, 63, 64, 65, 127, 500, 1000]             # tokens already in the cache, one new token each
    S = len(ctxs)
    seqs_k = [torch.randn(c + 1, KV, hd, generator=g).to(dt) for c in ctxs]
    seqs_v = [torch.randn(c + 1, KV, hd, generator=g).to(dt) for c in ctxs]
    total_pages = sum((c + 1 + page - 1) // page for c in ctxs) + 2
    cache, tables = build_paged(seqs_k, seqs_v, page, total_pages, KV, hd, dt, g)
    d = dev()
    qkv = (torch.randn(S, (H + 2 * KV) * hd, generator=g) * 1.5).to(dt).to(d)
    qw = (1 + 0.2 * torch.randn(hd, generator=g)).to(d) if norm else None
    kw = (1 + 0.2 * torch.randn(hd, generator=g)).to(d) if norm else None
    cos = sin = None
    if rope:
        inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2, dtype=torch.float64) / hd))
        ang = torch.arange(1100, dtype=torch.float64)[:, None] * inv[None, :]
        cos, sin = ang.cos().float().to(d), ang.sin().float().to(d)
    cu = torch.arange(S + 1, dtype=torch.int32, device=d)
    pos = torch.tensor(ctxs, dtype=torch.int32, device=d)
    slots = torch.tensor([int(tables[s, c // page]) * page + c % page for s, c in enumerate(ctxs)], dtype=torch.int32, device=d)
    scale = 1 / math.sqrt(hd)
    tables_d = tables.to(d)
    # the three kernels
    cache_a = cache.clone().to(d)
    q = torch.empty(S, H * hd, dtype=dt, device=d)
    ops.qk_norm_rope_kv(q, qkv, qw, kw, cos, sin, pos, slots, cache_a, H, KV, hd, page, 1e-6)
    want = torch.zeros(S, H * hd, dtype=dt, device=d)
    scratch = torch.zeros(ops.attn_decode_scratch_floats(S, KV, hd, 20), device=d)
    ops.attn_decode_bf16(want, q, cache_a, tables_d, cu, pos, S, H, KV, hd, page, scale, 3, scratch, window=window)
    for splits in (1, 3, 8, 20):
        cache_b = cache.clone().to(d)
        got = torch.zeros(S, H * hd, dtype=dt, device=d)
        ops.attn_decode_fused_bf16(got, qkv, cache_b, tables_d, cu, pos, slots, S, H, KV, hd, page, scale, splits, scratch,
                                   qw, kw, 1e-6, cos, sin, window=window)
        ops.check_device_errors(d)
        assert torch.equal(cache_a, cache_b)
        torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2e-2)


def test_tensor_core_attention_finds_one_far_key(ops):
    dt = torch.bfloat16
    H, KV, hd, page = 4, 2, 128, 16
    g = torch.Generator().manual_seed(5)
    n = 1500
    k = torch.randn(n, KV, hd, generator=g) * 0.1
    v = torch.randn(n, KV, hd, generator=g)
    q = torch.randn(2, H, hd, generator=g)          # token 0: single decoded token of request 0; token 1.. a portion of request 1
    far = 70
    k[far, 0] = q[0, 1] * 2.0                         # head 1 (kv head 0) of the decoded token must return v[far, 0]
    cache, tables = build_paged([k.to(dt), k.to(dt)], [v.to(dt), v.to(dt)], page, 200, KV, hd, dt, g)
    d = dev()
    cu = torch.tensor([0, 1, 3], dtype=torch.int32, device=d)
    qq = torch.cat([q[:1], q[1:2], q[:1]]).to(dt)     # request 1 brings two tokens at positions n-2, n-1; its last equals token 0
    pos = torch.tensor([n - 1, n - 2, n - 1], dtype=torch.int32, device=d)
    out = torch.zeros(3, H * hd, dtype=dt, device=d)
    ops.attn_prefill_tcgen05(out, qq.view(3, -1).to(d), cache.to(d), tables.to(d), cu, pos, 2, ops.prefill_tiles_tcgen05([1, 2], H, KV),
                             H, KV, hd, page, 1 / math.sqrt(hd))
    scratch = torch.zeros(ops.attn_decode_scratch_floats(2, KV, hd, 5), device=d)
    ops.attn_decode_bf16(out, qq.view(3, -1).to(d), cache.to(d), tables.to(d), cu, pos, 2, H, KV, hd, page, 1 / math.sqrt(hd), 5, scratch)
    o = out.float().cpu().view(3, H, hd)
    want = v[far, 0].to(dt).float()
    torch.testing.assert_close(o[0, 1], want, atol=3e-2, rtol=3e-2)      # decode kernel
    torch.testing.assert_close(o[2, 1], want, atol=3e-2, rtol=3e-2)      # prefill kernel, same query
    ops.check_device_errors(d)


def test_tensor_core_attention_refuses_what_it_does_not_cover(ops):
    d = dev()
    z = torch.zeros(1, 2 * 32, dtype=torch.bfloat16, device=d)
    i = torch.zeros(2, dtype=torch.int32, device=d)
    with pytest.raises(ops.KernelError, match="does not cover"):
        ops.attn_prefill_bf16(z, z, torch.zeros(2, 2, 1, 16, 32, dtype=torch.bfloat16, device=d), i.view(1, 2), i, i, 1, 1, 2, 1, 32, 16, 0.1)
    assert not ops.fast_attention_supported(torch.float32, 4, 2, 128) and not ops.fast_attention_supported(torch.bfloat16, 4, 2, 96)
    z = torch.zeros(1, 2 * 64, dtype=torch.bfloat16, device=d)
    with pytest.raises(ops.KernelError, match="scratch"):
        ops.attn_decode_bf16(z, z, torch.zeros(2, 2, 1, 16, 64, dtype=torch.bfloat16, device=d), i.view(1, 2), i, i, 1, 2, 1, 64, 16, 0.1, 4, None,
                             cluster_merge=False)


# ---- weight-streaming products for a few rows -----------------------------------------------------------------

@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(1024, 2048), (4096, 1024), (40, 72), (1000, 3064)])
def test_gemv_plain_norm_and_swiglu_forms(ops, M, N, K):
    dt = torch.bfloat16
    g = torch.Generator().manual_seed(M * 31 + N + K)
    d = dev()
    W = (torch.randn(N, K, generator=g) * 0.05).to(dt).to(d)
    x = torch.randn(M, K, generator=g).to(dt).to(d)
    assert ops.gemv_supported(dt, W, M) and not ops.gemv_supported(dt, W, 17) and not ops.gemv_supported(torch.float32, W, 1)
    big = torch.empty(8192, 2048, dtype=dt, device="meta")                       # 32 MB: more than 8 rows go to the library
    assert ops.gemv_supported(dt, big, 8) and not ops.gemv_supported(dt, big, 9)
    # plain
    out = torch.full((M, N), float("nan"), dtype=dt, device=d)
    ops.gemv_bf16(out, x, W, M)
    ref = (x.float() @ W.float().t())
    torch.testing.assert_close(out.float(), rnd(ref, dt), atol=2e-2, rtol=2e-2)
    # norm prologue with residual add
    delta = (torch.randn(M, K, generator=g) * 0.3).to(dt).to(d)
    nw = (1 + 0.2 * torch.randn(K, generator=g)).to(d)
    eps = 1e-5
    h2 = torch.zeros_like(x)
    ops.gemv_bf16(out, x, W, M, norm_weight=nw, eps=eps, delta=delta, resid_out=h2)
    s_ = rnd(x.float() + delta.float(), dt)
    assert torch.equal(h2.float(), s_)
    xn = rnd(rnd(s_ * torch.rsqrt((s_ * s_).mean(-1, keepdim=True) + eps), dt) * nw, dt)
    torch.testing.assert_close(out.float(), rnd(xn @ W.float().t(), dt), atol=3e-2, rtol=3e-2)
    # norm prologue without add leaves the residual alone; SwiGLU epilogue
    out2 = torch.full((M, N // 2), float("nan"), dtype=dt, device=d)
    ops.gemv_bf16(out2, x, W, M, norm_weight=nw, eps=eps, swiglu=True)
    xf = x.float()
    xn = rnd(rnd(xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + eps), dt) * nw, dt)
    gu = rnd(xn @ W.float().t(), dt)
    gate, up = gu[:, :N // 2], gu[:, N // 2:]
    torch.testing.assert_close(out2.float(), rnd(rnd(gate / (1 + torch.exp(-gate)), dt) * up, dt), atol=3e-2, rtol=3e-2)
    with pytest.raises(ops.KernelError, match="resid_out"):
        ops.gemv_bf16(out, x, W, M, norm_weight=nw, eps=eps, delta=delta, resid_out=x)


@pytest.mark.parametrize("dependent", [True, False])
@pytest.mark.parametrize("M", [1, 3, 8, 9, 13, 16])
@pytest.mark.parametrize("N,K", [(1024, 2048), (4096, 1024), (6144, 1024), (1024, 3072), (40, 72), (1000, 3064), (3, 8), (302, 40)])
def test_gemv_stream_forms(ops, M, N, K, dependent):
    """The product that fetches its block's weights by bulk copy ahead of its dependency (one block per SM): plain, with the
    norm prologue and residual add, with the SwiGLU epilogue; one and two groups of eight activation rows; row counts per
    block that are no multiple of a tile, inner sizes that are no multiple of 32; twice in a row; with and without the dependent-launch attribute; against float32."""
    dt = torch.bfloat16
    g = torch.Generator().manual_seed(M * 37 + N + K)
    d = dev()
    W = (torch.randn(N, K, generator=g) * 0.05).to(dt).to(d)
    assert ops.gemv_stream_supported(dt, W, M) and not ops.gemv_stream_supported(dt, W, 17)
    assert not ops.gemv_stream_supported(torch.float32, W, 1)
    assert not ops.gemv_stream_supported(dt, torch.empty(8192, 4096, dtype=dt, device="meta"), 1)    # 64 MB: not in one piece
    for rep in range(2):
        x = torch.randn(M, K, generator=g).to(dt).to(d)
        out = torch.full((M, N), float("nan"), dtype=dt, device=d)
        ops.gemv_stream_bf16(out, x, W, M, dependent=dependent, prefetch=W if rep else None, late_trigger=bool(rep))
        torch.testing.assert_close(out.float(), rnd(x.float() @ W.float().t(), dt), atol=2e-2, rtol=2e-2)
        # the residual sum folded into the store, in place: exactly rnd(h + y) for the y the kernel has just produced
        h = torch.randn(M, N, generator=g).to(dt).to(d)
        want = rnd(h.float() + out.float(), dt)
        ops.gemv_stream_bf16(h, x, W, M, dependent=dependent, add_to=h)
        assert torch.equal(h.float(), want)
        delta = (torch.randn(M, K, generator=g) * 0.3).to(dt).to(d)
        nw = (1 + 0.2 * torch.randn(K, generator=g)).to(d)
        eps = 1e-5
        h2 = torch.zeros_like(x)
        ops.gemv_stream_bf16(out, x, W, M, norm_weight=nw, eps=eps, delta=delta, resid_out=h2, dependent=dependent)
        s_ = rnd(x.float() + delta.float(), dt)
        assert torch.equal(h2.float(), s_)
        xn = rnd(rnd(s_ * torch.rsqrt((s_ * s_).mean(-1, keepdim=True) + eps), dt) * nw, dt)
        torch.testing.assert_close(out.float(), rnd(xn @ W.float().t(), dt), atol=3e-2, rtol=3e-2)
        if N % 2 == 0:
            out2 = torch.full((M, N // 2), float("nan"), dtype=dt, device=d)
            ops.gemv_stream_bf16(out2, x, W, M, norm_weight=nw, eps=eps, swiglu=True, dependent=dependent)
            xf = x.float()
            xn = rnd(rnd(xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + eps), dt) * nw, dt)
            gu = rnd(xn @ W.float().t(), dt)
            gate, up = gu[:, :N // 2], gu[:, N // 2:]
            torch.testing.assert_close(out2.float(), rnd(rnd(gate / (1 + torch.exp(-gate)), dt) * up, dt), atol=3e-2, rtol=3e-2)
    ops.check_device_errors(d)


@pytest.mark.parametrize("M,N,K", [(1, 200, 1000), (5, 128, 512), (8, 1031, 2056), (3, 4096, 4096)])
def test_split_k_weight_streaming_product(ops, M, N, K):
    """The product for large weights (inner dimension split over blocks, last block adds the parts) at sizes that are no
    multiples of its tiles, twice in a row (the counters must be back at zero), against float32."""
    g = torch.Generator().manual_seed(M * 1000 + N + K)
    W = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16)
    for rep in range(2):
        x = torch.randn(M, K, generator=g).to(torch.bfloat16)
        out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev())
        ops.gemv_splitk_bf16(out, x.to(dev()), W.to(dev()), M)
        ref = x.float() @ W.float().t()
        torch.testing.assert_close(out.float().cpu(), rnd(ref, torch.bfloat16), atol=2e-2, rtol=2e-2)
    ops.check_device_errors(dev())


# ---- tcgen05 matrix product -----------------------------------------------------------------------------------

@pytest.mark.parametrize("M,N,K,tile_n", [(128, 128, 64, 128), (2048, 1024, 2048, 128), (300, 520, 200, 128), (1, 8, 8, 128),
                                          (257, 4096, 1024, 256), (129, 264, 3072, 256), (2048, 6144, 1024, 256),
                                          (2100, 4104, 136, 128), (5000, 2560, 72, 256)])
def test_tcgen05_gemm_against_float32(ops, M, N, K, tile_n):
    """One tile, fewer tiles than SMs, and several tiles per block (the kernel is persistent: a block's tiles alternate
    between two accumulators and share one ring of stages), with edges in every dimension."""
    g = torch.Generator().manual_seed(M + N + K)
    d = dev()
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(d)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(d)
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=d)
    ops.gemm_bf16_tcgen05(out, x, w, tile_n=tile_n)
    ops.check_device_errors(d)
    ref = x.float() @ w.float().t()
    torch.testing.assert_close(out.float(), rnd(ref, torch.bfloat16), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("M,N,K,tile_n", [(128, 128, 64, 128), (300, 520, 200, 128), (2048, 1024, 3072, 128), (2500, 4096, 264, 256)])
def test_tcgen05_gemm_with_residual_epilogue(ops, M, N, K, tile_n):
    """out = round(x W^T) + residual, in place over the residual: what the norm after an attention or feed-forward output
    product would otherwise add."""
    dt = torch.bfloat16
    g = torch.Generator().manual_seed(M + N + K + 1)
    d = dev()
    x = torch.randn(M, K, generator=g).to(dt).to(d)
    w = (torch.randn(N, K, generator=g) * 0.05).to(dt).to(d)
    resid = torch.randn(M, N, generator=g).to(dt).to(d)
    ref = rnd(rnd(x.float() @ w.float().t(), dt) + resid.float(), dt)
    out = resid.clone()
    ops.gemm_bf16_tcgen05(out, x, w, tile_n=tile_n, resid=out)
    other = torch.full((M, N), float("nan"), dtype=dt, device=d)
    ops.gemm_bf16_tcgen05(other, x, w, tile_n=tile_n, resid=resid)
    ops.check_device_errors(d)
    assert torch.equal(out, other)
    torch.testing.assert_close(out.float(), ref, atol=3e-2, rtol=2e-2)


@pytest.mark.parametrize("M,I,K", [(128, 128, 64), (2048, 3072, 1024), (77, 200, 136), (3000, 1544, 200)])
def test_tcgen05_gemm_with_swiglu_epilogue(ops, M, I, K):
    dt = torch.bfloat16
    g = torch.Generator().manual_seed(M + I + K)
    d = dev()
    x = torch.randn(M, K, generator=g).to(dt).to(d)
    w = (torch.randn(2 * I, K, generator=g) * 0.08).to(dt).to(d)
    out = torch.full((M, I), float("nan"), dtype=dt, device=d)
    ops.gemm_bf16_tcgen05(out, x, w, swiglu=True)
    ops.check_device_errors(d)
    gu = rnd(x.float() @ w.float().t(), dt)
    gate, up = gu[:, :I], gu[:, I:]
    torch.testing.assert_close(out.float(), rnd(rnd(gate / (1 + torch.exp(-gate)), dt) * up, dt), atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("M,N,K", [(1, 200, 1000), (5, 128, 512), (8, 1031, 2056), (3, 4096, 4096), (8, 6144, 4096), (2, 300, 12288),
                                   (7, 16, 8), (4, 149, 1024), (8, 2368, 1032)])
def test_ring_buffered_streaming_product(ops, M, N, K):
    """The product for large weights (one block per SM, its rows through a ring of bulk copies): row counts that do not
    divide among the SMs, inner sizes that are no multiple of a chunk, fewer rows than SMs; twice in a row; against float32."""
    g = torch.Generator().manual_seed(M * 1000 + N + K)
    W = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(dev())
    assert ops.gemv_ring_supported(torch.bfloat16, W, M) and not ops.gemv_ring_supported(torch.bfloat16, W, 9)
    for rep in range(2):
        x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(dev())
        out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev())
        ops.gemv_ring_bf16(out, x, W, M, dependent=bool(rep))
        ref = x.float() @ W.float().t()
        torch.testing.assert_close(out.float(), rnd(ref, torch.bfloat16), atol=2e-2, rtol=2e-2)
    ops.check_device_errors(dev())


# ---- a bounded wait that runs out ------------------------------------------------------------------------------------

def test_a_wait_that_runs_out_is_reported_and_the_kernel_ends(ops):
    """Every wait on a barrier inside the package's kernels is bounded by a cycle count.  Here a block waits on a barrier
    that nothing arrives on, with a limit of about a millisecond: the kernel returns, the error word says 5, the error
    is raised as text on the host and cleared, and the device goes on working."""
    d = dev()
    ops.check_device_errors(d)
    assert ops.selftest_wait_runs_out(2_000_000) == 1
    with pytest.raises(ops.KernelError, match="bounded wait"):
        ops.check_device_errors(d)
    ops.check_device_errors(d)                                   # cleared by the report
    a = torch.ones(5, 8, dtype=torch.float32, device=d)
    ops.add_(a, a.clone())
    assert float(a.sum()) == 80.0
