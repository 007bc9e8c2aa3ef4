"""The Qwen3-0.6B shape (28 layers, hidden 1024, 16/8 heads of 128, intermediate 3072, vocabulary 151936, tied) with
random weights: the engine in float32 and in bfloat16 against the plain implementation, on a prompt that is cut
into portions and then decoded token by token.  This is the size at which the tensor-core attention kernels, the
weight-streaming products and the chunked sampler run; the tiny models use the general kernels."""
import os

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
import tiny_models

pytestmark = pytest.mark.gpu

SHAPE = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=1024, num_hidden_layers=28,
             num_attention_heads=16, num_key_value_heads=8, head_dim=128, intermediate_size=3072, vocab_size=151936,
             rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=40960)


@pytest.fixture(scope="module")
def model_0p6b(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("qwen3_0p6b") / "m")
    return tiny_models.write_model(d, SHAPE, seed=0, std=0.02, spread=0.1)


def run_cut(model_dir, dtype, toks, cuts, decode_from):
    from cppvllm_b200.engine.runner import ModelRunner, StepEntry
    r = ModelRunner(model_dir, dtype=dtype, page_size=32, num_pages=16, max_step_tokens=256, max_seqs=4, max_model_len=256)
    r.cache.admit("a")
    r.cache.reserve("a", len(toks))
    rows, pos = [], 0
    for n in cuts:
        rows.append(r.step([StepEntry("a", toks[pos:pos + n], pos, list(range(n)))]).cpu().clone())
        pos += n
    assert pos == decode_from
    while pos < len(toks):
        rows.append(r.step([StepEntry("a", toks[pos:pos + 1], pos, [0])]).cpu().clone())
        pos += 1
    r.check_errors()
    assert r.stats["graph_steps"] == len(toks) - decode_from
    return torch.cat(rows)


def test_engine_matches_the_plain_implementation_at_the_0p6b_shape(model_0p6b):
    toks = tiny_models.random_tokens(10000, 96, 5)
    ref32 = plain.forward(model_0p6b, toks, "float32")
    scale = float(ref32.abs().max())
    got32 = run_cut(model_0p6b, torch.float32, toks, (40, 2, 30), 72)
    err32 = float((got32 - ref32).abs().max()) / scale
    assert err32 < 2e-5, f"float32 engine is {err32:.2e} of the largest logit away from the plain implementation"
    got16 = run_cut(model_0p6b, torch.bfloat16, toks, (40, 2, 30), 72)
    ref16 = plain.forward(model_0p6b, toks, "bfloat16")
    noise = float((ref16 - ref32).abs().max()) / scale              # what bfloat16 rounding alone does at this depth
    err16 = float((got16 - ref16).abs().max()) / scale
    assert err16 < max(2e-2, 1.5 * noise), f"bfloat16 engine {err16:.2e} vs rounding noise {noise:.2e}"
    assert float((got16 - ref32).abs().max()) / scale < 4e-2 + 2 * noise
    # most arg-maxima agree (random weights give flat logits, so near-ties are common; a wrong cache would agree nowhere)
    agree = (got16.argmax(-1) == ref32.argmax(-1)).float().mean().item()
    assert agree > 0.5


# ---- the four cuttings and larger decode batches at the layer sizes of Qwen3-0.6B -----------------------------------
# 4 of the 28 layers and a vocabulary of 32,003 instead of 151,936 (the plain implementation runs on the CPU; the layers'
# own sizes, which decide the kernels, are the model's: hidden 1024, 16 query and 8 key/value heads of 128, intermediate
# 3072).  Prompts of 300 to 700 tokens: the tensor-core prompt attention walks several key tiles and pages, the decode
# attention runs its splits over hundreds of keys.

SHAPE_4L = dict(SHAPE, num_hidden_layers=4, vocab_size=32003)


@pytest.fixture(scope="module")
def model_4l(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("qwen3_0p6b_4l") / "m")
    return tiny_models.write_model(d, SHAPE_4L, seed=1, std=0.02, spread=0.1)


def _check(rows, reqs, model_dir, dtype, want_rows):
    """rows: {(request, position): logits}; the plain implementation computes logits at the wanted positions only."""
    act = "float32" if dtype == torch.float32 else "bfloat16"
    c, w = plain.read_config(model_dir), plain.read_weights(model_dir)
    worst = 0.0
    for rid, toks in reqs.items():
        pos = sorted(p for (r, p) in rows if r == rid)
        assert pos == sorted(want_rows[rid]), rid
        ref = plain.forward(model_dir, toks, act, weights=w, cfg=c, rows=pos)
        scale = max(1.0, float(ref.abs().max()))
        limit = 2e-5 if dtype == torch.float32 else 2e-2
        if dtype == torch.bfloat16:
            ref32 = plain.forward(model_dir, toks, "float32", weights=w, cfg=c, rows=pos)
            limit = max(limit, 1.5 * float((ref - ref32).abs().max()) / scale)       # what bfloat16 rounding alone does
        for i, p_ in enumerate(pos):
            err = float(np.abs(rows[(rid, p_)] - ref[i].numpy()).max()) / scale
            assert err <= limit, f"request {rid} position {p_}: {err:.2e} of the largest logit (limit {limit:.1e})"
            worst = max(worst, err)
    return worst


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_four_cuttings_at_the_0p6b_layer_sizes(model_4l, dtype):
    from cppvllm_b200.engine.runner import ModelRunner
    from test_trace_replay import mixed_trace
    from trace_util import TraceBuilder, needed_max_tokens, rows_by_position, run_trace_in_process
    lens = {"w": 333, "t": 300, "p": 421, "m0": 700, "m1": 305, "m2": 512, "m3": 390, "m4": 640, "m5": 450}
    reqs = {k: tiny_models.random_tokens(10000, n, 40 + i) for i, (k, n) in enumerate(lens.items())}
    # whole (logits at a spread of positions: all of them would be 333 rows of 32,003); tail one by one; portions
    tb = TraceBuilder()
    tb.add([("w", reqs["w"], list(range(0, 333, 7)) + [332])], end=["w"])
    tb.add([("t", reqs["t"][:268], [0, 100, 267])])
    for i in range(268, 300):
        tb.add([("t", reqs["t"][i:i + 1], [0])], end=["t"] if i == 299 else [])
    pos = 0
    for n in (130, 2, 65, 3, 127, 2, 92):
        tb.add([("p", reqs["p"][pos:pos + n], [0, n - 1])], end=["p"] if pos + n == 421 else [])
        pos += n
    assert pos == 421
    single = tb.steps
    # mixed: four live requests, portions beside decoded tokens, a pool that holds less than all of them
    mixed = mixed_trace({k: v for k, v in reqs.items() if k.startswith("m")}, prefill_sizes=(130, 2, 257, 64, 3, 200), tail=24).steps
    for st in mixed:                                              # fewer rows: the last of a portion, every decoded token
        for e in st["entries"]:
            e["want"] = [len(e["tokens"]) - 1]
    pool = needed_max_tokens(mixed)
    assert pool < sum((lens[k] + 63) // 64 * 64 for k in lens if k.startswith("m"))
    r = ModelRunner(model_4l, dtype=dtype, page_size=32, num_pages=pool // 32, max_step_tokens=2048, max_seqs=8, max_model_len=1024)
    want = {}
    rows = {}
    for steps in (single, mixed):
        out = run_trace_in_process(r, steps)
        got = rows_by_position(steps, out)
        rows.update(got)
    for (rid, p_) in rows:
        want.setdefault(rid, []).append(p_)
    assert set(want) == set(reqs)
    _check(rows, reqs, model_4l, dtype, want)
    assert r.stats["graph_steps"] > 20                           # the decoded tokens of "t" replayed captured graphs
    r.cache.check_invariants()


def scale_of(t):
    return max(1.0, float(t.abs().max()))


def test_a_late_portion_attended_in_pieces_matches_the_whole_prompt(model_4l, monkeypatch):
    """A portion of a few hundred tokens behind two thousand cached ones is few query blocks with many key tiles each: the
    tensor-core attention shares each block's tiles out among several blocks and adds their shares up.  The same prompt
    in one step is many blocks and no pieces.  Both against the plain implementation, and against each other."""
    from cppvllm_b200.csrc import ops
    from cppvllm_b200.engine.runner import ModelRunner, StepEntry
    toks = tiny_models.random_tokens(10000, 2600, 77)
    rows = [2048, 2049, 2175, 2176, 2300, 2598, 2599]
    outs, used, seen = [], [], []
    real = ops.attn_prefill_tcgen05

    def recording(*a, **kw):
        seen.append(kw.get("pieces", 1))
        return real(*a, **kw)
    monkeypatch.setattr(ops, "attn_prefill_tcgen05", recording)
    for cuts in ((2600,), (2048, 552)):
        seen.clear()
        r = ModelRunner(model_4l, dtype=torch.bfloat16, page_size=32, num_pages=96, max_step_tokens=4096, max_seqs=8,
                        max_model_len=4096)
        r.cache.admit("a")
        r.cache.reserve("a", len(toks))
        got, pos = {}, 0
        for n in cuts:
            want = [p_ - pos for p_ in rows if pos <= p_ < pos + n]
            out = r.step([StepEntry("a", toks[pos:pos + n], pos, want)]).float().cpu()
            got.update({pos + w: out[i] for i, w in enumerate(want)})
            pos += n
        r.check_errors()
        outs.append(torch.stack([got[p_] for p_ in rows]))
        used.append(max(seen))
    assert used[0] == 1 and used[1] >= 2, "the second cutting's last portion should have been attended in pieces"
    # the same cutting again, for other requests on the same runner: from the second time on a shape replays a captured
    # graph, in which the pieces are allowed for the longest context the model takes
    r.cache.release("a")
    before = r.stats["graph_steps"]
    for rid in ("b", "c"):
        r.cache.admit(rid)
        r.cache.reserve(rid, len(toks))
        r.step([StepEntry(rid, toks[:2048], 0, [0])])
        want = [p_ - 2048 for p_ in rows]
        again = r.step([StepEntry(rid, toks[2048:], 2048, want)]).float().cpu()
        r.check_errors()
        assert float((again - outs[1]).abs().max()) / scale_of(outs[1]) < 1e-3
        r.cache.release(rid)
    assert r.stats["graph_steps"] >= before + 2
    assert ops.prefill_pieces_tcgen05(ops.prefill_tiles_tcgen05([552], 16, 8), 8) >= 2
    c, w = plain.read_config(model_4l), plain.read_weights(model_4l)
    ref16 = plain.forward(model_4l, toks, "bfloat16", weights=w, cfg=c, rows=rows)
    ref32 = plain.forward(model_4l, toks, "float32", weights=w, cfg=c, rows=rows)
    scale = float(ref32.abs().max())
    limit = max(2e-2, 1.5 * float((ref16 - ref32).abs().max()) / scale)
    for got in outs:
        assert float((got - ref16).abs().max()) / scale <= limit
    assert float((outs[0] - outs[1]).abs().max()) / scale <= limit


@pytest.mark.parametrize("batch", [12, 20])
def test_decode_batches_beyond_eight_rows_at_the_0p6b_layer_sizes(model_4l, batch):
    """12 rows: the weight-streaming products in their 16-row form; 20 rows: the library's products; both through the
    decode graphs of their bucket.  bfloat16, six decoded tokens per request after prompts of 30 to 200 tokens."""
    from cppvllm_b200.engine.runner import ModelRunner, StepEntry
    rng = np.random.RandomState(batch)
    lens = [int(x) for x in rng.randint(30, 200, size=batch)]
    n_dec = 6
    reqs = {f"d{i}": tiny_models.random_tokens(10000, n + n_dec, 70 + i) for i, n in enumerate(lens)}
    r = ModelRunner(model_4l, dtype=torch.bfloat16, page_size=32, num_pages=batch * 8, max_step_tokens=4096, max_seqs=32,
                    max_model_len=256)
    for rid in reqs:
        r.cache.admit(rid)
        r.cache.reserve(rid, len(reqs[rid]))
    rows = {}
    logits = r.step([StepEntry(rid, reqs[rid][:n], 0, [n - 1]) for rid, n in zip(reqs, lens)]).float().cpu().numpy()
    for i, (rid, n) in enumerate(zip(reqs, lens)):
        rows[(rid, n - 1)] = logits[i].copy()
    for s in range(n_dec):
        logits = r.step([StepEntry(rid, reqs[rid][n + s:n + s + 1], n + s, [0]) for rid, n in zip(reqs, lens)]).float().cpu().numpy()
        for i, (rid, n) in enumerate(zip(reqs, lens)):
            rows[(rid, n + s)] = logits[i].copy()
    r.check_errors()
    assert r.stats["graph_steps"] == n_dec
    want = {rid: [n - 1 + s for s in range(n_dec + 1)] for rid, n in zip(reqs, lens)}
    _check(rows, reqs, model_4l, torch.bfloat16, want)
