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
