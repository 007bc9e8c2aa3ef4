"""Checks of the plain implementation itself (CPU): it is the yardstick of every GPU test, so its own
properties are tested here, and it is compared once with a second restatement of the formulas in float64
numpy that handles one token at a time."""
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
import tiny_models


def numpy_forward(cfg, w, tokens):
    """Token-by-token float64 restatement: explicit loops over positions, heads and keys."""
    w = {k: v.double().numpy() for k, v in w.items()}
    D, H, KV, hd, eps = cfg["D"], cfg["H"], cfg["KV"], cfg["hd"], cfg["eps"]
    inv_freq = np.array([cfg["theta"] ** (-2.0 * i / hd) for i in range(hd // 2)])

    def norm(x, g):
        return x / math.sqrt(float(np.mean(x * x)) + eps) * g

    def rope(x, pos):
        out = x.copy()
        for i in range(hd // 2):
            c, s = math.cos(pos * inv_freq[i]), math.sin(pos * inv_freq[i])
            out[i] = x[i] * c - x[i + hd // 2] * s
            out[i + hd // 2] = x[i + hd // 2] * c + x[i] * s
        return out

    ks = [[] for _ in range(cfg["L"])]
    vs = [[] for _ in range(cfg["L"])]
    logits = []
    for pos, tok in enumerate(tokens):
        h = w["model.embed_tokens.weight"][tok].copy()
        for l in range(cfg["L"]):
            p = f"model.layers.{l}."
            x = norm(h, w[p + "input_layernorm.weight"])
            q = (w[p + "self_attn.q_proj.weight"] @ x).reshape(H, hd)
            k = (w[p + "self_attn.k_proj.weight"] @ x).reshape(KV, hd)
            v = (w[p + "self_attn.v_proj.weight"] @ x).reshape(KV, hd)
            q = np.stack([rope(norm(q[i], w[p + "self_attn.q_norm.weight"]), pos) for i in range(H)])
            k = np.stack([rope(norm(k[i], w[p + "self_attn.k_norm.weight"]), pos) for i in range(KV)])
            ks[l].append(k)
            vs[l].append(v)
            att = np.zeros((H, hd))
            for i in range(H):
                g = i // (H // KV)
                s = np.array([q[i] @ ks[l][j][g] / math.sqrt(hd) for j in range(pos + 1)])
                pr = np.exp(s - s.max())
                pr /= pr.sum()
                att[i] = sum(pr[j] * vs[l][j][g] for j in range(pos + 1))
            h = h + w[p + "self_attn.o_proj.weight"] @ att.reshape(-1)
            x = norm(h, w[p + "post_attention_layernorm.weight"])
            gate, up = w[p + "mlp.gate_proj.weight"] @ x, w[p + "mlp.up_proj.weight"] @ x
            h = h + w[p + "mlp.down_proj.weight"] @ (gate / (1 + np.exp(-gate)) * up)
        y = norm(h, w["model.norm.weight"])
        head = w["model.embed_tokens.weight"] if cfg["tie"] else w["lm_head.weight"]
        logits.append(head @ y)
    return np.stack(logits)


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_two_restatements_agree(model_dirs, name):
    d = model_dirs[name]
    cfg, w = plain.read_config(d), plain.read_weights(d)
    toks = tiny_models.random_tokens(cfg["V"], 19, 3)
    a = plain.forward(d, toks, "float32").numpy()
    b = numpy_forward(cfg, w, toks)
    assert np.abs(a - b).max() < 2e-5 * max(1.0, np.abs(b).max())


def test_config_reading(model_dirs):
    a, b = plain.read_config(model_dirs["tiny_a"]), plain.read_config(model_dirs["tiny_b"])
    assert (a["theta"], b["theta"], a["tie"], b["tie"], a["hd"], b["hd"]) == (1e4, 1e6, True, False, 16, 32)


def test_causality_and_prefix_property(model_dirs):
    d = model_dirs["tiny_b"]
    toks = tiny_models.random_tokens(320, 40, 1)
    full = plain.forward(d, toks)
    assert torch.allclose(plain.forward(d, toks[:25]), full[:25], atol=1e-6)
    other = toks[:30] + [(t + 1) % 320 for t in toks[30:]]
    assert torch.allclose(plain.forward(d, other)[:30], full[:30], atol=1e-6)
    assert not torch.allclose(plain.forward(d, other)[30:], full[30:], atol=1e-3)


def test_parts():
    x = torch.randn(5, 12)
    w = torch.rand(12) + 0.5
    y = plain.rms_norm(x, w, 1e-5, "float32")
    assert torch.allclose(y, x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5) * w, atol=1e-6)
    cos, sin = plain.rope_tables(8, 100.0, 16)
    n = torch.randn(16, 3, 8)
    r = plain.apply_rope(n, cos, sin, torch.arange(16), "float32")
    assert torch.allclose(r.norm(dim=-1), n.norm(dim=-1), atol=1e-5)            # a rotation keeps lengths
    assert torch.allclose(r[0], n[0])                                            # position 0: identity
    q, k = torch.randn(16, 1, 8), torch.randn(16, 1, 8)
    rq = plain.apply_rope(q, cos, sin, torch.arange(16), "float32")
    rk = plain.apply_rope(k.roll(1, 0), cos, sin, torch.arange(16), "float32")
    # scores depend on relative position only: shifting both by the same offset keeps q.k
    rq2 = plain.apply_rope(q[:8], cos, sin, torch.arange(3, 11), "float32")
    rk2 = plain.apply_rope(k[:8], cos, sin, torch.arange(3, 11), "float32")
    rq1 = plain.apply_rope(q[:8], cos, sin, torch.arange(0, 8), "float32")
    rk1 = plain.apply_rope(k[:8], cos, sin, torch.arange(0, 8), "float32")
    assert torch.allclose((rq1[5, 0] * rk1[2, 0]).sum(), (rq2[5, 0] * rk2[2, 0]).sum(), atol=1e-5)
    g, u = torch.randn(4, 6), torch.randn(4, 6)
    assert torch.allclose(plain.swiglu(g, u, "float32"), torch.nn.functional.silu(g) * u, atol=1e-6)
    # grouped heads: heads 0..2 of 6 read kv head 0
    qq, kk, vv = torch.randn(7, 6, 4), torch.randn(7, 2, 4), torch.randn(7, 2, 4)
    o = plain.attention(qq, kk, vv, "float32")
    o2 = plain.attention(qq, kk.repeat_interleave(3, 1), vv.repeat_interleave(3, 1), "float32")
    assert torch.allclose(o, o2, atol=1e-6)
    assert torch.allclose(o[0], vv[0].repeat_interleave(3, 0), atol=1e-6)       # first token sees only itself


def test_bfloat16_rounding_mode_stays_close(model_dirs):
    d = model_dirs["tiny_a"]
    toks = tiny_models.random_tokens(256, 33, 2)
    a, b = plain.forward(d, toks, "float32"), plain.forward(d, toks, "bfloat16")
    assert 0 < (a - b).abs().max() < 0.03 * a.abs().max()
    assert plain.greedy_generate(d, toks[:5], 3) == plain.greedy_generate(d, toks[:5], 3)
