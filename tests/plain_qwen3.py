"""Plain, slow implementation of the Qwen3 dense decoder, written from the reference's formulas.

Whole sequences, no cache, no batching, one function for each part, on the CPU.  It shares no code with the
package under test: it has its own config.json reading, its own safetensors reading (through the `safetensors`
library) and its own arithmetic.  The reference's model code cannot be imported or compiled on a machine
without a GPU (it needs libtorch with CUDA, its own CUDA kernels and FlashAttention fetched at configure time,
CMakeLists.txt:43-57; it has no CPU path and no 32-bit path), so this file rests on the formulas; each function
cites where the reference computes the same thing.

``act`` chooses the activation type ``T``: "float32" makes ``rnd`` the identity (the true 32-bit model);
"bfloat16" rounds to bfloat16 wherever the reference rounds to its activation type (kernels/fused_ops.cu:27),
with float32 arithmetic in between, matrix products included.
"""
from __future__ import annotations

import json
import math
import os

import torch


def rnd(x: torch.Tensor, act: str) -> torch.Tensor:
    """Round to the activation type and back (reference kernels/fused_ops.cu:27)."""
    return x.to(torch.bfloat16).to(torch.float32) if act == "bfloat16" else x


def read_config(model_dir: str) -> dict:
    """config.json keys and defaults as the reference parses them (config.h:34-59), plus a top-level rope_theta."""
    with open(os.path.join(model_dir, "config.json")) as f:
        j = json.load(f)
    c = {
        "D": j["hidden_size"], "L": j["num_hidden_layers"], "H": j["num_attention_heads"],
        "KV": j.get("num_key_value_heads", j["num_attention_heads"]),
        "V": j["vocab_size"], "I": j["intermediate_size"],
        "eps": j.get("rms_norm_eps", 1e-6), "max_pos": j.get("max_position_embeddings", 40960),
        "tie": j.get("tie_word_embeddings", False),
    }
    c["hd"] = j.get("head_dim", c["D"] // c["H"])
    theta = 1e6
    if "rope_parameters" in j and "rope_theta" in j["rope_parameters"]:
        theta = j["rope_parameters"]["rope_theta"]
    if "rope_theta" in j:
        theta = j["rope_theta"]
    c["theta"] = float(theta)
    return c


def read_weights(model_dir: str) -> dict:
    from safetensors import safe_open
    w = {}
    for fn in sorted(os.listdir(model_dir)):
        if fn.endswith(".safetensors"):
            with safe_open(os.path.join(model_dir, fn), "pt") as f:
                for k in f.keys():
                    w[k] = f.get_tensor(k).to(torch.float32)
    return w


def embedding(table: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
    """h[t] = embed[tokens[t]] (model/model_architecture.cpp:149)."""
    return table[tokens]


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float, act: str) -> torch.Tensor:
    """y = T( rnd(x * rsqrt(mean(x^2) + eps)) * w ) (kernels/fused_ops.cu:61-88)."""
    inv = torch.rsqrt((x * x).mean(-1, keepdim=True) + eps)
    return rnd(rnd(x * inv, act) * w, act)


def linear(x: torch.Tensor, w: torch.Tensor, act: str) -> torch.Tensor:
    """y = x W^T, no bias, float32 accumulation, result in T (at::linear, model_architecture.cpp:155,178,182,185)."""
    return rnd(x @ w.t(), act)


def rope_tables(hd: int, theta: float, max_pos: int):
    """inv_freq_i = theta^(-2i/hd); angles in float64, cos/sin stored float32 (model_architecture.cpp:67-75)."""
    idx = torch.arange(0, hd, 2, dtype=torch.float64)
    freqs = 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float64), idx / hd)
    ang = torch.outer(torch.arange(max_pos, dtype=torch.float64), freqs)
    return ang.cos().to(torch.float32), ang.sin().to(torch.float32)


def qk_norm(x: torch.Tensor, w: torch.Tensor, eps: float, act: str) -> torch.Tensor:
    """Per-head RMSNorm over head_dim with one weight vector for all heads:
    n = rnd( rnd(x * rsqrt(mean(x^2) + eps)) * w ) (kernels/fused_ops.cu:148-156).  x: [T, heads, hd]."""
    inv = torch.rsqrt((x * x).mean(-1, keepdim=True) + eps)
    return rnd(rnd(x * inv, act) * w, act)


def apply_rope(n: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, positions: torch.Tensor, act: str) -> torch.Tensor:
    """Rotate-half pairs (i, i + hd/2): out_i = n_i c - n_{i+hd/2} s; out_{i+hd/2} = n_{i+hd/2} c + n_i s
    (kernels/fused_ops.cu:157-166).  n: [T, heads, hd]; result rounded to T."""
    half = n.shape[-1] // 2
    c = cos[positions][:, None, :]
    s = sin[positions][:, None, :]
    a, b = n[..., :half], n[..., half:]
    return rnd(torch.cat([a * c - b * s, b * c + a * s], dim=-1), act)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, act: str) -> torch.Tensor:
    """Causal grouped-query attention over one whole sequence.  Query head h uses kv head h // (H // KV)
    (kernels/paged_attention.cu:117,142); s_j = q.k_j / sqrt(hd) for j <= t (model_architecture.cpp:134,147);
    softmax and the weighted sum in float32; output rounded to T.  q: [T, H, hd]; k, v: [T, KV, hd]."""
    T, H, hd = q.shape
    KV = k.shape[1]
    group = H // KV
    scale = 1.0 / math.sqrt(hd)
    out = torch.empty_like(q)
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for h in range(H):
        g = h // group
        s = (q[:, h, :] @ k[:, g, :].t()) * scale
        s = s.masked_fill(~mask, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ v[:, g, :]
    return rnd(out, act)


def swiglu(gate: torch.Tensor, up: torch.Tensor, act: str) -> torch.Tensor:
    """act = T( rnd(g / (1 + exp(-g))) * u ) (kernels/fused_ops.cu:210-220)."""
    return rnd(rnd(gate / (1.0 + torch.exp(-gate)), act) * up, act)


def lm_head(y: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """logits = float32(y W^T) (model_architecture.cpp:222-226); the float32 accumulators are kept unrounded."""
    return y @ w.t()


def forward(model_dir: str, tokens, act: str = "float32", weights: dict = None, cfg: dict = None, rows=None) -> torch.Tensor:
    """Logits [T, V] at every position of one whole sequence (model_architecture.cpp:130-191, 222-236); with `rows`,
    only at those positions (the reference, too, picks rows before the final norm, :232-234)."""
    c = cfg or read_config(model_dir)
    w = weights or read_weights(model_dir)
    if act == "bfloat16":
        w = {k: rnd(t, act) for k, t in w.items()}
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    T = tokens.shape[0]
    positions = torch.arange(T)
    cos, sin = rope_tables(c["hd"], c["theta"], max(c["max_pos"], T))
    H, KV, hd, eps = c["H"], c["KV"], c["hd"], c["eps"]

    h = embedding(w["model.embed_tokens.weight"], tokens)
    for l in range(c["L"]):
        p = f"model.layers.{l}."
        x = rms_norm(h, w[p + "input_layernorm.weight"], eps, act)
        q = linear(x, w[p + "self_attn.q_proj.weight"], act).view(T, H, hd)
        k = linear(x, w[p + "self_attn.k_proj.weight"], act).view(T, KV, hd)
        v = linear(x, w[p + "self_attn.v_proj.weight"], act).view(T, KV, hd)
        q = apply_rope(qk_norm(q, w[p + "self_attn.q_norm.weight"], eps, act), cos, sin, positions, act)
        k = apply_rope(qk_norm(k, w[p + "self_attn.k_norm.weight"], eps, act), cos, sin, positions, act)
        att = attention(q, k, v, act).reshape(T, H * hd)
        h = rnd(h + linear(att, w[p + "self_attn.o_proj.weight"], act), act)          # residual 1 (fused_ops.cu:70-87)
        x = rms_norm(h, w[p + "post_attention_layernorm.weight"], eps, act)
        g = linear(x, w[p + "mlp.gate_proj.weight"], act)
        u = linear(x, w[p + "mlp.up_proj.weight"], act)
        m = linear(swiglu(g, u, act), w[p + "mlp.down_proj.weight"], act)
        h = rnd(h + m, act)                                                            # residual 2 (:187-188)
    if rows is not None:
        h = h[torch.as_tensor(list(rows), dtype=torch.long)]
    y = rms_norm(h, w["model.norm.weight"], eps, act)
    head = w["model.embed_tokens.weight"] if c["tie"] else w["lm_head.weight"]
    return lm_head(y, head)


def greedy_generate(model_dir: str, prompt, n_new: int, act: str = "float32"):
    """Greedy continuation by re-running the whole sequence for every new token; ties go to the lowest index
    (kernels/fused_ops.cu:303-304)."""
    c, w = read_config(model_dir), read_weights(model_dir)
    toks = list(prompt)
    out = []
    for _ in range(n_new):
        logits = forward(model_dir, toks, act, weights=w, cfg=c)[-1]
        nxt = int(torch.argmax(logits))
        out.append(nxt)
        toks.append(nxt)
    return out
