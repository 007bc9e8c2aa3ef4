"""Two tiny Qwen3 configurations that differ in every size and option, and helpers to write their folders.

            layers hidden heads kv  head_dim  q width   inter vocab theta  eps   tied  max_pos  page
    tiny_a     2     64     4    2     16     64 = D     128   256  1e4    1e-6  yes    256     16
    tiny_b     3     96     6    2     32     192 != D   224   320  1e6    1e-5  no     512     32
Groups are 2 and 3; widths 96, 224 and 320 are no powers of two.  `*_sharp` variants scale the per-head norm
weights of q so that attention concentrates on few keys: a key read from a wrong page or a wrong position then
changes the logits by far more than rounding."""
import json
import os

import torch

TINY_A = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=64, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=128, vocab_size=256,
              rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=256)
TINY_B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=96, num_hidden_layers=3,
              num_attention_heads=6, num_key_value_heads=2, head_dim=32, intermediate_size=224, vocab_size=320,
              rope_parameters={"rope_theta": 1000000.0}, rms_norm_eps=1e-5, tie_word_embeddings=False,
              max_position_embeddings=512)

# head size 64 with a group of 3: the smallest shape that the tensor-core attention kernels take
TINY_C = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=80, num_hidden_layers=2,
              num_attention_heads=6, num_key_value_heads=2, head_dim=64, intermediate_size=144, vocab_size=200,
              rope_theta=50000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=512)

# sizes that fit no vector width: hidden 100 and intermediate 172 (rows of bf16 that are no multiple of 16 bytes),
# an odd vocabulary, head size 48 with a group of 3
TINY_D = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=100, num_hidden_layers=2,
              num_attention_heads=3, num_key_value_heads=1, head_dim=48, intermediate_size=172, vocab_size=257,
              rope_theta=20000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=300)

# name -> (config, seed, std, norm spread, page size)
SETUPS = {
    "tiny_a": (TINY_A, 0, 0.02, 0.1, 16),
    "tiny_b": (TINY_B, 1, 0.03, 0.2, 32),
    "tiny_c": (TINY_C, 2, 0.03, 0.1, 16),
    "tiny_d": (TINY_D, 3, 0.03, 0.1, 64),
}


def write_model(path, cfg, seed, std, spread, sharpen=0.0, store_dtype=torch.bfloat16):
    from cppvllm_b200.weights.random_init import random_tensors
    from cppvllm_b200.weights.safetensors_io import save_safetensors
    import cppvllm_b200.models  # noqa: F401
    os.makedirs(path, exist_ok=True)
    tensors = random_tensors(cfg, seed, std, spread, store_dtype)
    if sharpen:
        for k in list(tensors):
            if k.endswith("q_norm.weight"):
                tensors[k] = (tensors[k].float() * sharpen).to(store_dtype)
            if k.endswith("_proj.weight") or k.endswith("embed_tokens.weight"):
                tensors[k] = (tensors[k].float() * 3.0).to(store_dtype)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_safetensors(os.path.join(path, "model.safetensors"), tensors)
    return path


def write_all(base):
    out = {}
    for name, (cfg, seed, std, spread, page) in SETUPS.items():
        out[name] = write_model(os.path.join(base, name), cfg, seed, std, spread)
        out[name + "_sharp"] = write_model(os.path.join(base, name + "_sharp"), cfg, seed + 10, std, spread, sharpen=6.0)
    return out


def page_size(name):
    return SETUPS[name.replace("_sharp", "")][4]


def config(name):
    return SETUPS[name.replace("_sharp", "")][0]


def random_tokens(vocab, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
