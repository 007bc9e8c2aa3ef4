"""Qwen3 dense (``Qwen3ForCausalLM``) as data: the typed configuration becomes a ``ModelSpec``.

Structure and tensor names follow the reference (model/model_architecture.cpp:77-120,130-191): a token
embedding, ``num_hidden_layers`` identical pre-norm blocks of grouped-query attention (per-head RMSNorm on q
and k, rotate-half rotary at ``rope_theta`` over the whole head, no biases, no window) and a SwiGLU
feed-forward, a final RMSNorm and an output head that is the embedding table when ``tie_word_embeddings``.
Every size below comes from the configuration.
"""
from __future__ import annotations

from ..config.model_config import Qwen3Config
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec


def build_qwen3_spec(cfg: Qwen3Config) -> ModelSpec:
    D, eps = cfg.hidden_size, cfg.rms_norm_eps
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        layers.append(LayerSpec(
            mixer=PartSpec("paged_attention", dict(
                hidden_size=D, num_heads=cfg.num_attention_heads, num_kv_heads=cfg.num_key_value_heads,
                head_dim=cfg.head_dim, qk_norm=True, qk_norm_eps=eps, window=0, position="rope"),
                prefix=p + "self_attn."),
            ffn=PartSpec("swiglu", dict(hidden_size=D, intermediate_size=cfg.intermediate_size), prefix=p + "mlp."),
            mixer_norm=PartSpec("rmsnorm", dict(size=D, eps=eps, buffer="normed"), prefix=p + "input_layernorm."),
            ffn_norm=PartSpec("rmsnorm", dict(size=D, eps=eps, buffer="normed"), prefix=p + "post_attention_layernorm."),
            block="prenorm"))
    head_names = {"weight": "model.embed_tokens.weight"} if cfg.tie_word_embeddings else {}
    return ModelSpec(
        architecture=cfg.architecture,
        hidden_size=D,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("token_embedding", dict(vocab_size=cfg.vocab_size, hidden_size=D), prefix="model.embed_tokens."),
        layers=layers,
        final_norm=PartSpec("rmsnorm", dict(size=D, eps=eps, buffer="head_normed"), prefix="model.norm."),
        lm_head=PartSpec("lm_head", dict(vocab_size=cfg.vocab_size, hidden_size=D), prefix="lm_head.", names=head_names),
        positions={"rope": PartSpec("rotary", dict(rotary_dim=cfg.head_dim, theta=cfg.rope_theta,
                                                   max_positions=cfg.max_position_embeddings, pairing="half"))},
        run_order=None,
        max_positions=cfg.max_position_embeddings,
        eos_token_ids=tuple(cfg.eos_token_ids),
    )


register_architecture("Qwen3ForCausalLM", Qwen3Config.from_dict, build_qwen3_spec, model_types=("qwen3",), replace=True)
