"""Configuration and registry (CPU)."""
import json

import pytest

import cppvllm_b200.models  # noqa: F401
from cppvllm_b200.config.engine_config import EngineConfig
from cppvllm_b200.config.model_config import ConfigError, Qwen3Config, read_config_json
from cppvllm_b200.config.registry import (register_architecture, registered_architectures, resolve_architecture,
                                          unregister_architecture)
from cppvllm_b200.models.qwen3 import build_qwen3_spec
from tiny_models import TINY_A, TINY_B


def test_keys_and_defaults_follow_the_reference():
    c = Qwen3Config.from_dict(dict(hidden_size=128, num_hidden_layers=2, num_attention_heads=8, vocab_size=100,
                                   intermediate_size=256))
    assert c.num_key_value_heads == 8 and c.head_dim == 16
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 1e6 and c.max_position_embeddings == 40960
    assert c.tie_word_embeddings is False and c.eos_token_ids == (151645,)


def test_every_size_comes_from_the_file():
    a, b = Qwen3Config.from_dict(TINY_A), Qwen3Config.from_dict(TINY_B)
    assert (a.hidden_size, a.num_hidden_layers, a.num_attention_heads, a.num_key_value_heads, a.head_dim) == (64, 2, 4, 2, 16)
    assert (b.hidden_size, b.num_hidden_layers, b.num_attention_heads, b.num_key_value_heads, b.head_dim) == (96, 3, 6, 2, 32)
    assert b.q_width == 192 != b.hidden_size and b.gqa_group == 3 and a.gqa_group == 2
    assert a.rope_theta == 1e4 and b.rope_theta == 1e6          # top-level key and rope_parameters
    assert a.rms_norm_eps == 1e-6 and b.rms_norm_eps == 1e-5
    assert a.tie_word_embeddings and not b.tie_word_embeddings


def test_rope_theta_top_level_wins_and_eos_forms():
    d = dict(TINY_A, rope_parameters={"rope_theta": 5.0}, rope_theta=7.0, eos_token_id=9)
    c = Qwen3Config.from_dict(d)
    assert c.rope_theta == 7.0 and c.eos_token_ids == (9,)
    assert Qwen3Config.from_dict(dict(TINY_A, eos_token_id=[3, 4])).eos_token_ids == (3, 4)


@pytest.mark.parametrize("key", ["hidden_size", "num_hidden_layers", "num_attention_heads", "vocab_size", "intermediate_size"])
def test_missing_required_key_is_named(key):
    d = dict(TINY_A)
    del d[key]
    with pytest.raises(ConfigError, match=key):
        Qwen3Config.from_dict(d)


def test_bad_values_are_refused():
    with pytest.raises(ConfigError, match="multiple"):
        Qwen3Config.from_dict(dict(TINY_A, num_key_value_heads=3))
    with pytest.raises(ConfigError, match="even"):
        Qwen3Config.from_dict(dict(TINY_A, head_dim=15))
    with pytest.raises(ConfigError, match="positive"):
        Qwen3Config.from_dict(dict(TINY_A, vocab_size=0))


def test_round_trip_through_json(tmp_path):
    c = Qwen3Config.from_dict(TINY_B)
    (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
    assert Qwen3Config.from_dict(read_config_json(str(tmp_path))) == c
    with pytest.raises(ConfigError, match="no config.json"):
        read_config_json(str(tmp_path / "nowhere"))


def test_registry_resolves_by_name_then_model_type():
    assert "Qwen3ForCausalLM" in registered_architectures()
    assert resolve_architecture({"architectures": ["Qwen3ForCausalLM"]}).name == "Qwen3ForCausalLM"
    assert resolve_architecture({"model_type": "qwen3"}).name == "Qwen3ForCausalLM"
    with pytest.raises(ConfigError, match="not registered.*Qwen3ForCausalLM"):
        resolve_architecture({"architectures": ["NopeForCausalLM"]})
    register_architecture("ToyArch", lambda d: d, lambda c: None, model_types=("toy",))
    try:
        assert resolve_architecture({"model_type": "toy"}).name == "ToyArch"
        with pytest.raises(ConfigError, match="names no architecture"):
            resolve_architecture({})
        with pytest.raises(ValueError, match="already registered"):
            register_architecture("ToyArch", None, None)
    finally:
        unregister_architecture("ToyArch")
    assert resolve_architecture({}).name == "Qwen3ForCausalLM"     # the only one registered


def test_spec_is_data_with_sizes_from_config():
    spec = build_qwen3_spec(Qwen3Config.from_dict(TINY_B))
    assert len(spec.layers) == 3 and spec.vocab_size == 320 and spec.hidden_size == 96
    m = spec.layers[1].mixer
    assert m.kind == "paged_attention" and m.prefix == "model.layers.1.self_attn."
    assert m.params["num_heads"] == 6 and m.params["num_kv_heads"] == 2 and m.params["head_dim"] == 32
    assert m.params["qk_norm_eps"] == 1e-5 and m.params["window"] == 0
    assert spec.layers[0].ffn.params == dict(hidden_size=96, intermediate_size=224)
    assert spec.positions["rope"].params["theta"] == 1e6
    assert spec.lm_head.names == {}                                       # untied
    tied = build_qwen3_spec(Qwen3Config.from_dict(TINY_A))
    assert tied.lm_head.names == {"weight": "model.embed_tokens.weight"}
    order = spec.resolved_run_order()
    assert [(e.layer, e.cache, e.writes_cache) for e in order] == [(0, 0, True), (1, 1, True), (2, 2, True)]


def test_run_order_checks():
    from cppvllm_b200.parts.spec import RunEntry
    spec = build_qwen3_spec(Qwen3Config.from_dict(TINY_A))
    spec.run_order = [RunEntry(0), RunEntry(0), RunEntry(1, cache=0, writes_cache=False)]
    with pytest.raises(ValueError, match="before any entry wrote"):
        spec.resolved_run_order()
    spec.run_order = [RunEntry(0, cache=0), RunEntry(1, cache=0, writes_cache=False), RunEntry(0)]
    assert [(e.layer, e.cache) for e in spec.resolved_run_order()] == [(0, 0), (1, 0), (0, 1)]
    spec.run_order = [RunEntry(5)]
    with pytest.raises(ValueError, match="names layer 5"):
        spec.resolved_run_order()


def test_engine_config_names_and_checks():
    e = EngineConfig(model_path="x")
    assert (e.max_num_batched_tokens, e.max_num_seqs, e.max_chunk_tokens, e.max_model_len) == (4096, 256, 1024, 4096)
    assert e.gpu_memory_utilization == 0.90 and e.num_kv_blocks == -1 and not e.enforce_eager and e.seed == 0
    with pytest.raises(ValueError, match="one GPU"):
        EngineConfig(tensor_parallel_size=2)
    with pytest.raises(ValueError, match="dtype"):
        EngineConfig(dtype="float16")
    with pytest.raises(ValueError, match="block_size"):
        EngineConfig(block_size=24)
