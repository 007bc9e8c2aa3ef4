"""Safetensors reading and writing, binding by name with one clear error, random-weights mode (CPU)."""
import json
import os
import struct

import pytest
import torch

import cppvllm_b200.models  # noqa: F401
import cppvllm_b200.parts  # noqa: F401
from cppvllm_b200.config.registry import resolve_architecture
from cppvllm_b200.parts.base import Runtime, Workspace
from cppvllm_b200.parts.model import CausalLM
from cppvllm_b200.weights.loader import WeightError, load_weights
from cppvllm_b200.weights.random_init import random_tensors, write_random_model
from cppvllm_b200.weights.safetensors_io import SafetensorsError, SafetensorsFile, save_safetensors
from tiny_models import TINY_A, TINY_B


def cpu_model(cfg, dtype=torch.float32):
    arch = resolve_architecture(cfg)
    cpu = torch.device("cpu")
    return CausalLM(arch.build_spec(arch.parse_config(cfg)), Runtime(cpu, dtype, Workspace(cpu, 0)))


def test_safetensors_round_trip_and_foreign_reader(tmp_path):
    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.arange(7, dtype=torch.int32), "c": torch.randn(4)}
    p = str(tmp_path / "x.safetensors")
    save_safetensors(p, t, {"k": "v"})
    with SafetensorsFile(p) as f:
        assert sorted(f.names()) == ["a", "b", "c"] and f.metadata == {"k": "v"}
        for k in t:
            assert f.dtype(k) == t[k].dtype and torch.equal(f.tensor(k), t[k])
    from safetensors import safe_open                       # an independent reader accepts the file
    with safe_open(p, "pt") as f:
        assert torch.equal(f.get_tensor("a"), t["a"])


def test_malformed_files_are_refused(tmp_path):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="does not fit"):
        SafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 4) + b"nope")
    with pytest.raises(SafetensorsError, match="not valid JSON"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)       # truncated data
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"w": {"dtype": "Q7", "shape": [1], "data_offsets": [0, 1]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0")
    with pytest.raises(SafetensorsError, match="unsupported dtype"):
        SafetensorsFile(str(p))
    with pytest.raises(SafetensorsError, match="cannot open"):
        SafetensorsFile(str(tmp_path / "missing.safetensors"))


def test_random_weights_are_a_function_of_seed_and_name(tmp_path):
    a1, a2, a3 = random_tensors(TINY_A, 0), random_tensors(TINY_A, 0), random_tensors(TINY_A, 1)
    assert a1.keys() == a2.keys()
    assert all(torch.equal(a1[k], a2[k]) for k in a1)
    assert not torch.equal(a1["model.embed_tokens.weight"], a3["model.embed_tokens.weight"])
    assert "lm_head.weight" not in a1 and "lm_head.weight" in random_tensors(TINY_B, 0)     # tied / untied
    w = a1["model.layers.0.input_layernorm.weight"].float()
    assert (w - 1).abs().max() <= 0.1 + 1e-2 and w.std() > 0.01
    e = random_tensors(TINY_A, 0, std=0.05)["model.embed_tokens.weight"].float()
    assert abs(e.std().item() - 0.05) < 0.005
    d = write_random_model(str(tmp_path / "m"), TINY_B, 3, std=0.03, norm_spread=0.2)
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    assert json.load(open(os.path.join(d, "config.json")))["hidden_size"] == 96


def test_loader_binds_and_converts(tmp_path):
    d = write_random_model(str(tmp_path / "m"), TINY_A, 0)
    m = cpu_model(TINY_A, torch.bfloat16)
    w = load_weights(m, d, "cpu", torch.bfloat16)
    assert w["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert w["model.norm.weight"].dtype == torch.float32                    # vectors reach kernels as float32
    w32 = load_weights(cpu_model(TINY_A), d, "cpu", torch.float32)
    assert w32["model.layers.1.mlp.down_proj.weight"].dtype == torch.float32
    assert torch.equal(w32["model.layers.1.mlp.down_proj.weight"], w["model.layers.1.mlp.down_proj.weight"].float())
    m.bind(w)
    assert m.head.weight is m.embedding.table                                # tied head shares the table
    assert m.blocks[0].mixer.w_qkv.shape == (4 * 16 + 2 * 2 * 16, 64)


def test_tensor_stored_in_32_bit_stays_so(tmp_path):
    d = write_random_model(str(tmp_path / "m"), TINY_A, 0, store_dtype=torch.float32)
    w = load_weights(cpu_model(TINY_A, torch.bfloat16), d, "cpu", torch.bfloat16)
    assert w["model.layers.0.self_attn.q_proj.weight"].dtype == torch.float32


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    t = random_tensors(TINY_B, 1)
    del t["model.layers.2.self_attn.k_norm.weight"]
    del t["lm_head.weight"]
    t["model.layers.7.extra.weight"] = torch.zeros(2)
    t["model.layers.0.mlp.up_proj.weight"] = torch.zeros(224, 95, dtype=torch.bfloat16)
    d = tmp_path / "m"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(TINY_B))
    save_safetensors(str(d / "model.safetensors"), t)
    with pytest.raises(WeightError) as ei:
        load_weights(cpu_model(TINY_B), str(d), "cpu", torch.float32)
    e = ei.value
    assert e.missing == ["lm_head.weight", "model.layers.2.self_attn.k_norm.weight"]
    assert e.unexpected == ["model.layers.7.extra.weight"]
    assert len(e.wrong_shape) == 1 and "up_proj" in e.wrong_shape[0] and "[224, 95]" in e.wrong_shape[0] and "[224, 96]" in e.wrong_shape[0]
    msg = str(e)
    assert "missing tensors (2)" in msg and "unexpected tensors (1)" in msg and "wrong shapes (1)" in msg


def test_tied_checkpoint_may_carry_its_own_head_and_duplicates_are_errors(tmp_path):
    t = random_tensors(TINY_A, 0)
    d = tmp_path / "m"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(TINY_A))
    t2 = dict(t, **{"lm_head.weight": t["model.embed_tokens.weight"].clone()})
    save_safetensors(str(d / "model.safetensors"), t2)
    load_weights(cpu_model(TINY_A), str(d), "cpu", torch.float32)            # ignorable, no error
    save_safetensors(str(d / "model-2.safetensors"), {"model.norm.weight": t["model.norm.weight"]})
    with pytest.raises(WeightError, match="occurs in both"):
        load_weights(cpu_model(TINY_A), str(d), "cpu", torch.float32)
    with pytest.raises(SafetensorsError, match="no .safetensors"):
        load_weights(cpu_model(TINY_A), str(tmp_path), "cpu", torch.float32)
