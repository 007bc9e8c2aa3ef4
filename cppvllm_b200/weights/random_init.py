"""Random-weights mode: writes a model folder (``config.json`` + ``model.safetensors``) from a configuration
and a seed, so that a random model takes the same path through the loader as a real checkpoint.  The reference
has no such mode.

Every tensor the architecture declares is drawn from its own generator, seeded by (seed, tensor name): the
values do not depend on the order of tensors.  Matrices and tables ~ N(0, std); norm weights ~ 1 + U(-spread,
spread).  Values are drawn in float32 and stored in `store_dtype` (bfloat16 by default).
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Any, Dict, Mapping

import torch

from ..config.registry import resolve_architecture
from ..parts.base import Runtime, Workspace
from ..parts.model import CausalLM
from .safetensors_io import save_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensors(config_dict: Mapping[str, Any], seed: int, std: float = 0.02, norm_spread: float = 0.1,
                   store_dtype: torch.dtype = torch.bfloat16) -> Dict[str, torch.Tensor]:
    arch = resolve_architecture(config_dict)
    cfg = arch.parse_config(config_dict)
    spec = arch.build_spec(cfg)
    cpu = torch.device("cpu")
    model = CausalLM(spec, Runtime(cpu, torch.float32, Workspace(cpu, 0)))
    out = {}
    for name, ws in sorted(model.weight_specs().items()):
        g = torch.Generator(device="cpu")
        g.manual_seed(_tensor_seed(seed, name))
        if ws.role == "int_table":
            out[name] = torch.randint(0, 2 ** 15, ws.shape, generator=g, dtype=torch.int32)
            continue
        if ws.init == "norm":
            t = 1.0 + (torch.rand(ws.shape, generator=g, dtype=torch.float32) * 2.0 - 1.0) * norm_spread
        else:
            t = torch.randn(ws.shape, generator=g, dtype=torch.float32) * std
        out[name] = t.to(store_dtype)
    return out


def write_random_model(model_dir: str, config_dict: Mapping[str, Any], seed: int, std: float = 0.02,
                       norm_spread: float = 0.1, store_dtype: torch.dtype = torch.bfloat16) -> str:
    """Create `model_dir` with config.json and model.safetensors; returns the folder."""
    os.makedirs(model_dir, exist_ok=True)
    tensors = random_tensors(config_dict, seed, std, norm_spread, store_dtype)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(dict(config_dict), f, indent=1)
    save_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                     metadata={"format": "pt", "seed": str(seed), "std": str(std), "norm_spread": str(norm_spread)})
    return model_dir
