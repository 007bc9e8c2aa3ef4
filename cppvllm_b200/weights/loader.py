"""Binding of checkpoint tensors to a model by tensor name.

The model declares what it needs (``CausalLM.weight_specs()``: full Hugging Face tensor names with shapes
and roles).  The loader reads every ``*.safetensors`` of the folder (reference utils/tensor.h:50-62; a name that
occurs in two files is an error, tensor.h:57), compares names and shapes with the declaration and, if anything
is off, raises ONE ``WeightError`` that lists the missing tensors, the unexpected tensors and the tensors of
wrong shape.  (The reference surfaces a missing tensor as an anonymous ``out_of_range`` and checks no shapes,
model/model_architecture.cpp:78.)

Element types: matrices stored in bfloat16 stay bfloat16 under bfloat16 activations and are widened (exactly)
under float32 activations; a tensor stored in 32-bit floating point stays float32; 16-bit halves and 64-bit
floats are converted to the activation type; norm weights and other vectors are always handed to the kernels
as float32 (exact for bfloat16 storage); integer tables become int32.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..parts.base import WeightSpec
from .safetensors_io import SafetensorsError, SafetensorsFile, list_safetensors_files


class WeightError(ValueError):
    def __init__(self, model_dir: str, missing: List[str], unexpected: List[str], wrong_shape: List[str], other: List[str] = ()):
        self.missing, self.unexpected, self.wrong_shape, self.other = list(missing), list(unexpected), list(wrong_shape), list(other)
        lines = [f"checkpoint at {model_dir} does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(self.wrong_shape))
        if self.other:
            lines.append("  other: " + "; ".join(self.other))
        super().__init__("\n".join(lines))


def _convert(t: torch.Tensor, spec: WeightSpec, act_dtype: torch.dtype) -> torch.Tensor:
    if spec.role == "int_table":
        return t.to(torch.int32)
    if not t.dtype.is_floating_point:
        raise TypeError(f"stored as {t.dtype}, but a floating-point tensor is needed")
    if spec.role == "vector":
        return t.to(torch.float32)
    if t.dtype == torch.float32:
        return t                                   # stored in 32-bit: stays so
    return t.to(act_dtype)


def load_weights(model, model_dir: str, device, act_dtype: torch.dtype) -> Dict[str, torch.Tensor]:
    """Read, check and convert the tensors `model` declares; returns name -> tensor on `device`."""
    expected: Dict[str, WeightSpec] = model.weight_specs()
    ignorable = set(model.ignorable_weights()) if hasattr(model, "ignorable_weights") else set()
    files = [SafetensorsFile(p) for p in list_safetensors_files(model_dir)]
    try:
        where: Dict[str, SafetensorsFile] = {}
        other: List[str] = []
        for f in files:
            for name in f.names():
                if name in where:
                    other.append(f"tensor '{name}' occurs in both {where[name].path} and {f.path}")
                where[name] = f
        missing = sorted(n for n in expected if n not in where)
        unexpected = sorted(n for n in where if n not in expected and n not in ignorable)
        wrong = []
        for n, spec in expected.items():
            if n in where and tuple(where[n].shape(n)) != tuple(spec.shape):
                wrong.append(f"{n}: checkpoint {list(where[n].shape(n))}, model {list(spec.shape)}")
        for n, spec in expected.items():
            if n in where and spec.role != "int_table" and not where[n].dtype(n).is_floating_point:
                other.append(f"tensor '{n}' is stored as {where[n].dtype(n)}, not a floating-point type")
        if missing or unexpected or wrong or other:
            raise WeightError(model_dir, missing, unexpected, sorted(wrong), other)
        out = {}
        for n, spec in expected.items():
            out[n] = _convert(where[n].tensor(n), spec, act_dtype).contiguous().to(device)
        return out
    finally:
        for f in files:
            f.close()
