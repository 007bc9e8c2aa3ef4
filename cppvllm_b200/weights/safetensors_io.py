"""Reader and writer for the ``.safetensors`` container.

Layout (as parsed by the reference, utils/safetensors.cpp:69-116): an unsigned 64-bit little-endian header
length, a JSON header ``{name: {"dtype", "shape", "data_offsets": [begin, end]}}`` whose offsets are relative
to the end of the header, an optional ``__metadata__`` entry, then the raw little-endian tensor bytes.
Unlike the reference's reader (which leaves open/mmap results, dtype strings and name look-ups unchecked,
safetensors.cpp:30-38,60-63,95-101), every malformed input raises ``SafetensorsError`` with the file and
the reason.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, List, Mapping, Tuple

import numpy as np
import torch


class SafetensorsError(ValueError):
    pass


# safetensors dtype string -> (bytes per element, torch dtype, numpy carrier dtype)
_DTYPES = {
    "F64": (8, torch.float64, np.float64),
    "F32": (4, torch.float32, np.float32),
    "F16": (2, torch.float16, np.float16),
    "BF16": (2, torch.bfloat16, np.uint16),
    "I64": (8, torch.int64, np.int64),
    "I32": (4, torch.int32, np.int32),
    "I16": (2, torch.int16, np.int16),
    "I8": (1, torch.int8, np.int8),
    "U8": (1, torch.uint8, np.uint8),
    "BOOL": (1, torch.bool, np.bool_),
}
_TORCH_TO_ST = {v[1]: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    """A memory-mapped ``.safetensors`` file: names, shapes and dtypes from the header, tensors on demand."""

    def __init__(self, path: str):
        self.path = path
        try:
            size = os.path.getsize(path)
            self._fh = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"{path}: cannot open ({e.strerror})") from e
        if size < 8:
            raise SafetensorsError(f"{path}: too short to hold a safetensors header ({size} bytes)")
        (hlen,) = struct.unpack("<Q", self._fh.read(8))
        if hlen <= 0 or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._fh.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from e
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        self.metadata = header.pop("__metadata__", None)
        self._data_start = 8 + hlen
        data_len = size - self._data_start
        self.entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, info in header.items():
            try:
                dt, shape, (b, e) = info["dtype"], tuple(int(s) for s in info["shape"]), info["data_offsets"]
            except (KeyError, TypeError, ValueError) as ex:
                raise SafetensorsError(f"{path}: entry '{name}' is malformed") from ex
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype '{dt}'")
            n = 1
            for s in shape:
                n *= s
            if b < 0 or e < b or e > data_len or e - b != n * _DTYPES[dt][0]:
                raise SafetensorsError(f"{path}: tensor '{name}' ({dt}{list(shape)}) has data_offsets [{b}, {e}] "
                                       f"that do not match its size or the file (truncated file?)")
            self.entries[name] = (dt, shape, b, e)
        self._mm = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def names(self) -> List[str]:
        return list(self.entries)

    def shape(self, name: str) -> Tuple[int, ...]:
        return self.entries[name][1]

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self.entries[name][0]][1]

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor with a private copy of the data (the file may be closed afterwards)."""
        if name not in self.entries:
            raise SafetensorsError(f"{self.path}: no tensor named '{name}'")
        dt, shape, b, e = self.entries[name]
        _, tdt, ndt = _DTYPES[dt]
        arr = np.frombuffer(self._mm, dtype=ndt, count=(e - b) // np.dtype(ndt).itemsize, offset=self._data_start + b)
        t = torch.from_numpy(arr.copy())
        if dt == "BF16":
            t = t.view(torch.bfloat16)
        return t.reshape(shape)

    def close(self) -> None:
        if self._mm is not None:
            self._mm.close()
            self._mm = None
        self._fh.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def list_safetensors_files(model_dir: str) -> List[str]:
    """Every ``*.safetensors`` of a folder in sorted order, or the path itself if it is a file
    (reference utils/safetensors.cpp:118-133)."""
    if os.path.isfile(model_dir):
        return [model_dir]
    if not os.path.isdir(model_dir):
        raise SafetensorsError(f"{model_dir}: no such model folder")
    files = sorted(os.path.join(model_dir, f) for f in os.listdir(model_dir) if f.endswith(".safetensors"))
    if not files:
        raise SafetensorsError(f"{model_dir}: holds no .safetensors file")
    return files


def save_safetensors(path: str, tensors: Mapping[str, torch.Tensor], metadata: Mapping[str, str] | None = None) -> None:
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs = []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _TORCH_TO_ST:
            raise SafetensorsError(f"tensor '{name}' has dtype {t.dtype}, which safetensors cannot hold here")
        raw = (t.view(torch.uint16) if t.dtype == torch.bfloat16 else t).numpy().tobytes()
        header[name] = {"dtype": _TORCH_TO_ST[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    hjson = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hjson += b" " * ((8 - len(hjson) % 8) % 8)
    tmp = path + f".{os.getpid()}.tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hjson)))
        f.write(hjson)
        for raw in blobs:
            f.write(raw)
    os.replace(tmp, path)
