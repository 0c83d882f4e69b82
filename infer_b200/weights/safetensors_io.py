"""Reader and writer for the safetensors container, written against the format itself.

Layout (as the reference's loader reads it, src/loader.h:3-6, src/loader.cpp:56-120): an
8-byte little-endian header length N, N bytes of JSON ``{name: {dtype, shape, data_offsets}}``
(``__metadata__`` is skipped), then the data section; offsets are relative to its start.
Tensors are returned as torch tensors that view a memory map of the file, so a checkpoint is
not read twice.

Dtypes on the way in: BF16 stays bfloat16; F32 stays float32; F16 is widened to float32 (exact);
I64/I32 integer tables become int32 (values are range-checked).  Anything else is refused.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Mapping, Tuple

import numpy as np
import torch


class SafetensorsError(ValueError):
    pass


_ITEMSIZE = {"BF16": 2, "F16": 2, "F32": 4, "I64": 8, "I32": 4}
_TORCH_TO_NAME = {torch.bfloat16: "BF16", torch.float16: "F16", torch.float32: "F32",
                  torch.int64: "I64", torch.int32: "I32"}


class SafetensorsFile:
    """A read-only view of one ``.safetensors`` file."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: file too small to be safetensors ({size} bytes)")
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._mm[:8])
        if 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} exceeds the file size {size}")
        try:
            header = json.loads(self._mm[8:8 + hlen].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from None
        self._data0 = 8 + hlen
        data_len = size - self._data0
        self.entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, info in header.items():
            if name == "__metadata__":
                continue
            try:
                dtype, shape, (b, e) = info["dtype"], tuple(int(s) for s in info["shape"]), info["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed header entry for {name!r}") from None
            if dtype not in _ITEMSIZE:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dtype}")
            numel = int(np.prod(shape, dtype=np.int64)) if shape else 1
            if not (0 <= b <= e <= data_len) or e - b != numel * _ITEMSIZE[dtype]:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} has bad offsets [{b},{e}) for shape {list(shape)} {dtype}")
            self.entries[name] = (dtype, shape, int(b), int(e))

    def names(self):
        return sorted(self.entries)

    def __contains__(self, name: str) -> bool:
        return name in self.entries

    def shape(self, name: str) -> Tuple[int, ...]:
        return self.entries[name][1]

    def dtype_name(self, name: str) -> str:
        return self.entries[name][0]

    def get(self, name: str) -> torch.Tensor:
        """The tensor in its in-memory dtype (see module docstring); a copy, safe after close()."""
        dtype, shape, b, e = self.entries[name]
        raw = np.frombuffer(self._mm, dtype=np.uint8, count=e - b, offset=self._data0 + b)
        if dtype == "BF16":
            t = torch.from_numpy(raw.view(np.int16).copy()).view(torch.bfloat16)
        elif dtype == "F32":
            t = torch.from_numpy(raw.view(np.float32).copy())
        elif dtype == "F16":
            t = torch.from_numpy(raw.view(np.float16).astype(np.float32))
        else:
            a = raw.view(np.int64 if dtype == "I64" else np.int32)
            if a.size and (a.min() < -2**31 or a.max() >= 2**31):
                raise SafetensorsError(f"{self.path}: integer tensor {name!r} does not fit int32")
            t = torch.from_numpy(a.astype(np.int32))
        return t.reshape(shape)

    def close(self):
        try:
            self._mm.close()
        except BufferError:
            pass
        self._f.close()


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor], metadata: Mapping[str, str] = None) -> None:
    """Writes tensors (bf16 / f16 / f32 / i32 / i64, CPU) in name order."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _TORCH_TO_NAME:
            raise SafetensorsError(f"cannot write tensor {name!r} of dtype {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _TORCH_TO_NAME[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            if t.dtype == torch.bfloat16:
                t = t.view(torch.int16)
            f.write(t.numpy().tobytes())
    os.replace(tmp, path)


def open_checkpoint(model_dir: str) -> Iterable[SafetensorsFile]:
    """Every shard of a model folder: ``model.safetensors``, or the files that
    ``model.safetensors.index.json`` names (src/model.cpp:36-48)."""
    index = os.path.join(model_dir, "model.safetensors.index.json")
    single = os.path.join(model_dir, "model.safetensors")
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as f:
            shards = sorted(set(json.load(f)["weight_map"].values()))
        return [SafetensorsFile(os.path.join(model_dir, s)) for s in shards]
    if os.path.isfile(single):
        return [SafetensorsFile(single)]
    raise SafetensorsError(f"{model_dir}: no model.safetensors or model.safetensors.index.json")
