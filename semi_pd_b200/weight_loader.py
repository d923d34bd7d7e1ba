"""Checkpoint reading for `--load-format safetensors`: a safetensors file is an 8-byte
little-endian header length, that many bytes of JSON (name -> dtype, shape, data_offsets), then
the tensor bytes.  Tensors are yielded one at a time as CPU torch tensors over a memory map (the
model's load_weights() converts and uploads them), the contract of the reference's
`safetensors_weights_iterator` (python/sglang/srt/model_loader/weight_utils.py)."""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Iterator, Tuple

import torch

_DTYPES = {"BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "F64": torch.float64,
           "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
           "BOOL": torch.bool}


def safetensors_weights_iterator(path: str) -> Iterator[Tuple[str, torch.Tensor]]:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_COPY)
    base = 8 + n
    for name, info in header.items():
        if name == "__metadata__":
            continue
        try:
            dtype = _DTYPES[info["dtype"]]
        except KeyError:
            raise ValueError(f"{path}: tensor {name} has unsupported dtype {info['dtype']}") from None
        lo, hi = info["data_offsets"]
        shape = tuple(info["shape"])
        if hi - lo == 0:
            yield name, torch.empty(shape, dtype=dtype)
            continue
        flat = torch.frombuffer(mm, dtype=dtype, count=(hi - lo) // torch.empty((), dtype=dtype).element_size(),
                                offset=base + lo)
        yield name, flat.reshape(shape).clone()


def model_weights_path(model_path: str) -> str:
    return os.path.join(model_path, "model.safetensors")
