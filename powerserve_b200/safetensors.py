"""Reader (and a small writer, for synthetic models) of the safetensors container: an 8-byte little-endian header length,
that many bytes of JSON (tensor name -> dtype, shape, data_offsets relative to the end of the header), then the data.

Tensors are exposed the way gguf.GGUFTensor exposes GGUF tensors: a numpy view of the memory-mapped file plus the host
pointer and a ggml-style type id, so the C ABI's weight binding (ps_cuda_tensor = host pointer + type) takes both
containers alike.  bfloat16 has no numpy dtype: such tensors are uint16 views, `to_float32` widens them exactly.
"""
from __future__ import annotations

import json
import mmap
import struct
from typing import Dict, Iterable, Tuple

import numpy as np

# ggml type ids (libs/ggml/include/ggml.h of the reference): F32 0, F16 1, I32 26, BF16 30
PS_F32, PS_F16, PS_I32, PS_BF16 = 0, 1, 26, 30
_DTYPES = {"F32": (np.float32, PS_F32), "F16": (np.float16, PS_F16), "I32": (np.int32, PS_I32), "BF16": (np.uint16, PS_BF16)}


class SafeTensor:
    def __init__(self, name: str, data: np.ndarray, ps_type: int):
        self.name, self.data, self.ps_type = name, data, ps_type
        self.shape: Tuple[int, ...] = tuple(data.shape)

    @property
    def host_ptr(self) -> int:
        return self.data.ctypes.data

    # the name the GGUF side uses for the same thing
    @property
    def ggml_type(self) -> int:
        return self.ps_type

    def to_float32(self) -> np.ndarray:
        if self.ps_type == PS_BF16:
            return (self.data.astype(np.uint32) << 16).view(np.float32)
        return self.data.astype(np.float32)


class SafeTensorsFile:
    def __init__(self, path: str):
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        (n,) = struct.unpack("<Q", self._mm[:8])
        header = json.loads(self._mm[8:8 + n].decode("utf-8"))
        base = 8 + n
        self.tensors: Dict[str, SafeTensor] = {}
        buf = np.frombuffer(self._mm, dtype=np.uint8)
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            if meta["dtype"] not in _DTYPES:
                raise ValueError(f"{path}: tensor {name} has unsupported dtype {meta['dtype']}")
            dt, ps = _DTYPES[meta["dtype"]]
            lo, hi = meta["data_offsets"]
            a = buf[base + lo:base + hi].view(dt).reshape(meta["shape"])
            self.tensors[name] = SafeTensor(name, a, ps)

    def __contains__(self, name: str) -> bool:
        return name in self.tensors

    def __getitem__(self, name: str) -> SafeTensor:
        return self.tensors[name]

    def names(self) -> Iterable[str]:
        return self.tensors.keys()


def float32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """round-to-nearest-even"""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16).reshape(np.shape(a))


def write_file(path: str, tensors: Dict[str, np.ndarray]) -> None:
    """float32 arrays are stored as bfloat16 (rounded to nearest even), int32 arrays as they are"""
    header, blobs, off = {}, [], 0
    for name, a in tensors.items():
        if a.dtype == np.int32:
            dt, raw = "I32", np.ascontiguousarray(a).tobytes()
        elif a.dtype == np.uint16:
            dt, raw = "BF16", np.ascontiguousarray(a).tobytes()
        else:
            dt, raw = "BF16", float32_to_bf16_bits(a).tobytes()
        header[name] = {"dtype": dt, "shape": list(a.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    h = json.dumps(header, separators=(",", ":")).encode()
    h += b" " * (-len(h) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for b in blobs:
            f.write(b)
