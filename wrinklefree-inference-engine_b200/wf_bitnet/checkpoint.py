"""Reader of `model.safetensors` files that needs nothing but numpy: an 8-byte little-endian header length, that many bytes of JSON
(name -> dtype, shape, data_offsets), then the raw little-endian data.  bfloat16 tensors come back as uint16 bit patterns
(numpy has no bfloat16); `to_float32` widens them exactly."""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path
from typing import Dict, Iterator, Tuple

import numpy as np

_DTYPES = {"BF16": np.uint16, "F16": np.float16, "F32": np.float32, "F64": np.float64, "I32": np.int32, "I64": np.int64, "U8": np.uint8,
           "I8": np.int8, "I16": np.int16, "BOOL": np.bool_}


class SafetensorsFile:
    def __init__(self, path):
        self.path = Path(path)
        self._f = open(self.path, "rb")
        (n,) = struct.unpack("<Q", self._f.read(8))
        self.header = json.loads(self._f.read(n).decode("utf-8"))
        self.header.pop("__metadata__", None)
        self._base = 8 + n
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)

    def names(self):
        return list(self.header)

    def info(self, name) -> Tuple[str, Tuple[int, ...]]:
        h = self.header[name]
        return h["dtype"], tuple(h["shape"])

    def get(self, name) -> Tuple[np.ndarray, str]:
        """-> (array in its stored element type, BF16 as uint16 bits; safetensors dtype string)."""
        h = self.header[name]
        if h["dtype"] not in _DTYPES:
            raise ValueError(f"{self.path}: tensor {name!r} has unsupported dtype {h['dtype']}")
        lo, hi = h["data_offsets"]
        a = np.frombuffer(self._mm, dtype=_DTYPES[h["dtype"]], count=(hi - lo) // np.dtype(_DTYPES[h["dtype"]]).itemsize, offset=self._base + lo)
        return a.reshape(h["shape"]), h["dtype"]

    def items(self) -> Iterator[Tuple[str, np.ndarray, str]]:
        for name in self.header:
            a, dt = self.get(name)
            yield name, a, dt

    def close(self):
        try:
            self._mm.close()
        except BufferError:
            pass                    # arrays handed out still reference the mapping
        self._f.close()


def to_float32(a: np.ndarray, dtype: str) -> np.ndarray:
    if dtype == "BF16":
        return (a.astype(np.uint32) << 16).view(np.float32)
    return a.astype(np.float32)


def to_bfloat16_bits(a: np.ndarray, dtype: str) -> np.ndarray:
    """uint16 bit patterns of the values rounded to bfloat16 (round to nearest even)."""
    if dtype == "BF16":
        return np.ascontiguousarray(a)
    u = np.ascontiguousarray(a.astype(np.float32)).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def read_config(model_dir) -> Dict:
    return json.loads((Path(model_dir) / "config.json").read_text())
