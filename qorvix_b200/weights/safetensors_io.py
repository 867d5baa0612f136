"""Reading and writing the safetensors container (the format is public: an 8-byte
little-endian header length, a JSON header {name: {dtype, shape, data_offsets}}, raw data).

The reference reads GGUF by tensor name (runtime/include/qorvix/runtime/tensor_load.hpp:27-96);
this is the same service for config.json + safetensors model folders.
"""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path
from typing import Dict, Iterable, Tuple

import numpy as np
import torch

_DTYPES = {
    "F64": (torch.float64, np.float64, 8), "F32": (torch.float32, np.float32, 4),
    "F16": (torch.float16, np.float16, 2), "BF16": (torch.bfloat16, np.uint16, 2),
    "I64": (torch.int64, np.int64, 8), "I32": (torch.int32, np.int32, 4),
    "I16": (torch.int16, np.int16, 2), "I8": (torch.int8, np.int8, 1),
    "U8": (torch.uint8, np.uint8, 1), "BOOL": (torch.bool, np.bool_, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One mapped file; tensors are views of the mapping until copied."""

    def __init__(self, path):
        self.path = Path(path)
        with open(self.path, "rb") as fh:
            head = fh.read(8)
            if len(head) < 8:
                raise SafetensorsError(f"{self.path}: too short to be a safetensors file")
            (hlen,) = struct.unpack("<Q", head)
            size = self.path.stat().st_size
            if hlen <= 0 or 8 + hlen > size:
                raise SafetensorsError(f"{self.path}: header length {hlen} does not fit the file ({size} bytes)")
            try:
                header = json.loads(fh.read(hlen).decode("utf-8"))
            except (UnicodeDecodeError, json.JSONDecodeError) as e:
                raise SafetensorsError(f"{self.path}: header is not JSON ({e})") from None
            self._map = mmap.mmap(fh.fileno(), 0, access=mmap.ACCESS_READ)
        self._base = 8 + hlen
        self.metadata = header.pop("__metadata__", {})
        self.entries: Dict[str, dict] = header
        for name, meta in self.entries.items():
            if meta.get("dtype") not in _DTYPES:
                raise SafetensorsError(f"{self.path}: tensor '{name}' has unsupported dtype {meta.get('dtype')!r}")
            b, e = meta["data_offsets"]
            n = int(np.prod(meta["shape"], dtype=np.int64)) if meta["shape"] else 1
            if e - b != n * _DTYPES[meta["dtype"]][2]:
                raise SafetensorsError(f"{self.path}: tensor '{name}' holds {e - b} bytes, shape {meta['shape']} needs {n * _DTYPES[meta['dtype']][2]}")
            if self._base + e > size:
                raise SafetensorsError(f"{self.path}: tensor '{name}' reaches beyond the end of the file")

    def names(self) -> Iterable[str]:
        return self.entries.keys()

    def shape(self, name: str) -> Tuple[int, ...]:
        return tuple(self.entries[name]["shape"])

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self.entries[name]["dtype"]][0]

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that aliases the mapping (read-only memory: copy before writing)."""
        meta = self.entries[name]
        tdt, ndt, _ = _DTYPES[meta["dtype"]]
        b, e = meta["data_offsets"]
        n = (e - b) // np.dtype(ndt).itemsize
        arr = np.frombuffer(self._map, dtype=ndt, count=n, offset=self._base + b)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")          # non-writable buffer; it is only read
            t = torch.from_numpy(arr)
        if tdt == torch.bfloat16:
            t = t.view(torch.bfloat16)
        return t.reshape(meta["shape"])


def write_safetensors(path, tensors: Iterable[Tuple[str, torch.Tensor]], metadata: dict = None) -> None:
    """Writes tensors in the given order.  `tensors` may be a generator; data is staged
    tensor by tensor so that a large model never sits in memory twice."""
    path = Path(path)
    header, blobs, offset = {}, [], 0
    tmp_data = path.with_suffix(path.suffix + ".data.tmp")
    with open(tmp_data, "wb") as data:
        for name, t in tensors:
            t = t.detach().cpu().contiguous()
            if t.dtype not in _NAMES:
                raise SafetensorsError(f"tensor '{name}': dtype {t.dtype} cannot be stored")
            raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
            header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
            data.write(raw)
            offset += len(raw)
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    hbytes = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hbytes += b" " * ((8 - len(hbytes) % 8) % 8)
    with open(path, "wb") as out, open(tmp_data, "rb") as data:
        out.write(struct.pack("<Q", len(hbytes)))
        out.write(hbytes)
        while True:
            chunk = data.read(1 << 24)
            if not chunk:
                break
            out.write(chunk)
    tmp_data.unlink()
