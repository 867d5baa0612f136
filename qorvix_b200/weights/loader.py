"""Weights by tensor name, with one error that lists everything wrong.

The reference loads each tensor by name and fails on the first missing one
(runtime/src/weights.cpp:17-49, tensor_load.hpp:32-45).  Here the model states every
tensor it expects (name -> shape); the checkpoint is compared against that list once and
a single WeightError names all missing tensors, all unexpected tensors and all wrong shapes.

Storage rule: floating tensors are kept in bfloat16 on the bfloat16 path, except that a
tensor stored in 32-bit stays 32-bit; integer tables become int32; on the float32 path
every floating tensor is float32.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, Iterable, Mapping, Optional, Tuple

import torch

from .safetensors_io import SafetensorsError, SafetensorsFile


class WeightError(ValueError):
    """Checkpoint and model disagree.  `.missing`, `.unexpected`, `.wrong_shape` hold the lists."""

    def __init__(self, where, missing, unexpected, wrong_shape, other=()):
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.wrong_shape = sorted(wrong_shape)
        self.other = list(other)
        lines = [f"{where}: the checkpoint does not fit the model"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(
                f"{n}: stored {list(got)}, expected {list(exp)}" for n, got, exp in self.wrong_shape))
        lines.extend(f"  {o}" for o in self.other)
        super().__init__("\n".join(lines))


def storage_dtype(stored: torch.dtype, compute_dtype: torch.dtype) -> torch.dtype:
    if not stored.is_floating_point:
        return torch.int32
    if compute_dtype == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


class Checkpoint:
    """The tensors of a model folder: model.safetensors, or the shards that
    model.safetensors.index.json names."""

    def __init__(self, model_dir):
        self.model_dir = Path(model_dir)
        self._files: Dict[str, SafetensorsFile] = {}
        self._where: Dict[str, str] = {}
        index = self.model_dir / "model.safetensors.index.json"
        single = self.model_dir / "model.safetensors"
        if single.is_file():
            shards = [single.name]
        elif index.is_file():
            shards = sorted(set(json.loads(index.read_text())["weight_map"].values()))
        else:
            raise WeightError(str(self.model_dir), [], [], [], ["no model.safetensors (or model.safetensors.index.json) in the model folder"])
        for shard in shards:
            try:
                f = SafetensorsFile(self.model_dir / shard)
            except (OSError, SafetensorsError) as e:
                raise WeightError(str(self.model_dir), [], [], [], [str(e)]) from None
            self._files[shard] = f
            for n in f.names():
                self._where[n] = shard

    def names(self) -> Iterable[str]:
        return self._where.keys()

    def shape(self, name) -> Tuple[int, ...]:
        return self._files[self._where[name]].shape(name)

    def dtype(self, name) -> torch.dtype:
        return self._files[self._where[name]].dtype(name)

    def tensor(self, name) -> torch.Tensor:
        return self._files[self._where[name]].tensor(name)


class TensorSource:
    """What parts draw their weights from: `get(name)` returns the tensor on the device in
    its storage dtype.  Backed by a Checkpoint or by tensors in memory."""

    def __init__(self, tensors: Mapping[str, torch.Tensor] = None, checkpoint: Checkpoint = None,
                 device="cuda", compute_dtype=torch.bfloat16, where="weights"):
        self._tensors = dict(tensors) if tensors is not None else None
        self._ckpt = checkpoint
        self.device = torch.device(device)
        self.compute_dtype = compute_dtype
        self.where = where

    def names(self):
        return list(self._tensors.keys()) if self._tensors is not None else list(self._ckpt.names())

    def shape(self, name):
        return tuple(self._tensors[name].shape) if self._tensors is not None else self._ckpt.shape(name)

    def check(self, expected: Mapping[str, Tuple[int, ...]], optional: Iterable[str] = (), ignored: Iterable[str] = ()) -> None:
        """Raises WeightError unless the stored names and shapes are exactly the expected ones
        (names in `optional` may be present or absent; names that match a pattern of `ignored` are
        buffers some checkpoints of the architecture store beside the weights, such as a rotary
        table, and are passed over).  The reference reads optional tensors the same way
        (runtime/include/qorvix/runtime/tensor_load.hpp:82-92) and never looks at names it does not ask for."""
        import fnmatch
        have = set(self.names())
        optional = set(optional)
        ignored = tuple(ignored)
        missing = [n for n in expected if n not in have and n not in optional]
        unexpected = [n for n in have if n not in expected and n not in optional
                      and not any(fnmatch.fnmatchcase(n, pat) for pat in ignored)]
        wrong = [(n, self.shape(n), tuple(expected[n])) for n in expected
                 if n in have and tuple(self.shape(n)) != tuple(expected[n])]
        if missing or unexpected or wrong:
            raise WeightError(self.where, missing, unexpected, wrong)

    def has(self, name) -> bool:
        return name in (self._tensors if self._tensors is not None else self._ckpt._where)

    def get(self, name: str, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        t = self._tensors[name] if self._tensors is not None else self._ckpt.tensor(name)
        want = dtype or storage_dtype(t.dtype, self.compute_dtype)
        if t.device != self.device:
            t = t.to(self.device, non_blocking=False)
        if t.dtype != want:
            t = t.to(want)
        return t.contiguous()
