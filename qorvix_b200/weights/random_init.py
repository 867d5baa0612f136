"""Random-weights mode: a configuration and a seed become a model folder.

The reference has deterministic fills for its tests only (tests/benchmark_test.cpp:45-50).
Here any registered architecture states its tensors (name, shape, kind) and this module
draws them: matrices from N(0, 0.02), norm weights from 1 + N(0, 0.1).  Each tensor has its own
generator seeded from (seed, name), so a tensor's values do not depend on the order or on
which other tensors exist.
"""
from __future__ import annotations

import json
import zlib
from pathlib import Path
from typing import Iterator, Tuple

import torch

from ..config import lookup_architecture
from .safetensors_io import write_safetensors

MATRIX_STD = 0.02
NORM_STD = 0.1


def _generator(seed: int, name: str, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed((int(seed) * 1000003 + zlib.crc32(name.encode())) % (2 ** 63 - 1))
    return g


def draw_tensor(name: str, shape, kind: str, seed: int, device="cpu", dtype=torch.bfloat16) -> torch.Tensor:
    """kind: 'matrix' -> N(0, 0.02); 'norm' -> 1 + N(0, 0.1).  Drawn in float32, then rounded."""
    g = _generator(seed, name, torch.device(device))
    t = torch.randn(tuple(shape), generator=g, device=device, dtype=torch.float32)
    if kind == "norm":
        t = 1.0 + NORM_STD * t
    elif kind == "matrix":
        t = MATRIX_STD * t
    else:
        raise ValueError(f"unknown tensor kind {kind!r}")
    return t.to(dtype)


def random_tensors(config, seed: int, device="cpu", dtype=torch.bfloat16) -> Iterator[Tuple[str, torch.Tensor]]:
    """(name, tensor) for every tensor the architecture's model expects."""
    entry = lookup_architecture(config.architecture)
    spec = entry.build_spec(config)
    for name, (shape, kind) in spec.tensor_table().items():
        yield name, draw_tensor(name, shape, kind, seed, device, dtype)


def write_random_model(model_dir, config, seed: int, dtype=torch.bfloat16) -> Path:
    """Writes config.json and model.safetensors into `model_dir` (created if needed)."""
    model_dir = Path(model_dir)
    model_dir.mkdir(parents=True, exist_ok=True)
    (model_dir / "config.json").write_text(json.dumps(config.to_dict(), indent=1))
    write_safetensors(model_dir / "model.safetensors", random_tensors(config, seed, "cpu", dtype),
                      metadata={"format": "pt", "seed": seed})
    return model_dir
