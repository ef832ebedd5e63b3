"""Random weights from a configuration and a seed.

Matrices and the embedding table are N(0, 0.02); vectors (norm weights, the
per-head norms of q and k included) are 1 + U(-0.1, 0.1).  Every tensor has a
generator of its own, keyed by (seed, tensor name), so a tensor's values do not
depend on which other tensors exist.  The reference has no such mode (its tests
fill tensors with one byte value, tests/qwen_weights_test.cc:207-221).
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Iterator, Tuple

import torch

from ..parts.base import Runtime, TensorSpec
from .safetensors_io import write_safetensors

MATRIX_STD = 0.02
VECTOR_SPREAD = 0.1


def _generator(seed: int, name: str, device: torch.device) -> torch.Generator:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    g = torch.Generator(device=device)
    g.manual_seed(int.from_bytes(digest[:8], "little") & (2**63 - 1))
    return g


def random_tensor(spec: TensorSpec, seed: int, dtype: torch.dtype,
                  device: torch.device = torch.device("cpu")) -> torch.Tensor:
    g = _generator(seed, spec.name, device)
    if spec.kind == "int":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    if len(spec.shape) >= 2:
        t = torch.empty(spec.shape, dtype=torch.float32, device=device).normal_(0.0, MATRIX_STD, generator=g)
    else:
        t = torch.empty(spec.shape, dtype=torch.float32, device=device).uniform_(
            1.0 - VECTOR_SPREAD, 1.0 + VECTOR_SPREAD, generator=g)
    return t.to(dtype)


def random_tensors(model, seed: int, dtype: torch.dtype,
                   device: torch.device = torch.device("cpu")) -> Iterator[Tuple[str, torch.Tensor]]:
    for spec in model.expected_tensors(None):
        yield spec.name, random_tensor(spec, seed, dtype, device)


def write_random_model(config_object: dict, out_dir: str, seed: int,
                       dtype: torch.dtype = torch.bfloat16) -> str:
    """Write ``out_dir/config.json`` and ``out_dir/model.safetensors`` for the
    architecture that ``config_object`` (the content of a config.json) names."""
    from ..config.registry import find_architecture
    from ..engine.model import DecoderModel

    arch = find_architecture(config_object)
    config = arch.read_config(config_object)
    spec = arch.model_spec(config)
    model = DecoderModel(spec, Runtime(torch.device("cpu"), dtype, None))
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config_object, f, indent=1, sort_keys=True)
    write_safetensors(os.path.join(out_dir, "model.safetensors"), random_tensors(model, seed, dtype))
    return out_dir


def bind_random_weights(model, seed: int, runtime: Runtime) -> None:
    """Fill a model with random weights made on its device (no file)."""
    tensors = {}
    for spec in model.expected_tensors(None):
        tensors[spec.name] = random_tensor(spec, seed, runtime.dtype, runtime.device)
    model.bind(tensors)
