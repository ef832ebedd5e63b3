"""Random weights from a configuration and a seed.

Matrices and the embedding table are N(0, 0.02); vectors (norm weights, the
per-head norms of q and k included) are 1 + U(-0.1, 0.1).  The generator is
counter based: the value of element ``i`` of a tensor depends only on (seed,
tensor name, i), through integer mixing (the splitmix64 finaliser) and a
Box-Muller step in 64-bit floats, so the same values come out on the CPU and
on the device, in any chunking, and a model made in device memory can be handed
to a plain implementation element by element.  A tensor's values do not depend
on which other tensors exist.  The reference has no such mode (its tests fill
tensors with one byte value, tests/qwen_weights_test.cc:207-221).
"""
from __future__ import annotations

import hashlib
import json
import math
import os
from typing import Iterator, Tuple

import torch

from ..parts.base import Runtime, TensorSpec
from .safetensors_io import write_safetensors

MATRIX_STD = 0.02
VECTOR_SPREAD = 0.1
_CHUNK = 1 << 24            # elements made at a time (bounds the 64-bit temporaries)


def _signed(x: int) -> int:
    """A 64-bit pattern as the int64 that holds it."""
    x &= (1 << 64) - 1
    return x - (1 << 64) if x >= (1 << 63) else x


_GAMMA = _signed(0x9E3779B97F4A7C15)
_MUL1 = _signed(0xBF58476D1CE4E5B9)
_MUL2 = _signed(0x94D049BB133111EB)


def _lsr(x: torch.Tensor, s: int) -> torch.Tensor:
    """Logical shift right of int64 (torch's >> keeps the sign)."""
    return (x >> s) & ((1 << (64 - s)) - 1)


def _mix(counter: torch.Tensor, key: int) -> torch.Tensor:
    """splitmix64: 64 mixed bits for each counter value (int64, wrapping)."""
    z = counter * _GAMMA + key
    z = (z ^ _lsr(z, 30)) * _MUL1
    z = (z ^ _lsr(z, 27)) * _MUL2
    return z ^ _lsr(z, 31)


def _key(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return _signed(int.from_bytes(digest[:8], "little"))


def _fill(out: torch.Tensor, key: int, normal: bool) -> None:
    flat = out.view(-1)
    n = flat.numel()
    for start in range(0, n, _CHUNK):
        stop = min(n, start + _CHUNK)
        bits = _mix(torch.arange(start + 1, stop + 1, dtype=torch.int64, device=out.device), key)
        hi = _lsr(bits, 32).to(torch.float64)
        u1 = (hi + 0.5) * (1.0 / 4294967296.0)
        if normal:
            lo = (bits & 0xFFFFFFFF).to(torch.float64)
            u2 = (lo + 0.5) * (1.0 / 4294967296.0)
            v = torch.sqrt(-2.0 * torch.log(u1)) * torch.cos((2.0 * math.pi) * u2) * MATRIX_STD
        else:
            v = 1.0 + (2.0 * u1 - 1.0) * VECTOR_SPREAD
        flat[start:stop] = v.to(torch.float32).to(out.dtype)


def random_tensor(spec: TensorSpec, seed: int, dtype: torch.dtype,
                  device: torch.device = torch.device("cpu")) -> torch.Tensor:
    if spec.kind == "int":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    t = torch.empty(spec.shape, dtype=dtype, device=device)
    _fill(t, _key(seed, spec.name), normal=len(spec.shape) >= 2)
    return t


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


def bind_random_weights(model, seed: int, runtime: Runtime, stored: torch.dtype = torch.bfloat16) -> None:
    """Fill a model with random weights made on its device (no file): the values
    that ``write_random_model`` would store as ``stored`` with the same seed,
    widened to the run's type as the loader widens a checkpoint's."""
    tensors = {}
    for spec in model.expected_tensors(None):
        t = random_tensor(spec, seed, stored, runtime.device)
        tensors[spec.name] = t if t.dtype in (runtime.dtype, torch.int32) else t.to(runtime.dtype)
    model.bind(tensors)
