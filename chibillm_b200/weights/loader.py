"""Loading a model's tensors from safetensors by tensor name.

Everything is checked before anything is read (src/model_format/
weight_reader.cc:16-30, src/qwen/qwen_weights.cc:150-179): one error lists all
missing tensors, all tensors the model does not expect, all wrong shapes and
all element types it cannot take.

Element types on the device: in the bfloat16 engine a tensor stored as BF16
stays bfloat16 (F16 is converted to it), a tensor stored in 32-bit stays
32-bit (F64 is narrowed to it); in the 32-bit engine every floating tensor is
widened to float32, which is exact for BF16 and F16.  Integer tables become
int32.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..parts.base import Runtime, TensorSpec
from .safetensors_io import Checkpoint, SafetensorsError

_FLOAT = {"BF16", "F16", "F32", "F64"}
_INT = {"I64", "I32", "I16", "I8", "U8"}


class WeightError(ValueError):
    """``missing``, ``unexpected``, ``wrong_shape`` and ``wrong_dtype`` list the
    offending tensor names."""

    def __init__(self, message: str, missing=(), unexpected=(), wrong_shape=(), wrong_dtype=()):
        super().__init__(message)
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)


def check_checkpoint(expected: List[TensorSpec], checkpoint: Checkpoint) -> None:
    by_name = {t.name: t for t in expected}
    if len(by_name) != len(expected):
        raise WeightError("the model declares a tensor name twice")
    missing = [n for n in by_name if n not in checkpoint]
    unexpected = [n for n in checkpoint.names() if n not in by_name]
    wrong_shape, wrong_dtype = [], []
    shape_lines, dtype_lines = [], []
    for name, spec in by_name.items():
        if name not in checkpoint:
            continue
        info = checkpoint.info(name)
        if tuple(info.shape) != tuple(spec.shape):
            wrong_shape.append(name)
            shape_lines.append(f"{name}: stored {list(info.shape)}, expected {list(spec.shape)}")
        allowed = _FLOAT if spec.kind == "float" else _INT
        if info.dtype not in allowed:
            wrong_dtype.append(name)
            dtype_lines.append(f"{name}: stored {info.dtype}, expected one of {sorted(allowed)}")
    if not (missing or unexpected or wrong_shape or wrong_dtype):
        return
    parts = ["the checkpoint does not match the model:"]
    if missing:
        parts.append(f"  missing tensors ({len(missing)}): " + ", ".join(sorted(missing)))
    if unexpected:
        parts.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(sorted(unexpected)))
    if shape_lines:
        parts.append(f"  wrong shapes ({len(shape_lines)}): " + "; ".join(shape_lines))
    if dtype_lines:
        parts.append(f"  unsupported element types ({len(dtype_lines)}): " + "; ".join(dtype_lines))
    raise WeightError("\n".join(parts), missing, unexpected, wrong_shape, wrong_dtype)


def device_dtype(stored: torch.dtype, kind: str, runtime_dtype: torch.dtype) -> torch.dtype:
    if kind == "int":
        return torch.int32
    if runtime_dtype == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


def load_weights(model, model_dir: str, runtime: Runtime) -> Dict[str, torch.Tensor]:
    """Check, read and hand the tensors to the model's parts."""
    try:
        checkpoint = Checkpoint.open_model(model_dir)
    except SafetensorsError as e:
        raise WeightError(str(e)) from None
    expected = model.expected_tensors(checkpoint.names())
    check_checkpoint(expected, checkpoint)
    tensors: Dict[str, torch.Tensor] = {}
    for spec in expected:
        stored = checkpoint.read(spec.name)
        target = device_dtype(stored.dtype, spec.kind, runtime.dtype)
        tensors[spec.name] = stored.to(device=runtime.device, dtype=target, copy=True)
    model.bind(tensors)
    return tensors
