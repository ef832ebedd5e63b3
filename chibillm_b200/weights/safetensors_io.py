"""Reading and writing safetensors files without a helper library.

Layout of a file: 8 bytes little-endian header length, a JSON header that maps
each tensor name to ``{"dtype", "shape", "data_offsets"}``, then the data.  The
checks follow the reference's reader (src/model_format/safetensors.cc:233-286):
header length within the file and under 100 MiB, byte count equal to shape
times element size, every range inside the data section, ranges sorted and
gap-free from 0 to the end.  The file is memory-mapped; a tensor is a view
until it is copied to the device.

Checkpoint discovery (src/model_format/safetensors.cc:291-387):
``model.safetensors``, else the shards of ``model.safetensors.index.json``,
else the only ``*.safetensors`` in the folder.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from dataclasses import dataclass
from typing import Dict, Iterable, List, Tuple

import torch

_DTYPES = {
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "F32": (torch.float32, 4),
    "F64": (torch.float64, 8),
    "I64": (torch.int64, 8),
    "I32": (torch.int32, 4),
    "I16": (torch.int16, 2),
    "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}
_MAX_HEADER = 100 * 1024 * 1024


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    begin: int
    end: int
    file_index: int


class SafetensorsFile:
    """One memory-mapped file."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"file_open_failed: {path}: {e}") from None
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"invalid_header: {path} is shorter than its length field")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen > _MAX_HEADER or hlen > size - 8:
            raise SafetensorsError(f"invalid_header: {path} declares a header of {hlen} bytes")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"invalid_header: {path}: {e}") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"invalid_header: {path}: header is not an object")
        self.data_start = 8 + hlen
        data_size = size - self.data_start
        self.tensors: Dict[str, TensorInfo] = {}
        ranges = []
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            try:
                dtype = meta["dtype"]
                shape = tuple(int(x) for x in meta["shape"])
                begin, end = (int(x) for x in meta["data_offsets"])
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"invalid_tensor_entry: {path}: '{name}'") from None
            if dtype not in _DTYPES:
                raise SafetensorsError(f"unsupported_dtype: {path}: '{name}' has dtype {dtype}")
            count = 1
            for d in shape:
                if d < 0:
                    raise SafetensorsError(f"invalid_tensor_entry: {path}: '{name}' has shape {shape}")
                count *= d
            if end - begin != count * _DTYPES[dtype][1] or begin < 0 or end > data_size:
                raise SafetensorsError(
                    f"invalid_tensor_range: {path}: '{name}' {dtype}{list(shape)} does not fit bytes {begin}..{end}")
            self.tensors[name] = TensorInfo(name, dtype, shape, begin, end, 0)
            ranges.append((begin, end, name))
        ranges.sort()
        cursor = 0
        for begin, end, name in ranges:
            if begin != cursor:
                raise SafetensorsError(f"invalid_tensor_range: {path}: gap or overlap before '{name}'")
            cursor = end
        if cursor != data_size:
            raise SafetensorsError(f"invalid_tensor_range: {path}: {data_size - cursor} unused bytes at the end")
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def read(self, name: str) -> torch.Tensor:
        info = self.tensors[name]
        dtype, _ = _DTYPES[info.dtype]
        count = 1
        for d in info.shape:
            count *= d
        if count == 0:
            return torch.empty(info.shape, dtype=dtype)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)   # the map is read-only; nobody writes to it
            t = torch.frombuffer(self._map, dtype=dtype, count=count, offset=self.data_start + info.begin)
        return t.reshape(info.shape)

    def close(self) -> None:
        # Views made by read() keep the map alive; closing is left to the collector.
        self._map = None
        self._f.close()


class Checkpoint:
    """All tensors of a model folder, whichever files hold them."""

    def __init__(self, files: List[SafetensorsFile], owner: Dict[str, int]):
        self.files = files
        self._owner = owner

    @classmethod
    def open_model(cls, model_dir: str) -> "Checkpoint":
        single = os.path.join(model_dir, "model.safetensors")
        index = os.path.join(model_dir, "model.safetensors.index.json")
        if os.path.isfile(single):
            paths = [single]
            listed = None
        elif os.path.isfile(index):
            try:
                with open(index, "r", encoding="utf-8") as f:
                    weight_map = json.load(f)["weight_map"]
                assert isinstance(weight_map, dict) and weight_map
            except Exception:
                raise SafetensorsError(f"invalid_checkpoint_index: {index}") from None
            shards = []
            for name, shard in weight_map.items():
                if (not isinstance(shard, str) or os.path.basename(shard) != shard
                        or not shard.endswith(".safetensors")):
                    raise SafetensorsError(f"invalid_checkpoint_index: {index}: shard {shard!r}")
                if shard not in shards:
                    shards.append(shard)
            paths = [os.path.join(model_dir, s) for s in shards]
            listed = {name: shards.index(shard) for name, shard in weight_map.items()}
        else:
            try:
                found = sorted(p for p in os.listdir(model_dir) if p.endswith(".safetensors"))
            except OSError as e:
                raise SafetensorsError(f"file_open_failed: {model_dir}: {e}") from None
            if not found:
                raise SafetensorsError(f"file_open_failed: no safetensors file in {model_dir}")
            if len(found) > 1:
                raise SafetensorsError(f"ambiguous_checkpoint: {model_dir} holds {found} and no index")
            paths = [os.path.join(model_dir, found[0])]
            listed = None
        files = [SafetensorsFile(p) for p in paths]
        owner: Dict[str, int] = {}
        for i, f in enumerate(files):
            for name in f.tensors:
                if name in owner:
                    raise SafetensorsError(f"invalid_checkpoint_index: '{name}' is in two shards")
                if listed is not None and listed.get(name) != i:
                    raise SafetensorsError(f"invalid_checkpoint_index: '{name}' is not listed for {f.path}")
                owner[name] = i
        if listed is not None:
            for name in listed:
                if name not in owner:
                    raise SafetensorsError(f"invalid_checkpoint_index: '{name}' is listed but not stored")
        return cls(files, owner)

    def names(self) -> List[str]:
        return list(self._owner)

    def __contains__(self, name: str) -> bool:
        return name in self._owner

    def info(self, name: str) -> TensorInfo:
        return self.files[self._owner[name]].tensors[name]

    def read(self, name: str) -> torch.Tensor:
        return self.files[self._owner[name]].read(name)


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]]) -> None:
    """Write named CPU tensors in the given order, contiguous and gap-free."""
    items = [(n, t.detach().contiguous().cpu()) for n, t in tensors]
    header = {}
    cursor = 0
    for name, t in items:
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"unsupported_dtype: '{name}' has dtype {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [cursor, cursor + nbytes]}
        cursor += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for _, t in items:
            if t.numel():
                f.write(t.view(torch.uint8).numpy().tobytes() if t.dim() else
                        t.reshape(1).view(torch.uint8).numpy().tobytes())
