"""A timeline of the kernels of a step, CTA by CTA, from inside the kernels.

Where the profiling mode (profile.py) times every launch alone, this mode
leaves the step as it is (replayed from a CUDA graph, kernels overlapping by
programmatic dependent launch) and has every CTA note when it started, when its
wait for the kernel before it ended, and when its last warp left.  It needs the
libraries built with ``-DCHIBI_TIMELINE`` (``CudaKernels(device, timeline=True)``
builds and loads them; the product's own libraries contain none of it).

    kernels = CudaKernels(device, timeline=True)
    ... run steps ...
    kernels.timeline.reset(); run one step; torch.cuda.synchronize()
    for launch in kernels.timeline.launches(): print(launch)
"""
from __future__ import annotations

from typing import Dict, List

import numpy as np
import torch

from ..csrc import build

RECORD = np.dtype([("unit", "<u4"), ("line", "<u4"), ("block", "<u4"), ("blocks", "<u4"), ("sm", "<u4"),
                   ("pad", "<u4"), ("start", "<u8"), ("waited", "<u8"), ("end", "<u8"), ("marks", "<u8", (4,))])
UNITS = {1: "elementwise", 2: "gemm_simt", 3: "gemm_tcgen05", 4: "attention_generic", 5: "sampling",
         6: "attention_mma", 7: "attention_tcgen05"}
DEFINE = "CHIBI_TIMELINE"


class Timeline:
    def __init__(self, device: torch.device, capacity: int = 1 << 17):
        self.capacity = capacity
        self.records = torch.zeros(capacity * RECORD.itemsize, dtype=torch.uint8, device=device)
        self.count = torch.zeros(1, dtype=torch.int32, device=device)
        self._names: Dict[tuple, str] = {}

    def attach(self, lib, library_name: str) -> None:
        """Point the kernels of every source file of a loaded library at the arrays."""
        import ctypes
        for source in build.LIBRARIES[library_name]:
            fn = getattr(lib, "chibi_timeline_set_" + source[:-3])
            fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint]
            fn.restype = ctypes.c_int
            status = fn(self.records.data_ptr(), self.count.data_ptr(), self.capacity)
            if status != 0:
                raise RuntimeError(f"chibi_timeline_set_{source[:-3]}: CUDA error {status}")

    def reset(self) -> None:
        self.count.zero_()

    def read(self) -> np.ndarray:
        torch.cuda.synchronize()
        n = min(int(self.count.item()), self.capacity)
        raw = self.records[:n * RECORD.itemsize].cpu().numpy()
        return raw.view(RECORD)

    def kernel_name(self, unit: int, line: int) -> str:
        """The kernel whose first statement stands at this line of this file."""
        key = (unit, line)
        if key not in self._names:
            name = f"{UNITS.get(unit, unit)}:{line}"
            try:
                import os
                import re
                with open(os.path.join(build.CSRC, UNITS[unit] + ".cu")) as f:
                    lines = f.readlines()
                for i in range(line - 1, max(line - 40, -1), -1):
                    m = re.search(r"\b(\w+_kernel)\s*\(", lines[i])
                    if m:
                        name = m.group(1)
                        break
            except (OSError, KeyError):
                pass
            self._names[key] = name
        return self._names[key]

    def launches(self) -> List[dict]:
        """The records grouped into launches, in order of start: every ``blocks``
        records of one kernel and grid size, in order of their start, are one
        launch.  Times in microseconds from the first record's start."""
        rec = self.read()
        if len(rec) == 0:
            return []
        t0 = int(rec["start"].min())
        groups: Dict[tuple, List[int]] = {}
        for i in np.argsort(rec["start"], kind="stable"):
            key = (int(rec["unit"][i]), int(rec["line"][i]), int(rec["blocks"][i]))
            groups.setdefault(key, []).append(int(i))
        out = []
        for (unit, line, blocks), idx in groups.items():
            for k in range(0, len(idx), blocks):
                part = rec[idx[k:k + blocks]]
                waited = part["waited"][part["waited"] > 0]
                out.append({
                    "kernel": self.kernel_name(unit, line), "blocks": blocks, "recorded": len(part),
                    "first_start": (int(part["start"].min()) - t0) / 1e3,
                    "last_start": (int(part["start"].max()) - t0) / 1e3,
                    "first_waited": (int(waited.min()) - t0) / 1e3 if len(waited) else None,
                    "last_waited": (int(waited.max()) - t0) / 1e3 if len(waited) else None,
                    "first_end": (int(part["end"].min()) - t0) / 1e3,
                    "last_end": (int(part["end"].max()) - t0) / 1e3,
                    "sms": int(len(np.unique(part["sm"]))),
                    # points inside the kernel (timeline_mark): earliest and latest CTA, None if unused
                    "marks": [((int(col[col > 0].min()) - t0) / 1e3, (int(col.max()) - t0) / 1e3)
                              if (col > 0).any() else None for col in part["marks"].T],
                })
        out.sort(key=lambda r: r["first_start"])
        return out
