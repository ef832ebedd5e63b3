"""A profiling mode for the kernels: the device time of every launch, by name.

The reference has ``CHIBILLM_PROFILE``: every dispatch gets a command buffer of
its own, is waited for, and its GPU time is added up under a profile name that
tells shapes apart; a table sorted by time is printed at the end
(src/metal/metal_context.mm:94-102,135-169), and ``CHIBILLM_PROFILE_PASSES``
prints encode / wait / GPU / total milliseconds of each forward pass
(src/metal/metal_context.mm:459-472).

Here a :class:`LaunchProfiler` wraps the loaded libraries: every call that
launches kernels is bracketed by a pair of CUDA events on the launching
stream.  Events between launches also switch off the overlap of consecutive
kernels (programmatic dependent launch), so the times are those of each kernel
alone; steps are not replayed from CUDA graphs and no step is launched ahead
while the mode is on.  It slows generation down and is meant for finding where
the time goes, not for throughput numbers.
"""
from __future__ import annotations

import sys
import time
from typing import Callable, Dict, List, Optional, Tuple

import torch

# entry points that ask a question or set something and launch nothing
_NOT_LAUNCHES = ("chibi_gemm_bf16_splits", "chibi_gemm_bf16_splits_capped", "chibi_gemm_bf16_norm_parts", "chibi_gemm_few_rows_max",
                 "chibi_gemm_set_stream_scratch", "chibi_gemm_reset_stream_counters", "chibi_gemm_set_pair_tiles",
                 "chibi_gemm_many_rows_plan",
                 "chibi_attention_mma_head_dim", "chibi_attention_tc_head_dim")

# where M, N, K stand among the arguments of the matrix products
_PRODUCT_SIZES = {"chibi_gemm_bf16": (5, 6, 7), "chibi_gemm_bf16_rows": (5, 6, 7), "chibi_gemm_bf16_fused": (5, 6, 7),
                  "chibi_gemm_bf16_partial": (2, 3, 4), "chibi_gemm_simt": (7, 8, 9)}


def launch_name(function: str, args: tuple) -> str:
    """The name a launch is filed under: the entry point and, for matrix
    products, the weight's shape and whether few (<= 64), up to 128 (where the narrow
    products still run the few-row kernel) or many rows ran."""
    name = function[6:] if function.startswith("chibi_") else function
    where = _PRODUCT_SIZES.get(function)
    if where is not None:
        m, n, k = (int(args[i]) for i in where)
        name += f" {n}x{k} {'few rows' if m <= 64 else ('up to 128 rows' if m <= 128 else 'many rows')}"
    return name


class LaunchProfiler:
    def __init__(self):
        self.totals: Dict[str, List[float]] = {}       # name -> [calls, milliseconds]
        self._open: List[Tuple[str, torch.cuda.Event, torch.cuda.Event]] = []
        self._step_started: Optional[float] = None
        self.steps: List[dict] = []

    # ---- launches
    def timed(self, function: str, fn: Callable, args: tuple):
        start = torch.cuda.Event(enable_timing=True)
        end = torch.cuda.Event(enable_timing=True)
        start.record()
        status = fn(*args)
        end.record()
        self._open.append((launch_name(function, args), start, end))
        return status

    def _collect(self) -> Tuple[int, float]:
        """Wait for the device and file the open launches; returns their number and time."""
        torch.cuda.synchronize()
        total = 0.0
        for name, start, end in self._open:
            ms = start.elapsed_time(end)
            entry = self.totals.setdefault(name, [0, 0.0])
            entry[0] += 1
            entry[1] += ms
            total += ms
        count = len(self._open)
        self._open.clear()
        return count, total

    # ---- steps
    def begin_step(self) -> None:
        self._collect()
        self._step_started = time.perf_counter()

    def end_step(self, tokens: int) -> dict:
        encoded = time.perf_counter()
        launches, gpu_ms = self._collect()
        done = time.perf_counter()
        started = self._step_started if self._step_started is not None else encoded
        record = {"tokens": tokens, "launches": launches, "encode_ms": (encoded - started) * 1e3,
                  "wait_ms": (done - encoded) * 1e3, "gpu_ms": gpu_ms, "total_ms": (done - started) * 1e3}
        self.steps.append(record)
        self._step_started = None
        return record

    # ---- report
    def table(self) -> List[str]:
        self._collect()
        rows = sorted(self.totals.items(), key=lambda kv: -kv[1][1])
        total = sum(v[1] for _, v in rows)
        lines = []
        for name, (calls, ms) in rows:
            share = 100.0 * ms / total if total else 0.0
            lines.append(f"[cuda-profile] {name:<44} calls={calls} total_ms={ms:9.3f} "
                         f"avg_us={ms * 1e3 / calls:9.3f} share={share:5.1f}%")
        lines.append(f"[cuda-profile] {'all instrumented work':<44} total_ms={total:9.3f}")
        return lines

    def dump(self, stream=None) -> None:
        for line in self.table():
            print(line, file=stream or sys.stderr)


class ProfiledLibrary:
    """A loaded library whose launching entry points report to a profiler."""

    def __init__(self, lib, profiler: LaunchProfiler):
        self._lib, self._profiler = lib, profiler
        self._wrapped: Dict[str, Callable] = {}

    def __getattr__(self, name: str):
        fn = getattr(self._lib, name)
        if name in _NOT_LAUNCHES or not name.startswith("chibi_"):
            return fn
        wrapped = self._wrapped.get(name)
        if wrapped is None:
            profiler = self._profiler

            def wrapped(*args, _fn=fn, _name=name):
                return profiler.timed(_name, _fn, args)

            self._wrapped[name] = wrapped
        return wrapped
