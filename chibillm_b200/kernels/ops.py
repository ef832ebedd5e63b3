"""The operations the parts are made of, each a launch of a CUDA kernel of this
package.  There is no other implementation behind these calls: a tensor that
is not on a CUDA device, or a library that cannot be built or loaded, raises.

All functions write into tensors the caller provides (so a step allocates
nothing once its workspace exists) and launch on torch's current stream.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional

import torch

from . import library
from ..csrc import build

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}


class KernelError(RuntimeError):
    pass


def _code(t: torch.Tensor) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"element type {t.dtype} is not supported (float32 or bfloat16)") from None


def _need_cuda(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("chibillm_b200 runs on a CUDA device only; got a tensor on "
                              f"'{t.device}' (there is no CPU path)")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _check(status: int, what: str) -> None:
    if status == 0:
        return
    if status == -1:
        raise KernelError(f"{what}: invalid argument")
    if status == -2:
        raise KernelError(f"{what}: sizes outside what the kernel supports")
    raise KernelError(f"{what}: CUDA error {status}")


def _rows_contiguous(t: torch.Tensor, what: str) -> None:
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{what} must be 2-d with contiguous rows, got shape {tuple(t.shape)} "
                          f"strides {t.stride()}")


class PendingSum:
    """The partial sums [splits, M, N] (32-bit) of a matrix product whose K range
    was split over CTAs, waiting for a kernel that adds them up together with what
    follows the product (residual and norm, SwiGLU, per-head norm and rotation).
    The sums live in one of two scratch arrays that split products take in turn,
    so a pending sum is good until two more split products have been started; one
    that is read later than that raises instead of handing out another product's
    numbers."""

    def __init__(self, kernels, partial: torch.Tensor, splits: int, M: int, N: int,
                 turn: int = 0, stamp: Optional[int] = None):
        self.kernels, self._partial, self.splits, self.M, self.N = kernels, partial, splits, M, N
        self._turn, self._stamp = turn, stamp

    @property
    def partial(self) -> torch.Tensor:
        if self._stamp is not None and self.kernels._partial_stamps[self._turn] != self._stamp:
            raise KernelError("the partial sums of this product have been overwritten: a pending product "
                              "must be consumed before two more split products are started")
        return self._partial

    def add_into(self, residual: torch.Tensor) -> None:
        """residual += the product."""
        self.kernels.reduce_residual_rmsnorm(self, residual, None, 0.0, 0.0, None)


class ScaledRows:
    """A norm's output without the factor of each row: ``tensor`` holds
    x * (w + offset) in bfloat16 and ``ssq`` [rows, parts] sums of squares of x, so
    that RMSNorm(x)[m] = tensor[m] * rsqrt(sum(ssq[m]) / n + eps).  The factor
    commutes with a matrix product, and ``linear`` / ``linear_swiglu`` apply it to
    their sums; ``materialise`` applies it in place for any other reader."""

    def __init__(self, kernels, tensor: torch.Tensor, ssq: torch.Tensor, parts: int, eps: float, n: int):
        self.kernels, self.tensor, self.ssq, self.parts, self.eps, self.n = kernels, tensor, ssq, parts, eps, n

    @property
    def shape(self):
        return self.tensor.shape

    @property
    def dtype(self):
        return self.tensor.dtype

    def materialise(self) -> torch.Tensor:
        self.kernels.scale_rows(self)
        return self.tensor


class DeferredProduct:
    """residual += x @ w^T of many rows, not launched yet: the norm that follows
    may have the product write the norm's output as well (``finish_with_norm``);
    anybody else adds it (``add_into``)."""

    def __init__(self, kernels, x: torch.Tensor, w: torch.Tensor):
        self.kernels, self.x, self.w = kernels, x, w

    def add_into(self, residual: torch.Tensor) -> None:
        self.kernels.linear(self.x, self.w, residual, residual=residual)

    def finish_with_norm(self, residual: torch.Tensor, weight: torch.Tensor, eps: float, offset: float,
                         out: torch.Tensor, scaled_ok: bool):
        """Adds the product into ``residual`` and normalises: returns ``out`` (the
        norm's output) or, if the reader takes them, ScaledRows over ``out``."""
        k = self.kernels
        if scaled_ok:
            scaled = k.linear_residual_norm(self.x, self.w, residual, weight, eps, offset, out)
            if scaled is not None:
                return scaled
        self.add_into(residual)
        k.rmsnorm(residual, weight, eps, offset, out)
        return out


_STREAM_SCRATCH: Dict[torch.device, torch.Tensor] = {}

# torch's own fast path to the current stream's handle (a plain integer): the public
# torch.cuda.current_stream() builds a Stream object through several Python layers, a quarter
# of the host time of a step that launches a few hundred kernels
_raw_current_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


class CudaKernels:
    """The one set of operations of the product path."""

    name = "cuda"

    def __init__(self, device: torch.device, timeline: bool = False):
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device is available; chibillm_b200 has no CPU path")
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise KernelError(f"device '{device}' is not a CUDA device; chibillm_b200 has no CPU path")
        # timeline: libraries built with -DCHIBI_TIMELINE, whose CTAs note their times (kernels/timeline.py)
        self.timeline = None
        self._defines = ()
        if timeline:
            from .timeline import DEFINE, Timeline
            self.timeline = Timeline(self.device)
            self._defines = (DEFINE,)
        self.lib = self._load("chibi_kernels")
        self.profiler = None        # a LaunchProfiler while the profiling mode is on
        self._device_index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self.error = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._error_host: Optional[torch.Tensor] = None
        self.launches = 0           # kernels of this package launched so far
        self.use_tensor_cores = True
        self.tensor_core_calls = 0  # matrix products that ran on the tcgen05 kernel
        self.tcgen05_attention_variant = 0   # 0: chosen by size; 1 / 2: query tiles per CTA (for tests)
        self._scratch_buf: Optional[torch.Tensor] = None
        self.scratch_generation = 0
        self.supports_graphs = True     # every op is a plain launch on the current stream
        self._attention_libs = {}
        self._attention_tc_libs = {}
        self.use_tcgen05_attention = True
        self._partial_bufs = [None, None]
        self._partial_turn = 0
        self._partial_stamps = [0, 0]     # how often each of the two arrays has been handed out
        self._ssq_bufs = [None, None]
        self._ssq_turn = 0
        # Many rows: the product that completes the residual also writes the following RMSNorm's
        # output, up to the factor of each row, which the next product applies to its sums.
        # up to so many rows a product streams the weights once with the rows as the instruction's
        # columns (and its K range split over CTAs); beyond, the kernel for many rows runs
        self.few_rows_max = int(self.lib.chibi_gemm_few_rows_max())
        self.fold_norms = True
        self.fold_heads = True           # many rows: the q | k | v product finishes its heads itself
        # The K range of a product with few rows is split over CTAs.  Their partial sums go through
        # global scratch to a second kernel that also does what follows the product.
        self.fuse_split_products = True
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        # the many-row product shares its last, partly filled round of tiles out by K blocks and
        # needs room for one tile of partial sums per SM
        # (one per process, never freed: the library keeps the pointer)
        if self.device not in _STREAM_SCRATCH:
            _STREAM_SCRATCH.clear()
            _STREAM_SCRATCH[self.device] = torch.empty(2 * self.sm_count * 128 * 256, dtype=torch.float32,
                                                       device=self.device)
            scratch = _STREAM_SCRATCH[self.device]
            _check(self.lib.chibi_gemm_set_stream_scratch(_ptr(scratch), scratch.numel()), "stream scratch")

    def enable_profiling(self):
        """Time every launch from now on (kernels/profile.py); returns the profiler.
        Steps are no longer captured into CUDA graphs while this is on."""
        from .profile import LaunchProfiler, ProfiledLibrary
        if self.profiler is None:
            self.profiler = LaunchProfiler()
            self.lib = ProfiledLibrary(self.lib, self.profiler)
            for libs in (self._attention_libs, self._attention_tc_libs):
                for d in list(libs):
                    libs[d] = ProfiledLibrary(libs[d], self.profiler)
            self.supports_graphs = False
        return self.profiler

    def _load(self, name: str, defines=()):
        lib = library.load(name, tuple(defines) + self._defines)
        if self.timeline is not None:
            self.timeline.attach(lib, name)
        return lib

    def _profiled(self, lib):
        if self.profiler is None:
            return lib
        from .profile import ProfiledLibrary
        return ProfiledLibrary(lib, self.profiler)

    def share_out_last_round(self, enabled: bool) -> None:
        """Whether the many-row product deals the K blocks of a thinly filled last round
        of tiles out to all SMs (the default) or computes every tile whole."""
        scratch = _STREAM_SCRATCH[self.device] if enabled else None
        _check(self.lib.chibi_gemm_set_stream_scratch(_ptr(scratch), scratch.numel() if enabled else 0),
               "stream scratch")

    def pairs_of_ctas(self, mode: str = "policy", min_rows: int = 256) -> None:
        """How the many-row product uses pairs of CTAs on tiles of 256 x 256 (tcgen05.mma of 256
        rows issued by one CTA for both): "policy" where that is the fastest cut of the output
        (the default, from ``min_rows`` rows on), "never", or "always" (from 256 rows on, whenever
        the columns come in whole tiles of 256)."""
        _check(self.lib.chibi_gemm_set_pair_tiles({"never": 0, "policy": 1, "always": 2, "always narrow": 3}[mode], int(min_rows)),
               "pairs of CTAs")

    def scale_rows(self, rows: ScaledRows) -> None:
        """rows.tensor *= the factor of each row, in place."""
        t = rows.tensor
        _rows_contiguous(t, "scale_rows")
        self.launches += 1
        _check(self.lib.chibi_scale_rows(_ptr(t), t.shape[0], t.shape[1], t.stride(0), _ptr(rows.ssq), rows.parts,
                                         float(rows.eps), rows.n, self._stream()), "scale_rows")

    def linear_residual_norm(self, x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor,
                             weight: torch.Tensor, eps: float, offset: float,
                             out: torch.Tensor) -> Optional[ScaledRows]:
        """residual += x @ w^T and, from the same kernel, the RMSNorm of the new
        residual without the rows' factor (see ScaledRows).  None if the kernel for
        many rows does not take these shapes; nothing has run then."""
        M, K = x.shape
        N = w.shape[0]
        parts = self.lib.chibi_gemm_bf16_norm_parts(M, N, K)
        if not (self.use_tensor_cores and self.fold_norms and M > self.few_rows_max and parts > 0 and x.dtype == torch.bfloat16
                and w.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and residual.dtype == torch.float32
                and residual.shape == (M, N) and out.shape == (M, N) and weight.shape == (N,)
                and weight.is_contiguous() and weight.dtype in (torch.bfloat16, torch.float32)):
            return None
        _need_cuda(x, w, residual, weight, out)
        for t, what in ((x, "x"), (w, "w"), (residual, "residual"), (out, "out")):
            _rows_contiguous(t, f"linear_residual_norm: {what}")
        ssq = self._ssq_buffer(M * parts)
        norm = library.NormOut(_ptr(weight), _code(weight), float(offset), _ptr(out), out.stride(0), _ptr(ssq),
                               ssq.numel())
        status = self.lib.chibi_gemm_bf16_rows(
            _ptr(x), _ptr(w), _ptr(residual), F32, _ptr(residual), M, N, K, x.stride(0), w.stride(0),
            residual.stride(0), residual.stride(0), 0, None, ctypes.byref(norm), None, _ptr(self.error),
            self._stream())
        if status == -2:
            return None
        _check(status, "linear (+ residual, + norm output)")
        self.launches += 1
        self.tensor_core_calls += 1
        return ScaledRows(self, out, ssq, parts, eps, N)

    def _ssq_buffer(self, floats: int) -> torch.Tensor:
        """Two buffers in turn: the sums of squares of one norm are read while the
        product that follows the next norm already writes its own."""
        self._ssq_turn ^= 1
        buf = self._ssq_bufs[self._ssq_turn]
        if buf is None or buf.numel() < floats:
            buf = torch.empty(max(floats, 1 << 16), dtype=torch.float32, device=self.device)
            self._ssq_bufs[self._ssq_turn] = buf
            self.scratch_generation += 1
        return buf

    def _linear_of_scaled(self, x: ScaledRows, w: torch.Tensor, out: torch.Tensor, swiglu: bool) -> bool:
        """out = (the factor of each row) * (x.tensor @ w^T), with SwiGLU if asked,
        from the kernel for many rows; False if it does not take the shapes."""
        t = x.tensor
        M, K = t.shape
        N = w.shape[0]
        if not (self.use_tensor_cores and M > self.few_rows_max and N % 128 == 0 and w.dtype == torch.bfloat16
                and out.dtype == torch.bfloat16 and w.shape[1] == K
                and out.shape == (M, N // 2 if swiglu else N)):
            return False
        _need_cuda(t, w, out)
        for u, what in ((t, "x"), (w, "w"), (out, "out")):
            _rows_contiguous(u, f"linear: {what}")
        scale = library.RowScale(_ptr(x.ssq), x.parts, float(x.eps), x.n)
        status = self.lib.chibi_gemm_bf16_rows(
            _ptr(t), _ptr(w), _ptr(out), BF16, None, M, N, K, t.stride(0), w.stride(0), out.stride(0), 0,
            1 if swiglu else 0, ctypes.byref(scale), None, None, _ptr(self.error), self._stream())
        if status == -2:
            return False
        _check(status, "linear (rows with a factor)")
        self.launches += 1
        self.tensor_core_calls += 1
        return True

    # ---- the q | k | v product of many rows that finishes its heads itself
    def finishes_heads(self, rows: int, d: int, rotary_dim: int, dtype: torch.dtype) -> bool:
        """Whether ``linear_heads`` takes a step of so many rows with this head size."""
        return bool(self.use_tensor_cores and self.fold_heads and rows > self.few_rows_max and d == 128 and rotary_dim == d
                    and dtype == torch.bfloat16)

    def rope_table(self, positions: torch.Tensor, inv_freq: torch.Tensor, rotary_dim: int,
                   out: torch.Tensor) -> None:
        """out[t] = the cosines, then the sines, of float(positions[t]) * inv_freq[j]."""
        _need_cuda(positions, inv_freq, out)
        T, half = positions.numel(), rotary_dim // 2
        if positions.dtype != torch.int32 or inv_freq.dtype != torch.float32 or inv_freq.numel() < half \
                or out.dtype != torch.float32 or out.shape != (T, 2 * half) or not out.is_contiguous():
            raise KernelError("rope_table: int32 positions, float32 inv_freq and out [T, rotary_dim]")
        self.launches += 1
        _check(self.lib.chibi_rope_table(_ptr(positions), _ptr(inv_freq), T, half, _ptr(out), self._stream()),
               "rope_table")

    def cache_slots(self, positions: torch.Tensor, seq_of_token: torch.Tensor, seq_rows: Optional[torch.Tensor],
                    block_table: torch.Tensor, nkv: int, page_size: int, num_pages: int, d: int,
                    out: torch.Tensor) -> None:
        """out[t] = where token t's key (and value) of kv head 0 lies in a cache
        [pages, nkv, page_size, d], in elements; -1 and a recorded error if its
        block table has no page there."""
        _need_cuda(positions, seq_of_token, seq_rows, block_table, out)
        _rows_contiguous(block_table, "cache_slots: block_table")
        T = positions.numel()
        if out.dtype != torch.int64 or out.numel() != T or not out.is_contiguous():
            raise KernelError("cache_slots: out must be contiguous int64 [T]")
        self.launches += 1
        _check(self.lib.chibi_cache_slots(_ptr(positions), _ptr(seq_of_token), _ptr(seq_rows), _ptr(block_table),
                                          block_table.stride(0), T, nkv, page_size, num_pages, d, _ptr(out),
                                          _ptr(self.error), self._stream()), "cache_slots")

    def linear_heads(self, x, w: torch.Tensor, q_out: torch.Tensor, k_cache: Optional[torch.Tensor],
                     v_cache: Optional[torch.Tensor], q_norm_w: Optional[torch.Tensor],
                     k_norm_w: Optional[torch.Tensor], cos_sin: torch.Tensor, slots: Optional[torch.Tensor],
                     nq: int, nkv: int, d: int, page_size: int, eps: float, norm_offset: float) -> bool:
        """q | k | v = x @ w^T of many rows with every head finished by the product's
        own epilogue: per-head RMSNorm (if weights are given), rotation of the whole
        head with ``cos_sin`` (``rope_table``), query heads to ``q_out``, key and
        value heads to the cache slots ``slots`` (``cache_slots``).  x may be
        ScaledRows.  False if the kernel does not take the shapes; nothing has run then."""
        scale = None
        if isinstance(x, ScaledRows):
            scale = library.RowScale(_ptr(x.ssq), x.parts, float(x.eps), x.n)
            x = x.tensor
        append = k_cache is not None
        T, K = x.shape
        N = w.shape[0]
        if not self.finishes_heads(T, d, d, x.dtype) or w.dtype != torch.bfloat16 or w.shape[1] != K \
                or N != (nq + (2 * nkv if append else 0)) * d or q_out.dtype != torch.bfloat16:
            return False
        for t in (q_norm_w, k_norm_w):
            if t is not None and (t.dtype not in (torch.bfloat16, torch.float32) or t.numel() != d
                                  or not t.is_contiguous()):
                return False
        if (q_norm_w is None) != (k_norm_w is None) or (q_norm_w is not None and q_norm_w.dtype != k_norm_w.dtype):
            return False
        _need_cuda(x, w, q_out, k_cache, v_cache, q_norm_w, k_norm_w, cos_sin, slots)
        _rows_contiguous(x, "linear_heads: x")
        _rows_contiguous(w, "linear_heads: w")
        if q_out.shape != (T, nq * d) or not q_out.is_contiguous() or cos_sin.dtype != torch.float32 \
                or cos_sin.shape != (T, d) or not cos_sin.is_contiguous():
            raise KernelError("linear_heads: q_out [T, nq * d] bfloat16 and cos_sin [T, d] float32")
        if append and (k_cache.dtype != torch.bfloat16 or tuple(k_cache.shape[1:]) != (nkv, page_size, d)
                       or not k_cache.is_contiguous() or v_cache is None or v_cache.shape != k_cache.shape
                       or not v_cache.is_contiguous() or slots is None or slots.dtype != torch.int64
                       or slots.numel() != T):
            raise KernelError("linear_heads: caches [pages, nkv, page_size, d] bfloat16 and int64 slots [T]")
        heads = library.HeadsOut(_ptr(cos_sin), _ptr(slots) if append else None, _ptr(q_out), _ptr(k_cache),
                                 _ptr(v_cache), _ptr(q_norm_w), _ptr(k_norm_w),
                                 _code(q_norm_w) if q_norm_w is not None else F32, nq, nkv if append else 0,
                                 page_size, float(eps), float(norm_offset))
        status = self.lib.chibi_gemm_bf16_rows(
            _ptr(x), _ptr(w), None, BF16, None, T, N, K, x.stride(0), w.stride(0), N, 0, 0,
            ctypes.byref(scale) if scale is not None else None, None, ctypes.byref(heads), _ptr(self.error),
            self._stream())
        if status == -2:
            return False
        _check(status, "linear (q | k | v heads)")
        self.launches += 1
        self.tensor_core_calls += 1
        return True

    def _scratch(self, floats: int) -> torch.Tensor:
        """32-bit scratch for kernels that split a reduction over several CTAs."""
        if self._scratch_buf is None or self._scratch_buf.numel() < floats:
            self._scratch_buf = torch.empty(max(floats, 1 << 22), dtype=torch.float32, device=self.device)
            self.scratch_generation += 1
        return self._scratch_buf

    # ------------------------------------------------------------------ helpers
    def _stream(self) -> int:
        """The handle of this device's current stream (asked for at every launch:
        the caller may be inside a stream capture or a stream context)."""
        if _raw_current_stream is not None:
            return _raw_current_stream(self._device_index)
        return torch.cuda.current_stream(self.device).cuda_stream

    def error_word_async(self) -> None:
        """Starts the copy of the error word to the host; ``check_error_copy`` reads it
        once the caller has waited for an event recorded after this call."""
        if self._error_host is None:
            self._error_host = torch.zeros(1, dtype=torch.int32, pin_memory=True)
        self._error_host.copy_(self.error, non_blocking=True)

    def check_error_copy(self) -> None:
        if self._error_host is not None:
            self._raise_for(int(self._error_host[0]))

    def check_error_word(self) -> None:
        """Synchronises and raises if a kernel met an index outside its tables."""
        self._raise_for(int(self.error.item()))

    def _raise_for(self, code: int) -> None:
        if code:
            self.error.zero_()
            # a shared-out round of tiles that gave up may have left its counters non-zero
            self.lib.chibi_gemm_reset_stream_counters(self._stream())
            what = {1: "a token id outside the vocabulary", 2: "a page id outside the pool (append)",
                    3: "a page id outside the pool (attention)",
                    4: "a block-table update outside the table",
                    11: "a wait that ran out (matrix product: loader)",
                    12: "a wait that ran out (matrix product: tensor-core issuer)",
                    13: "a wait that ran out (matrix product: epilogue)",
                    14: "a wait that ran out (matrix product: accumulator hand-over)",
                    15: "a wait that ran out (matrix product: partial sums of a shared tile)",
                    16: "a wait that ran out (matrix product: slot of a shared tile)",
                    17: "a wait that ran out (matrix product by pairs of CTAs: loader)",
                    18: "a wait that ran out (matrix product by pairs of CTAs: tensor-core issuer)",
                    19: "a wait that ran out (matrix product by pairs of CTAs: epilogue)",
                    20: "a wait that ran out (matrix product by pairs of CTAs: accumulator hand-over)",
                    **{c: f"a wait that ran out (tcgen05 attention, point {c})" for c in range(21, 30)}}.get(code, f"code {code}")
            raise KernelError(f"a kernel refused {what}")

    # ------------------------------------------------------------------ ops
    def embed(self, tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> None:
        _need_cuda(tokens, table, out)
        if tokens.dtype != torch.int32 or not tokens.is_contiguous():
            raise KernelError("embed: tokens must be contiguous int32")
        _rows_contiguous(table, "embed: table")
        if not out.is_contiguous() or out.shape != (tokens.numel(), table.shape[1]):
            raise KernelError("embed: out must be contiguous [tokens, hidden]")
        if not table.is_contiguous():
            raise KernelError("embed: table must be contiguous")
        self.launches += 1
        _check(self.lib.chibi_embed(_ptr(tokens), _ptr(table), _code(table), _ptr(out), _code(out),
                                    tokens.numel(), table.shape[1], table.shape[0],
                                    _ptr(self.error), self._stream()), "embed")

    def rmsnorm(self, x: torch.Tensor, weight: torch.Tensor, eps: float, offset: float,
                out: torch.Tensor) -> None:
        """x, out: [groups, n] (rows may be strided); weight [n]."""
        _need_cuda(x, weight, out)
        _rows_contiguous(x, "rmsnorm: x")
        _rows_contiguous(out, "rmsnorm: out")
        n = x.shape[1]
        if weight.shape != (n,) or not weight.is_contiguous() or out.shape != x.shape:
            raise KernelError(f"rmsnorm: weight {tuple(weight.shape)} / out {tuple(out.shape)} do not "
                              f"match x {tuple(x.shape)}")
        self.launches += 1
        _check(self.lib.chibi_rmsnorm(_ptr(x), _code(x), _ptr(weight), _code(weight), _ptr(out),
                                      _code(out), x.shape[0], n, x.stride(0), out.stride(0),
                                      float(eps), float(offset), self._stream()), "rmsnorm")

    def _partial_buffer(self, floats: int) -> torch.Tensor:
        self._partial_turn ^= 1
        self._partial_stamps[self._partial_turn] += 1
        buf = self._partial_bufs[self._partial_turn]
        if buf is None or buf.numel() < floats:
            buf = torch.empty(max(floats, 1 << 21), dtype=torch.float32, device=self.device)
            self._partial_bufs[self._partial_turn] = buf
            self.scratch_generation += 1
        return buf

    def linear_partial(self, x: torch.Tensor, w: torch.Tensor, max_splits: int = 0) -> Optional[PendingSum]:
        """Start x @ w^T with the K range split over CTAs and leave the partial
        sums for a fused consumer; None if this product is not one that is split
        (then use ``linear``).  ``max_splits``: at most so many splits (a consumer
        that fetches only so many partial sums in one go says so)."""
        if isinstance(x, ScaledRows):
            return None                  # many rows: such a product is not split
        if not (self.use_tensor_cores and self.fuse_split_products and x.is_cuda
                and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16):
            return None
        _rows_contiguous(x, "linear: x")
        _rows_contiguous(w, "linear: w")
        M, K = x.shape
        N = w.shape[0]
        if w.shape[1] != K:
            raise KernelError(f"linear: shapes x {tuple(x.shape)} w {tuple(w.shape)}")
        splits = self.lib.chibi_gemm_bf16_splits_capped(M, N, K, int(max_splits))
        if splits <= 1 or N % 4 != 0:
            return None
        buf = self._partial_buffer(splits * M * N)
        status = self.lib.chibi_gemm_bf16_partial(_ptr(x), _ptr(w), M, N, K, x.stride(0), w.stride(0),
                                                  _ptr(buf), buf.numel(), int(max_splits), _ptr(self.error),
                                                  self._stream())
        if status == -2:
            return None
        _check(status, "linear (split product)")
        self.launches += 1
        self.tensor_core_calls += 1
        return PendingSum(self, buf[:splits * M * N].view(splits, M, N), splits, M, N,
                          self._partial_turn, self._partial_stamps[self._partial_turn])

    @staticmethod
    def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> Optional[torch.Tensor]:
        """[gate; up] rearranged for ``linear_swiglu``: blocks of 64 gate rows, each
        followed by the 64 up rows of the same features.  None if the sizes do not
        allow it (the number of features must be a multiple of 64)."""
        inter, k = gate.shape
        if gate.shape != up.shape or inter % 64 != 0 or k % 8 != 0 or gate.dtype != torch.bfloat16 \
                or up.dtype != torch.bfloat16:
            return None
        return torch.stack([gate.view(inter // 64, 64, k), up.view(inter // 64, 64, k)], dim=1).reshape(2 * inter, k).contiguous()

    def linear_swiglu(self, x: torch.Tensor, w_interleaved: torch.Tensor, out: torch.Tensor) -> bool:
        """out[M, I] = silu(x @ gate^T) * (x @ up^T) in one kernel, with the weights
        as ``interleave_gate_up`` arranges them.  False if the kernel refuses the
        shapes (the caller then takes the two-kernel way)."""
        if isinstance(x, ScaledRows):
            if self._linear_of_scaled(x, w_interleaved, out, swiglu=True):
                return True
            x = x.materialise()
        _need_cuda(x, w_interleaved, out)
        _rows_contiguous(x, "linear_swiglu: x")
        _rows_contiguous(w_interleaved, "linear_swiglu: w")
        _rows_contiguous(out, "linear_swiglu: out")
        M, K = x.shape
        N = w_interleaved.shape[0]
        if w_interleaved.shape[1] != K or out.shape != (M, N // 2) or out.dtype != torch.bfloat16 \
                or x.dtype != torch.bfloat16 or w_interleaved.dtype != torch.bfloat16:
            raise KernelError("linear_swiglu: shapes or element types")
        if not self.use_tensor_cores:
            return False
        pending = self.linear_partial(x, w_interleaved) if M <= self.few_rows_max else None
        if pending is not None or M <= 64:
            if pending is None:
                # a shape whose K range is not split: the whole product, then the same kernel
                # that otherwise adds up the splits (here: one) applies SwiGLU
                buf = self._partial_buffer(M * N)
                self.linear(x, w_interleaved, buf[:M * N].view(M, N))
                pending = PendingSum(self, buf[:M * N].view(1, M, N), 1, M, N, self._partial_turn,
                                     self._partial_stamps[self._partial_turn])
            self.reduce_swiglu(pending, out, interleaved=True)
            return True
        status = self.lib.chibi_gemm_bf16_fused(
            _ptr(x), _ptr(w_interleaved), _ptr(out), BF16, None, M, N, K, x.stride(0),
            w_interleaved.stride(0), out.stride(0), 0, 1, _ptr(self.error), self._stream())
        if status == -2:
            return False
        _check(status, "linear_swiglu")
        self.launches += 1
        self.tensor_core_calls += 1
        return True

    def reduce_residual_rmsnorm(self, pending: PendingSum, residual: torch.Tensor,
                                weight: Optional[torch.Tensor], eps: float, offset: float,
                                out: Optional[torch.Tensor]) -> None:
        """residual += pending; out = RMSNorm(residual) if a weight is given."""
        _need_cuda(residual, weight, out)
        _rows_contiguous(residual, "reduce_residual_rmsnorm: residual")
        if residual.dtype != torch.float32 or residual.shape != (pending.M, pending.N):
            raise KernelError("reduce_residual_rmsnorm: residual must be float32 [M, N]")
        if weight is not None:
            _rows_contiguous(out, "reduce_residual_rmsnorm: out")
            if weight.shape != (pending.N,) or out.shape != residual.shape:
                raise KernelError("reduce_residual_rmsnorm: weight / out shapes")
        status = self.lib.chibi_reduce_residual_rmsnorm(
            _ptr(pending.partial), pending.splits, pending.M, pending.N, _ptr(residual), residual.stride(0),
            _ptr(weight), _code(weight) if weight is not None else F32, _ptr(out),
            _code(out) if out is not None else F32, out.stride(0) if out is not None else 0,
            float(eps), float(offset), self._stream())
        if status == -2:
            # a width the fused kernel does not take: add up, then normalise
            self.launches += 1
            _check(self.lib.chibi_add_into(_ptr(residual), _ptr(pending.partial[0]), F32,
                                           residual.numel(), self._stream()), "add_into")
            for s in range(1, pending.splits):
                self.launches += 1
                _check(self.lib.chibi_add_into(_ptr(residual), _ptr(pending.partial[s]), F32,
                                               residual.numel(), self._stream()), "add_into")
            if weight is not None:
                self.rmsnorm(residual, weight, eps, offset, out)
            return
        self.launches += 1
        _check(status, "reduce_residual_rmsnorm")

    def reduce_swiglu(self, pending: PendingSum, out: torch.Tensor, interleaved: bool = False) -> None:
        """out = silu(gate) * up from the pending [gate | up] product (or, with
        ``interleaved``, from a product with ``interleave_gate_up`` weights)."""
        _need_cuda(out)
        inter = pending.N // 2
        if not out.is_contiguous() or out.shape != (pending.M, inter):
            raise KernelError("reduce_swiglu: out must be contiguous [M, N / 2]")
        self.launches += 1
        _check(self.lib.chibi_reduce_swiglu(_ptr(pending.partial), pending.splits, pending.M, inter,
                                            _ptr(out), _code(out), 1 if interleaved else 0,
                                            self._stream()), "reduce_swiglu")

    def qk_norm_rope_append_partial(self, pending: PendingSum, q_out, k_cache, v_cache, q_norm_w, k_norm_w,
                                    inv_freq, rotary_dim, eps, norm_offset, positions, seq_of_token,
                                    block_table, nq, nkv, d, page_size, seq_rows=None) -> None:
        """qk_norm_rope_append on a pending q | k | v product (bfloat16 outputs)."""
        _need_cuda(q_out, k_cache, v_cache, q_norm_w, k_norm_w, inv_freq, positions, seq_of_token,
                   block_table, seq_rows)
        T = pending.M
        append = k_cache is not None
        width = (nq + 2 * nkv) * d if append else nq * d
        if pending.N != width or q_out.shape != (T, nq * d) or q_out.dtype != torch.bfloat16 \
                or not q_out.is_contiguous():
            raise KernelError("qk_norm_rope_append_partial: shapes")
        if append and (k_cache.dtype != torch.bfloat16 or tuple(k_cache.shape[1:]) != (nkv, page_size, d)
                       or not k_cache.is_contiguous() or not v_cache.is_contiguous()):
            raise KernelError("qk_norm_rope_append_partial: cache")
        w_type = _code(q_norm_w) if q_norm_w is not None else F32
        self.launches += 1
        _check(self.lib.chibi_qk_norm_rope_append_partial(
            _ptr(pending.partial), pending.splits, T, width, _ptr(q_out), _ptr(k_cache), _ptr(v_cache),
            _ptr(q_norm_w), _ptr(k_norm_w), w_type, _ptr(inv_freq), _ptr(positions), _ptr(seq_of_token),
            _ptr(seq_rows), _ptr(block_table), block_table.stride(0) if append else 0, nq, nkv, d,
            int(rotary_dim), page_size, k_cache.shape[0] if append else 0, float(eps), float(norm_offset),
            1 if append else 0, _ptr(self.error), self._stream()), "qk_norm_rope_append_partial")

    def linear(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor,
               residual: Optional[torch.Tensor] = None, defer: bool = False) -> Optional[PendingSum]:
        """out[M, N] = x[M, K] @ w[N, K]^T (+ residual, 32-bit, may alias out).
        With ``defer`` (only together with a residual that aliases out) a split
        product is left pending -- the caller adds it later -- and is returned."""
        if isinstance(x, ScaledRows):
            if residual is None and self._linear_of_scaled(x, w, out, swiglu=False):
                return None
            x = x.materialise()
        if defer and residual is not None and residual is out:
            pending = self.linear_partial(x, w)
            if pending is not None:
                return pending
            if self.use_tensor_cores and self.fold_norms and x.shape[0] > self.few_rows_max and x.dtype == torch.bfloat16 \
                    and w.dtype == torch.bfloat16 and residual.dtype == torch.float32:
                return DeferredProduct(self, x, w)
        _need_cuda(x, w, out, residual)
        _rows_contiguous(x, "linear: x")
        _rows_contiguous(w, "linear: w")
        _rows_contiguous(out, "linear: out")
        M, K = x.shape
        N = w.shape[0]
        if w.shape[1] != K or out.shape != (M, N):
            raise KernelError(f"linear: shapes x {tuple(x.shape)} w {tuple(w.shape)} out {tuple(out.shape)}")
        if residual is not None:
            _rows_contiguous(residual, "linear: residual")
            if residual.dtype != torch.float32 or residual.shape != (M, N):
                raise KernelError("linear: residual must be float32 [M, N]")
        if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and self.use_tensor_cores:
            splits = self.lib.chibi_gemm_bf16_splits(M, N, K)
            if splits > 0:
                scratch = self._scratch(splits * M * N) if splits > 1 else None
                status = self.lib.chibi_gemm_bf16(
                    _ptr(x), _ptr(w), _ptr(out), _code(out), _ptr(residual), M, N, K, x.stride(0),
                    w.stride(0), out.stride(0), residual.stride(0) if residual is not None else 0,
                    _ptr(scratch), scratch.numel() if scratch is not None else 0, _ptr(self.error),
                    self._stream())
                if status == 0:
                    self.launches += 2 if splits > 1 else 1
                    self.tensor_core_calls += 1
                    return
                if status != -2:
                    _check(status, "linear (tensor cores)")
        self.launches += 1
        _check(self.lib.chibi_gemm_simt(
            _ptr(x), _code(x), _ptr(w), _code(w), _ptr(out), _code(out), _ptr(residual), M, N, K,
            x.stride(0), w.stride(0), out.stride(0),
            residual.stride(0) if residual is not None else 0, self._stream()), "linear")

    def qk_norm_rope_append(self, qkv: torch.Tensor, q_out: torch.Tensor,
                            k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                            q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor],
                            inv_freq: Optional[torch.Tensor], rotary_dim: int, eps: float,
                            norm_offset: float, positions: torch.Tensor,
                            seq_of_token: torch.Tensor, block_table: Optional[torch.Tensor],
                            nq: int, nkv: int, d: int, page_size: int,
                            seq_rows: Optional[torch.Tensor] = None) -> None:
        """Per head: RMSNorm (when a weight is given), split-half rotation of the
        first ``rotary_dim`` features, then q -> q_out, k and v -> cache pages.
        qkv: [T, (nq + 2 nkv) d], or [T, nq d] when no cache is given (the layer
        then reads another layer's cache).  Cache: [pages, nkv, page_size, d].
        Sequence s uses row ``seq_rows[s]`` of the block table (row s when None)."""
        _need_cuda(qkv, q_out, k_cache, v_cache, q_norm_w, k_norm_w, inv_freq, positions,
                   seq_of_token, block_table, seq_rows)
        _rows_contiguous(qkv, "qk_norm_rope_append: qkv")
        T = qkv.shape[0]
        append = k_cache is not None
        width = (nq + 2 * nkv) * d if append else nq * d
        if qkv.shape[1] < width or not q_out.is_contiguous() or q_out.shape != (T, nq * d):
            raise KernelError("qk_norm_rope_append: qkv / q_out shapes")
        if q_out.dtype != qkv.dtype:
            raise KernelError("qk_norm_rope_append: q_out must have qkv's element type")
        if (q_norm_w is None) != (k_norm_w is None):
            raise KernelError("qk_norm_rope_append: give both norm weights or none")
        if rotary_dim and (inv_freq is None or inv_freq.dtype != torch.float32
                           or inv_freq.numel() < rotary_dim // 2):
            raise KernelError("qk_norm_rope_append: inv_freq must hold rotary_dim/2 float32 values")
        num_pages = 0
        table_stride = 0
        if append:
            if (k_cache.shape != v_cache.shape or k_cache.dim() != 4 or not k_cache.is_contiguous()
                    or not v_cache.is_contiguous() or tuple(k_cache.shape[1:]) != (nkv, page_size, d)):
                raise KernelError(f"qk_norm_rope_append: cache shape {tuple(k_cache.shape)}")
            num_pages = k_cache.shape[0]
            _rows_contiguous(block_table, "qk_norm_rope_append: block_table")
            table_stride = block_table.stride(0)
        w_type = _code(q_norm_w) if q_norm_w is not None else F32
        self.launches += 1
        _check(self.lib.chibi_qk_norm_rope_append(
            _ptr(qkv), _code(qkv), qkv.stride(0), _ptr(q_out), _ptr(k_cache), _ptr(v_cache),
            _code(k_cache) if append else F32, _ptr(q_norm_w), _ptr(k_norm_w), w_type,
            _ptr(inv_freq), _ptr(positions), _ptr(seq_of_token), _ptr(seq_rows), _ptr(block_table),
            table_stride, T,
            nq, nkv, d, int(rotary_dim), page_size, num_pages, float(eps), float(norm_offset),
            1 if append else 0, _ptr(self.error), self._stream()), "qk_norm_rope_append")

    def attention(self, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                  out: torch.Tensor, block_table: torch.Tensor, q_start: torch.Tensor,
                  ctx_len: torch.Tensor, seq_of_token: torch.Tensor, positions: torch.Tensor,
                  nq: int, nkv: int, d: int, page_size: int, scale: float,
                  window: Optional[int], max_q_len: int, max_ctx_len: int, min_q_len: int = 0,
                  seq_rows: Optional[torch.Tensor] = None) -> None:
        """Causal attention of every token over its sequence's pages.  bfloat16
        with a head size that is a multiple of 16 runs on the tensor cores (one
        library per head size, compiled when first needed); everything else, the
        32-bit path included, runs the plain kernel."""
        _need_cuda(q, k_cache, v_cache, out, block_table, q_start, ctx_len, seq_of_token, positions,
                   seq_rows)
        T = q.shape[0]
        if not q.is_contiguous() or not out.is_contiguous() or q.shape != (T, nq * d) or out.shape != q.shape:
            raise KernelError("attention: q / out must be contiguous [T, nq*d]")
        if out.dtype != q.dtype:
            raise KernelError("attention: out must have q's element type")
        if (k_cache.shape != v_cache.shape or k_cache.dim() != 4 or not k_cache.is_contiguous()
                or not v_cache.is_contiguous() or tuple(k_cache.shape[1:]) != (nkv, page_size, d)):
            raise KernelError(f"attention: cache shape {tuple(k_cache.shape)}")
        _rows_contiguous(block_table, "attention: block_table")
        if (self.use_tensor_cores and q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
                and d % 16 == 0 and d <= 256):
            self._attention_mma(q, k_cache, v_cache, out, block_table, q_start, ctx_len, nq, nkv, d,
                                page_size, scale, window, max_q_len, max_ctx_len, min_q_len, seq_rows)
            return
        self.launches += 1
        _check(self.lib.chibi_attention_generic(
            _ptr(q), _code(q), _ptr(k_cache), _ptr(v_cache), _code(k_cache), _ptr(out),
            _ptr(block_table), block_table.stride(0), _ptr(q_start), _ptr(ctx_len),
            _ptr(seq_of_token), _ptr(seq_rows), _ptr(positions), T, nq, nkv, d, page_size,
            k_cache.shape[0],
            float(scale), int(window or 0), _ptr(self.error), self._stream()), "attention")

    def decode_attention_splits(self, seqs: int, nq: int, nkv: int, max_ctx_len: int) -> int:
        """Key ranges per sequence of the decode attention kernel: as many CTAs as
        are resident at once (two per SM) and no more, so that no CTA waits for a
        second round; at least 128 keys per range (two tiles for each of a CTA's
        four warps) and at most 32 ranges: every range costs its CTA a prologue and
        the merge a partial result to fetch (one sequence of 2,048 keys: 33 ranges
        1.250 ms a step of 12 layers, 16 ranges 1.207; of 8,192 keys: 37 ranges
        1.296, 32 ranges 1.279, 64 ranges 1.374)."""
        ctas = seqs * nkv * ((nq // nkv + 15) // 16)
        slots = 2 * self.sm_count
        if ctas <= slots:
            return max(1, min(slots // ctas, -(-max_ctx_len // 128), 32))
        # More CTAs than slots even with one range each: a last round with a few CTAs in it
        # costs as much as a full one (38 sequences x 8 kv heads = 304 CTAs on 296 slots: 21 %
        # of a step more than 36 sequences).  With s ranges there are ceil(ctas * s / slots)
        # rounds of 1 / s of the keys each, and every CTA pays for its start and for its share
        # of the merge what 0.03 of the keys + 200 keys take (fitted to steps of 12 layers at 38
        # to 128 sequences of 2,048 keys and of 6 layers at 40 to 96 sequences of 8,192, the query
        # rows ready in memory): the s that makes rounds * (1 / s + that) least, more ranges only
        # where they gain a twentieth, at most four, of 512 keys or more.
        start = 0.03 + 200.0 / max(max_ctx_len, 1)
        best, least = 1, -(-ctas // slots) * (1.0 + start)
        for s in range(2, 5):
            if max_ctx_len // s < 512:
                break
            cost = -(-ctas * s // slots) * (1.0 / s + start)
            if cost < 0.95 * least:
                best, least = s, cost
        return best

    def prompt_attention_key_ranges(self, seqs: int, nq: int, nkv: int, max_q_len: int, max_ctx_len: int) -> int:
        """Key ranges per row tile of the tcgen05 prompt attention: 1 unless the step
        has so few query rows that the CTAs (a tile of 128 rows for each kv head and
        sequence) fill half the SMs or less while the context is long; then as many
        ranges as fill the SMs, of at least 512 keys each, at most eight."""
        ctas = -(-max_q_len * (nq // nkv) // 128) * nkv * seqs
        if ctas * 2 > self.sm_count or max_ctx_len < 1024:
            return 1
        return max(1, min(8, self.sm_count // ctas, max_ctx_len // 512))

    def _attention_mma(self, q, k_cache, v_cache, out, block_table, q_start, ctx_len, nq, nkv, d,
                       page_size, scale, window, max_q_len, max_ctx_len, min_q_len, seq_rows) -> None:
        lib = self._attention_libs.get(d)
        if lib is None:
            lib = self._load("chibi_attention_mma", (f"CHIBI_HEAD_DIM={d}",))
            if lib.chibi_attention_mma_head_dim() != d:
                raise KernelError(f"the attention library for head size {d} was built for another size")
            lib = self._attention_libs[d] = self._profiled(lib)
        seqs = ctx_len.numel()
        mode = 1 if max_q_len == 1 else (2 if min_q_len > 1 else 3)
        if mode & 2 and self.use_tcgen05_attention and d in build.TCGEN05_ATTENTION_HEAD_DIMS \
                and page_size >= 8 and 128 % page_size == 0:
            # prompt portions on tcgen05; one-token sequences stay with the split-key kernel
            tc = self._attention_tc_libs.get(d)
            if tc is None:
                tc = self._load("chibi_attention_tc", (f"CHIBI_HEAD_DIM={d}",))
                if tc.chibi_attention_tc_head_dim() != d:
                    raise KernelError(f"the tcgen05 attention library for head size {d} was built for another size")
                tc = self._attention_tc_libs[d] = self._profiled(tc)
            kv_splits = self.prompt_attention_key_ranges(seqs, nq, nkv, max_q_len, max_ctx_len)
            part = self._scratch(q.shape[0] * nq * kv_splits * (d + 2)) if kv_splits > 1 else None
            status = tc.chibi_attention_prefill_tc(
                _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), block_table.stride(0),
                _ptr(seq_rows), _ptr(q_start), _ptr(ctx_len), seqs, nq, nkv, page_size, k_cache.shape[0],
                float(scale), int(window or 0), 1 if mode & 1 else 0, int(max_q_len),
                int(self.tcgen05_attention_variant), kv_splits, _ptr(part),
                part.numel() if part is not None else 0, q.shape[0], _ptr(self.error), self._stream())
            if status == 0:
                # (key ranges belong to the kernel with one query tile per CTA, and bring a merge kernel)
                self.launches += 2 if kv_splits > 1 and self.tcgen05_attention_variant != 2 else 1
                mode &= 1
                if mode == 0:
                    return
            elif status != -2:
                _check(status, "attention (tcgen05)")
        splits, scratch = 1, None
        if mode & 1:
            splits = self.decode_attention_splits(seqs, nq, nkv, max_ctx_len)
            if splits > 1:
                scratch = self._scratch(seqs * nq * splits * (d + 2))
        status = lib.chibi_attention_mma(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), block_table.stride(0),
            _ptr(seq_rows), _ptr(q_start), _ptr(ctx_len), seqs, nq, nkv, page_size, k_cache.shape[0], float(scale),
            int(window or 0), mode, int(max_q_len), splits, _ptr(scratch),
            scratch.numel() if scratch is not None else 0, _ptr(self.error), self._stream())
        self.launches += (1 if mode & 1 else 0) + (1 if mode & 1 and splits > 1 else 0) + (1 if mode & 2 else 0)
        _check(status, "attention (tensor cores)")

    def attention_decode_from_partial(self, pending: PendingSum, k_cache: torch.Tensor, v_cache: torch.Tensor,
                                      out: torch.Tensor, block_table: torch.Tensor, q_start: torch.Tensor,
                                      ctx_len: torch.Tensor, nq: int, nkv: int, d: int, page_size: int,
                                      scale: float, window: Optional[int], max_ctx_len: int,
                                      q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor],
                                      inv_freq: torch.Tensor, rotary_dim: int, eps: float, norm_offset: float,
                                      append: bool, seq_rows: Optional[torch.Tensor] = None) -> bool:
        """Decode attention straight from the pending q | k | v product of a step in
        which every sequence brings one token: the attention kernel adds the partial
        sums, applies the per-head norm and the rotation and appends the new key and
        value itself.  False if the kernel does not take these sizes (the caller then
        runs ``qk_norm_rope_append_partial`` and ``attention``)."""
        if not (self.use_tensor_cores and d == 128 and rotary_dim == d and nq // nkv <= 6
                and k_cache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16):
            return False
        # More CTAs than are resident at once (from 38 sequences of 8 kv heads on): the sequences are
        # then cut into key ranges so that the rounds come out even, and every range's CTA would add
        # up, normalise and rotate the same query rows again; one kernel that leaves them in memory
        # and the attention kernel after it are 1 to 6 % of a step faster (12 layers, 2,048 keys,
        # 38 / 48 / 64 / 96 / 128 sequences: 2.39 / 2.50 / 2.68 / 3.47 / 4.17 -> 2.29 / 2.39 /
        # 2.65 / 3.40 / 4.09 ms).
        if ctx_len.numel() * nkv * ((nq // nkv + 15) // 16) > 2 * self.sm_count:
            return False
        for w in (q_norm_w, k_norm_w):
            if w is not None and w.dtype != torch.bfloat16:
                return False
        _need_cuda(k_cache, v_cache, out, block_table, q_start, ctx_len, seq_rows, q_norm_w, k_norm_w, inv_freq)
        seqs = ctx_len.numel()
        width = (nq + 2 * nkv) * d if append else nq * d
        if pending.M != seqs or pending.N != width or out.shape != (seqs, nq * d) or not out.is_contiguous() \
                or tuple(k_cache.shape[1:]) != (nkv, page_size, d) or not k_cache.is_contiguous() \
                or not v_cache.is_contiguous():
            raise KernelError("attention_decode_from_partial: shapes")
        lib = self._attention_libs.get(d)
        if lib is None:
            lib = self._load("chibi_attention_mma", (f"CHIBI_HEAD_DIM={d}",))
            lib = self._attention_libs[d] = self._profiled(lib)
        splits = self.decode_attention_splits(seqs, nq, nkv, max_ctx_len)
        scratch = self._scratch(seqs * nq * splits * (d + 2)) if splits > 1 else None
        status = lib.chibi_attention_decode_fused(
            _ptr(pending.partial), pending.splits, width, seqs, _ptr(k_cache), _ptr(v_cache), _ptr(out),
            _ptr(block_table), block_table.stride(0), _ptr(seq_rows), _ptr(q_start), _ptr(ctx_len), seqs, nq, nkv,
            page_size, k_cache.shape[0], float(scale), int(window or 0), splits, _ptr(scratch),
            scratch.numel() if scratch is not None else 0, _ptr(q_norm_w), _ptr(k_norm_w), _ptr(inv_freq),
            float(eps), float(norm_offset), 1 if append else 0, _ptr(self.error), self._stream())
        if status == -2:
            return False
        _check(status, "attention (decode, from the partial sums)")
        self.launches += 2 if splits > 1 else 1
        return True

    def apply_table_updates(self, table: torch.Tensor, updates: torch.Tensor, capacity: int) -> None:
        """table[row][index] = page for the (row, index, page) triples that follow
        the count in ``updates`` (int32: [count, row, index, page, ...])."""
        _need_cuda(table, updates)
        if table.dtype != torch.int32 or updates.dtype != torch.int32 or table.dim() != 2 \
                or not table.is_contiguous() or updates.numel() < 1 + 3 * capacity:
            raise KernelError("apply_table_updates: int32 table [rows, blocks] and 1 + 3 * capacity updates")
        self.launches += 1
        _check(self.lib.chibi_apply_table_updates(_ptr(table), table.shape[1], table.shape[0],
                                                  _ptr(updates), int(capacity), _ptr(self.error),
                                                  self._stream()), "apply_table_updates")

    def swiglu(self, gate_up: torch.Tensor, out: torch.Tensor) -> None:
        _need_cuda(gate_up, out)
        if not gate_up.is_contiguous() or not out.is_contiguous() or gate_up.shape[1] != 2 * out.shape[1] \
                or gate_up.shape[0] != out.shape[0]:
            raise KernelError("swiglu: gate_up must be contiguous [T, 2I] and out [T, I]")
        self.launches += 1
        _check(self.lib.chibi_swiglu(_ptr(gate_up), _code(gate_up), _ptr(out), _code(out),
                                     out.shape[0], out.shape[1], self._stream()), "swiglu")

    def gather_rows(self, x: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
        _need_cuda(x, rows, out)
        if not x.is_contiguous() or not out.is_contiguous() or rows.dtype != torch.int32 \
                or out.shape != (rows.numel(), x.shape[1]):
            raise KernelError("gather_rows: shapes")
        self.launches += 1
        _check(self.lib.chibi_gather_rows(_ptr(x), _code(x), _ptr(rows), _ptr(out), _code(out),
                                          rows.numel(), x.shape[1], x.shape[0], self._stream()),
               "gather_rows")

    def cast(self, x: torch.Tensor, out: torch.Tensor) -> None:
        _need_cuda(x, out)
        if not x.is_contiguous() or not out.is_contiguous() or x.numel() != out.numel():
            raise KernelError("cast: shapes")
        self.launches += 1
        _check(self.lib.chibi_cast(_ptr(x), _code(x), _ptr(out), _code(out), x.numel(),
                                   self._stream()), "cast")

    def add_into(self, acc: torch.Tensor, x: torch.Tensor) -> None:
        _need_cuda(acc, x)
        if acc.dtype != torch.float32 or not acc.is_contiguous() or not x.is_contiguous() \
                or acc.numel() != x.numel():
            raise KernelError("add_into: acc must be contiguous float32 of x's size")
        self.launches += 1
        _check(self.lib.chibi_add_into(_ptr(acc), _ptr(x), _code(x), x.numel(), self._stream()),
               "add_into")

    def sample(self, logits: torch.Tensor, temperature: Optional[torch.Tensor],
               uniform: Optional[torch.Tensor], out: torch.Tensor) -> None:
        """Greedy rows (temperature <= 0 or None) take the arg max, ties to the
        lowest id; other rows sample by inverse CDF with the given uniform."""
        _need_cuda(logits, temperature, uniform, out)
        _rows_contiguous(logits, "sample: logits")
        if logits.dtype != torch.float32 or out.dtype != torch.int32 or out.numel() != logits.shape[0]:
            raise KernelError("sample: logits float32 [R, V], out int32 [R]")
        for t in (temperature, uniform):
            if t is not None and (t.dtype != torch.float32 or t.numel() != logits.shape[0]):
                raise KernelError("sample: temperature / uniform must be float32 [R]")
        scratch = self._scratch(logits.shape[0] * 128) if temperature is None else None
        self.launches += 2 if temperature is None else 1
        _check(self.lib.chibi_sample(_ptr(logits), logits.stride(0), logits.shape[0], logits.shape[1],
                                     _ptr(temperature), _ptr(uniform), _ptr(out), _ptr(scratch),
                                     scratch.numel() if scratch is not None else 0, self._stream()),
               "sample")
