"""Interfaces of the parts a decoder is put together from, and their registries.

A part is built from its spec (sizes and constants as fields) and the names of
its tensors.  It declares which tensors it expects, takes them when they are
loaded, says what cache it needs, and runs on a batch.  No part knows which
model it is in.

Kinds are looked up in registries, so a new mixer, feed-forward, norm, position
encoding or block arrangement is a class plus one ``register_*`` call; nothing
in the framework's files has to change for it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple

import torch


# ------------------------------------------------------------------ runtime
@dataclass
class Runtime:
    """What every part needs to run: device, activation type, kernels."""

    device: torch.device
    dtype: torch.dtype           # activations and caches: torch.bfloat16 or torch.float32
    kernels: object              # the operations (chibillm_b200.kernels.ops.CudaKernels)

    @property
    def is_float32(self) -> bool:
        return self.dtype == torch.float32


# ------------------------------------------------------------------ tensors
@dataclass(frozen=True)
class TensorSpec:
    """A tensor a part expects in the checkpoint."""

    name: str
    shape: Tuple[int, ...]
    kind: str = "float"          # "float" (kept bfloat16 / 32-bit) or "int" (kept int32)


# ------------------------------------------------------------------ cache needs
@dataclass(frozen=True)
class PagedKVNeed:
    """Keys and values of every position, in pages; ``window`` None = all keys
    stay, an integer = only that many most recent ones are ever read."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class FixedStateNeed:
    """Per-request state of fixed size: named arrays, zeroed when a request is
    admitted.  ``arrays``: ((name, shape, dtype), ...)."""

    arrays: Tuple[Tuple[str, Tuple[int, ...], torch.dtype], ...]


# ------------------------------------------------------------------ parts
class Part:
    def expected_tensors(self) -> List[TensorSpec]:
        return []

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Take the loaded tensors (already on the device) this part declared."""

    def launch_key(self, ctx):
        """Host-side decisions of ``forward`` that depend on the batch's values
        (not only on its numbers of tokens and sequences), as a hashable; a
        decode step is replayed from a CUDA graph only while this stays the same.
        None (the default) means: never capture a step that runs this part --
        right for a part that reads values on the host or allocates while it runs."""
        return None


class Norm(Part):
    """y = norm(x) over the last ``spec.size`` features."""

    def forward(self, x: torch.Tensor, out: torch.Tensor) -> None:
        raise NotImplementedError

    def forward_fused(self, residual: torch.Tensor, pending, out: torch.Tensor, scaled_ok: bool = False):
        """residual += pending (a matrix product that its producer left for us to
        add, or None); out = norm(residual).  A norm may do both in one kernel.
        Returns what the reader is to be given: ``out``, or -- only if ``scaled_ok``
        says that the reader hands it to the kernels' matrix products unchanged --
        an object of the kernels that stands for ``out`` with a factor per row
        still to be applied."""
        if pending is not None:
            pending.add_into(residual)
        self.forward(residual, out)
        return out


class PositionEncoding(Part):
    """Position information applied to queries and keys inside a mixer.

    ``fused_rotation()`` returns (inv_freq table, rotary_dim) when the encoding
    is a split-half rotation that the attention kernels apply themselves, else
    None; then ``apply`` is called on q and k before they are cached.
    """

    def fused_rotation(self):
        return None

    def step_table(self, ctx):
        """[tokens, rotary_dim] float32: the cosines, then the sines, of every token
        of the step, for kernels that rotate from a table; computed once per step
        and shared through ``ctx.shared`` by all layers with the same constants.
        None if the encoding has no such table."""
        return None

    def apply(self, q: torch.Tensor, k: Optional[torch.Tensor], ctx) -> None:
        raise NotImplementedError


class Mixer(Part):
    """Mixes information between the tokens of a sequence.

    ``forward`` reads the normalised input ``x`` [T, hidden] and adds its result
    into the 32-bit ``residual`` [T, hidden].  ``cache`` is what the cache
    manager made for this run step from ``cache_need()`` (a PagedKVView, a
    FixedStateView or None).  It returns None -- or an object with
    ``add_into(residual)`` for a last product that it has not added yet (the
    block hands it to the next norm, which may add and normalise in one kernel).
    """

    # True: ``forward`` passes ``x`` on to ``kernels.linear`` / ``linear_swiglu`` / ``linear_partial``
    # and reads it in no other way, so the block may hand it a norm output whose factor per row
    # those products apply themselves.
    accepts_scaled_rows = False

    def cache_need(self):
        return None

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, cache) -> None:
        raise NotImplementedError


class FeedForward(Part):
    """Per-token transformation; adds its result into ``residual`` (or returns it
    pending, as a mixer may)."""

    accepts_scaled_rows = False      # as for a mixer

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx) -> None:
        raise NotImplementedError


class Block(Part):
    """An arrangement of mixer, feed-forward and norms around the residual."""

    mixer: Mixer

    def forward(self, residual: torch.Tensor, ctx, cache, pending=None):
        """``pending``: what the block before left to be added to the residual.
        Returns what this block leaves pending (or None)."""
        raise NotImplementedError


class Adapter(Part):
    """A part at one of the decoder's ends (AdapterSpec).  An input adapter gets
    the 32-bit residual [T, hidden] right after the token embedding, a logit
    adapter the 32-bit logits [R, vocab] of the wanted rows; both change their
    argument in place.  ``ctx`` is the step's context (positions, sequences)."""

    def forward(self, x: torch.Tensor, ctx) -> None:
        raise NotImplementedError


# ------------------------------------------------------------------ registries
_NORMS: Dict[str, Callable] = {}
_POSITIONS: Dict[str, Callable] = {}
_MIXERS: Dict[str, Callable] = {}
_FEED_FORWARDS: Dict[str, Callable] = {}
_BLOCKS: Dict[str, Callable] = {}
_ADAPTERS: Dict[str, Callable] = {}


def _register(table: Dict[str, Callable], what: str, kind: str, factory: Callable, replace: bool):
    if kind in table and not replace:
        raise ValueError(f"{what} kind '{kind}' is already registered")
    table[kind] = factory


def _lookup(table: Dict[str, Callable], what: str, kind: str) -> Callable:
    try:
        return table[kind]
    except KeyError:
        raise KeyError(f"{what} kind '{kind}' is not registered; known: {sorted(table)}") from None


def register_norm(kind: str, factory: Callable, replace: bool = False) -> None:
    """factory(spec: NormSpec, weight_name: str, runtime) -> Norm"""
    _register(_NORMS, "norm", kind, factory, replace)


def register_position(kind: str, factory: Callable, replace: bool = False) -> None:
    """factory(spec: PositionSpec, runtime) -> PositionEncoding"""
    _register(_POSITIONS, "position encoding", kind, factory, replace)


def register_mixer(kind: str, factory: Callable, replace: bool = False) -> None:
    """factory(spec: MixerSpec, names: dict role -> tensor name, runtime) -> Mixer"""
    _register(_MIXERS, "mixer", kind, factory, replace)


def register_feed_forward(kind: str, factory: Callable, replace: bool = False) -> None:
    """factory(spec: FeedForwardSpec, names: dict role -> tensor name, runtime) -> FeedForward"""
    _register(_FEED_FORWARDS, "feed-forward", kind, factory, replace)


def register_block(kind: str, factory: Callable, replace: bool = False) -> None:
    """factory(layer: LayerSpec, runtime) -> Block"""
    _register(_BLOCKS, "block arrangement", kind, factory, replace)


def register_adapter(kind: str, factory: Callable, replace: bool = False) -> None:
    """factory(spec: AdapterSpec, runtime) -> Adapter"""
    _register(_ADAPTERS, "adapter", kind, factory, replace)


def make_adapter(spec, runtime: Runtime) -> Adapter:
    return _lookup(_ADAPTERS, "adapter", spec.kind)(spec, runtime)


def make_norm(spec, weight_name: str, runtime: Runtime) -> Norm:
    return _lookup(_NORMS, "norm", spec.kind)(spec, weight_name, runtime)


def make_position(spec, runtime: Runtime) -> PositionEncoding:
    return _lookup(_POSITIONS, "position encoding", spec.kind)(spec, runtime)


def make_mixer(spec, names: Dict[str, str], runtime: Runtime) -> Mixer:
    return _lookup(_MIXERS, "mixer", spec.kind)(spec, names, runtime)


def make_feed_forward(spec, names: Dict[str, str], runtime: Runtime) -> FeedForward:
    return _lookup(_FEED_FORWARDS, "feed-forward", spec.kind)(spec, names, runtime)


def make_block(layer, runtime: Runtime) -> Block:
    return _lookup(_BLOCKS, "block arrangement", layer.arrangement)(layer, runtime)
