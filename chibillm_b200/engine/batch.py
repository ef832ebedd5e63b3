"""A step's batch: what is fed, flattened into the arrays the kernels read.

The reference flattens scheduled items into ``tokens``, ``positions`` and
per-row table offsets (src/model_batch.cc:34-125, 127-204) and runs prompt
chunks and decode tokens in separate batches.  Here one batch holds any mix:
every entry is (request, its next tokens, the places whose logits are wanted);
a decode token is an entry of one token.  Metadata is per sequence
(``q_start``, ``ctx_len``, one block-table row per group) plus per token
(``positions``, ``seq_of_token``).  The flattening itself, with its checks, is
``chibi_pack_step`` of the C++ runtime (``csrc/runtime.cc``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Sequence, Tuple

import torch


@dataclass
class StepEntry:
    """The next tokens of one request and the places (indices into ``tokens``)
    whose logits are wanted."""

    request_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


class BatchError(ValueError):
    pass


class Workspace:
    """Named scratch arrays that live across steps, so a step of a size seen
    before allocates nothing."""

    def __init__(self, device: torch.device):
        self.device = device
        self._buffers: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}
        # the views handed out, by (name, type, shape): a step asks for the same few dozen views
        # layer after layer, and building one costs as much host time as a fifth of a launch
        self._views: Dict[Tuple[str, torch.dtype, Tuple[int, ...]], torch.Tensor] = {}
        self.generation = 0        # counts allocations: a captured graph is valid for one value

    def get(self, name: str, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        shape = tuple(shape)
        view = self._views.get((name, dtype, shape))
        if view is not None:
            return view
        count = 1
        for s in shape:
            count *= int(s)
        key = (name, dtype)
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < count:
            grow = max(count, 1)
            if buf is not None:
                grow = max(grow, 2 * buf.numel()) if count < (1 << 28) else count
            buf = torch.empty(grow, dtype=dtype, device=self.device)
            self._buffers[key] = buf
            self.generation += 1
            for old in [k for k in self._views if k[0] == name and k[1] == dtype]:
                del self._views[old]           # views of the array that was replaced
        if len(self._views) > 4096:
            self._views.clear()                # many different step sizes: start over
        view = buf[:count].view(*shape)
        self._views[(name, dtype, shape)] = view
        return view

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._buffers.values())


@dataclass
class StepContext:
    """Everything a part may read about the running batch."""

    num_tokens: int
    num_seqs: int
    tokens: torch.Tensor                 # int32 [T]
    positions: torch.Tensor              # int32 [T]
    seq_of_token: torch.Tensor           # int32 [T]
    q_start: torch.Tensor                # int32 [S + 1]
    ctx_len: torch.Tensor                # int32 [S]  (tokens held after this step)
    state_slots: torch.Tensor            # int32 [S]: each sequence's state slot
    logit_rows: torch.Tensor             # int32 [R]
    tables: Dict[str, torch.Tensor]      # group -> int32 [slots, blocks]; a sequence's row is its slot
    workspace: Workspace
    # host copies, for sizing launches and for mixers that walk sequences
    request_ids: List[Hashable] = field(default_factory=list)
    q_lens: List[int] = field(default_factory=list)
    ctx_lens: List[int] = field(default_factory=list)
    slot_list: List[int] = field(default_factory=list)
    max_q_len: int = 0
    min_q_len: int = 0
    max_ctx_len: int = 0
    # what several layers of this step share: a part computes a value when it first needs it and
    # files it under a key that says what it depends on (a table of rotation angles, cache slots)
    shared: Dict[Hashable, object] = field(default_factory=dict)

    @property
    def seq_rows(self) -> torch.Tensor:
        """Row of the block tables per sequence (its state slot)."""
        return self.state_slots

    @property
    def decode_only(self) -> bool:
        return self.max_q_len == 1
