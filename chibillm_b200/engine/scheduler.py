"""The scheduler: admits requests, cuts prompts into portions under a token
budget, decodes, finishes and frees.

Kept from the reference (src/scheduler.cc, src/seq.cc):

* a sequence is ``waiting`` (prompt not fully processed), ``running`` (one
  token per step) or ``finished``; after the last portion of the prompt the
  sampled token is appended *unprocessed*, and every decode step processes it
  and appends the next (src/seq.cc:138-160; src/scheduler.cc:393-398);
* admission is three-way (src/scheduler.cc:162-235): ``too_large`` if the
  request alone can never fit, ``deferred`` if the live requests leave no
  sequence or page budget for it, else ``admitted``;
* the page budget is the worst case of every live request,
  1 + (prompt + max_new_tokens - 2) / page_size pages, the last sample never
  being fed back (src/scheduler.cc:13-22) -- so **pages cannot run out in the
  middle of a request**: a request that might not fit waits outside until a
  finish or a cancel frees budget; there is no preemption, swap or recompute;
* a portion is min(what is left, quantum, what the step's budget has left); the
  quantum is ``prefill_chunk_tokens`` while requests compete (more than one
  waiting, or any running) and the whole budget otherwise
  (src/scheduler.cc:259-275); a prompt that was not finished goes to the back of
  the waiting queue (src/scheduler.cc:376-383);
* stop: EOS first, then length (src/seq.cc:287-303); pages go back on finish
  and on cancel, not on abort (src/scheduler.cc:400-408,431-452,486).

Changed: the reference runs prefill batches and decode rounds in turns
(src/scheduler.cc:250-258,415-423).  Here every step takes one token of every
running sequence first and fills what is left of the budget with prompt
portions, in one mixed batch.

The queues, the counters and the decisions are C++ (``csrc/runtime.cc``); the
classes here hold a handle, keep the sampling parameters and the request ids (any
hashable), and admit to and release from the cache when the C++ side says so.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

from ..cache import native
from ..cache.manager import CacheError, CacheManager
from ..sampling.sampler import SamplingParams

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"
ADMITTED, DEFERRED, TOO_LARGE = "admitted", "deferred", "too_large"

_STATUS = (WAITING, RUNNING, FINISHED)
_REASONS = (None, "eos", "len_limit", "cancelled")
_ADMISSION = (ADMITTED, DEFERRED, TOO_LARGE)
_ERRORS = {-20: "batch_in_flight", -21: "duplicate_sequence_id", -22: "invalid_sequence_state",
           -23: "no_runnable_sequences", -24: "cache_capacity_exhausted", -25: "block_manager_failure",
           -26: "no_batch_in_flight", -27: "batch_id_mismatch", -28: "result_count_mismatch",
           -29: "unknown_sequence", -30: "sequence_not_finished", -31: "invalid_configuration"}


class SchedulerError(RuntimeError):
    def __init__(self, code: str, message: str = ""):
        super().__init__(f"{code}: {message}" if message else code)
        self.code = code


def _raise(status: int) -> None:
    message = native.error_message()
    if native.ERROR_CODES.get(status) == "invariant":
        raise AssertionError(message)
    raise SchedulerError(_ERRORS.get(status, native.ERROR_CODES.get(status, f"status {status}")), message)


@dataclass
class SchedulerConfig:
    """Defaults of the reference's serving mode (src/scheduler.h:30-39)."""

    max_sequences: int = 4
    max_batch_tokens: int = 128
    prefill_chunk_tokens: int = 64

    def validate(self) -> None:
        for name in ("max_sequences", "max_batch_tokens", "prefill_chunk_tokens"):
            if getattr(self, name) <= 0:
                raise SchedulerError("invalid_configuration", f"{name} must be positive")


class Sequence:
    """Token list with the counters processed <= processed + scheduled <= tokens
    (src/seq.cc:305-323).  Until a scheduler takes it, and again once it has been
    removed from one, the object holds its own values; in between they are read
    from the scheduler."""

    def __init__(self, seq_id: Hashable, prompt: Sequence[int], params: SamplingParams):
        if len(prompt) == 0:
            raise SchedulerError("seq.empty_prompt")
        if params.max_new_tokens <= 0:
            raise SchedulerError("seq.invalid_max_new_tokens")
        self.id = seq_id
        self.prompt_len = len(prompt)
        self.params = params
        self._owner: Optional["Scheduler"] = None
        self._number = -1
        self._tokens: List[int] = [int(t) for t in prompt]
        self._state = (0, 0, WAITING, None)         # processed, scheduled, status, finish reason

    # ---- values that the scheduler owns while it has the sequence
    def _info(self):
        return self._owner._info(self._number) if self._owner is not None else None

    @property
    def tokens(self) -> List[int]:
        if self._owner is None:
            return self._tokens
        return self._owner._tokens(self._number, 0, self._info()[4])

    def slice(self, first: int, count: int) -> List[int]:
        """tokens[first : first + count] without fetching the rest."""
        if self._owner is None:
            return self._tokens[first:first + count]
        return self._owner._tokens(self._number, first, count)

    @property
    def processed(self) -> int:
        info = self._info()
        return info[0] if info else self._state[0]

    @property
    def scheduled(self) -> int:
        info = self._info()
        return info[1] if info else self._state[1]

    @property
    def status(self) -> str:
        info = self._info()
        return _STATUS[info[2]] if info else self._state[2]

    @property
    def finish_reason(self) -> Optional[str]:
        info = self._info()
        return _REASONS[info[3]] if info else self._state[3]

    @property
    def length(self) -> int:
        info = self._info()
        return info[4] if info else len(self._tokens)

    @property
    def completion_len(self) -> int:
        return self.length - self.prompt_len

    @property
    def completion(self) -> List[int]:
        return self.slice(self.prompt_len, self.completion_len)

    @property
    def schedulable(self) -> int:
        return self.length - self.processed - self.scheduled

    @property
    def is_finished(self) -> bool:
        return self.status == FINISHED

    def _detach(self) -> None:
        """Take the values over from the scheduler that is about to forget the sequence."""
        info = self._info()
        self._tokens = self._owner._tokens(self._number, 0, info[4])
        self._state = (info[0], info[1], _STATUS[info[2]], _REASONS[info[3]])
        self._owner = None


@dataclass
class ScheduledItem:
    seq_id: Hashable
    first: int           # index of the portion's first token in the sequence
    count: int
    sample: bool         # the portion reaches the end of the known tokens


@dataclass
class ScheduledBatch:
    batch_id: int
    items: List[ScheduledItem] = field(default_factory=list)

    @property
    def token_count(self) -> int:
        return sum(i.count for i in self.items)

    @property
    def sample_count(self) -> int:
        return sum(1 for i in self.items if i.sample)


@dataclass
class SequenceUpdate:
    seq_id: Hashable
    token: int
    finish_reason: Optional[str]


class Scheduler:
    def __init__(self, config: SchedulerConfig, cache: CacheManager, eos_token: Optional[int],
                 on_admit=None, on_release=None):
        config.validate()
        self.config = config
        self.cache = cache
        self.eos_token = eos_token
        self.sequences: Dict[Hashable, Sequence] = {}
        self.active: Optional[ScheduledBatch] = None
        self._on_admit = on_admit or cache.admit
        self._on_release = on_release or cache.release
        self._lib = native.runtime()
        self._handle = self._lib.chibi_sched_new(cache.handle, config.max_sequences, config.max_batch_tokens,
                                                 config.prefill_chunk_tokens,
                                                 -1 if eos_token is None else int(eos_token))
        if not self._handle:
            raise SchedulerError("invalid_configuration", native.error_message())
        self._ids: Dict[int, Hashable] = {}        # the C++ side's number -> request id
        self._info_buf = (ctypes.c_int * 6)()
        self._items_buf = (ctypes.c_longlong * (4 * config.max_sequences))()
        self._updates_buf = (ctypes.c_longlong * (3 * config.max_sequences))()

    def __del__(self):
        if getattr(self, "_handle", None):
            self._lib.chibi_sched_delete(self._handle)
            self._handle = None

    # ---- what sequences read
    def _info(self, number: int):
        status = self._lib.chibi_sched_info(self._handle, number, self._info_buf)
        if status < 0:
            _raise(status)
        return tuple(self._info_buf)

    def _tokens(self, number: int, first: int, count: int) -> List[int]:
        out = (ctypes.c_int * max(count, 1))()
        status = self._lib.chibi_sched_tokens(self._handle, number, first, count, out)
        if status < 0:
            _raise(status)
        return list(out[:count])

    def _queue(self, which: int) -> List[Hashable]:
        n = self._lib.chibi_sched_queue(self._handle, which, None, 0)
        out = (ctypes.c_longlong * max(n, 1))()
        self._lib.chibi_sched_queue(self._handle, which, out, n)
        return [self._ids[out[i]] for i in range(n)]

    @property
    def waiting(self) -> List[Hashable]:
        return self._queue(0)

    @property
    def running(self) -> List[Hashable]:
        return self._queue(1)

    # ---- budget
    def fits_cache(self, seq: Sequence) -> bool:
        return bool(self._lib.chibi_sched_fits_cache(self._handle, seq.prompt_len, seq.params.max_new_tokens))

    # ---- admission
    def try_add(self, seq: Sequence) -> str:
        if seq.id in self.sequences:
            if self.active is not None:
                raise SchedulerError("batch_in_flight")
            raise SchedulerError("duplicate_sequence_id", repr(seq.id))
        if seq._owner is not None or seq.status != WAITING or seq.processed or seq.scheduled \
                or seq.length != seq.prompt_len:
            raise SchedulerError("invalid_sequence_state", repr(seq.id))
        decision = self._lib.chibi_sched_admission(self._handle, seq.prompt_len, seq.params.max_new_tokens)
        if decision < 0:
            _raise(decision)
        if decision != 0:
            return _ADMISSION[decision]
        try:
            self._on_admit(seq.id)
            self.cache.reserve(seq.id, 1)
        except CacheError as e:
            self._on_release(seq.id)
            raise SchedulerError("block_manager_failure", str(e)) from None
        number = self.cache.number_of(seq.id)
        prompt = (ctypes.c_int * seq.prompt_len)(*seq._tokens)
        status = self._lib.chibi_sched_add(self._handle, number, prompt, seq.prompt_len,
                                           seq.params.max_new_tokens, 1 if seq.params.ignore_eos else 0)
        if status < 0:
            self._on_release(seq.id)
            _raise(status)
        seq._owner, seq._number = self, number
        self._ids[number] = seq.id
        self.sequences[seq.id] = seq
        return ADMITTED

    def add(self, seq: Sequence) -> None:
        result = self.try_add(seq)
        if result == TOO_LARGE:
            raise SchedulerError("sequence_too_large", repr(seq.id))
        if result == DEFERRED:
            raise SchedulerError("capacity_deferred", repr(seq.id))

    # ---- one step
    def has_work(self) -> bool:
        return bool(self._lib.chibi_sched_has_work(self._handle))

    def schedule(self) -> ScheduledBatch:
        batch_id = ctypes.c_int()
        n = self._lib.chibi_sched_schedule(self._handle, self._items_buf, self.config.max_sequences,
                                           ctypes.byref(batch_id))
        if n < 0:
            _raise(n)
        b = self._items_buf
        batch = ScheduledBatch(batch_id.value, [
            ScheduledItem(self._ids[b[4 * i]], b[4 * i + 1], b[4 * i + 2], bool(b[4 * i + 3])) for i in range(n)])
        self.active = batch
        return batch

    def complete(self, batch_id: int, sampled: Sequence[int]) -> List[SequenceUpdate]:
        values = (ctypes.c_int * max(len(sampled), 1))(*[int(t) for t in sampled])
        n = self._lib.chibi_sched_complete(self._handle, int(batch_id), values, len(sampled), self._updates_buf,
                                           self.config.max_sequences)
        if n < 0:
            _raise(n)
        updates: List[SequenceUpdate] = []
        for i in range(n):
            seq_id = self._ids[self._updates_buf[3 * i]]
            reason = _REASONS[self._updates_buf[3 * i + 2]]
            if reason is not None:
                self._on_release(seq_id)
            updates.append(SequenceUpdate(seq_id, int(self._updates_buf[3 * i + 1]), reason))
        self.active = None
        return updates

    def abort(self, batch_id: int) -> None:
        """Undo the token reservations of the batch in flight; pages stay, so a
        retry schedules the same batch (src/scheduler.cc:431-452)."""
        status = self._lib.chibi_sched_abort(self._handle, int(batch_id))
        if status < 0:
            _raise(status)
        self.active = None

    def cancel(self, seq_id: Hashable) -> None:
        seq = self.sequences.get(seq_id)
        if seq is None:
            if self.active is not None:
                raise SchedulerError("batch_in_flight")
            raise SchedulerError("unknown_sequence", repr(seq_id))
        status = self._lib.chibi_sched_cancel(self._handle, seq._number)
        if status < 0:
            _raise(status)
        if status == 1:
            self._on_release(seq_id)

    def remove(self, seq_id: Hashable) -> Sequence:
        seq = self.sequences.get(seq_id)
        if seq is None:
            raise SchedulerError("unknown_sequence", repr(seq_id))
        if not seq.is_finished:
            raise SchedulerError("sequence_not_finished", repr(seq_id))
        seq_number = seq._number
        seq._detach()
        status = self._lib.chibi_sched_remove(self._handle, seq_number)
        if status < 0:
            _raise(status)
        self._ids.pop(seq_number, None)
        return self.sequences.pop(seq_id)

    def check_invariants(self) -> None:
        status = self._lib.chibi_sched_check(self._handle)
        if status < 0:
            _raise(status)
