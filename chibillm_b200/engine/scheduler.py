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
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Sequence

from ..cache.manager import CacheError, CacheManager, pages_for
from ..sampling.sampler import SamplingParams

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"
ADMITTED, DEFERRED, TOO_LARGE = "admitted", "deferred", "too_large"


class SchedulerError(RuntimeError):
    def __init__(self, code: str, message: str = ""):
        super().__init__(f"{code}: {message}" if message else code)
        self.code = code


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
    (src/seq.cc:305-323)."""

    def __init__(self, seq_id: Hashable, prompt: Sequence[int], params: SamplingParams):
        if len(prompt) == 0:
            raise SchedulerError("seq.empty_prompt")
        if params.max_new_tokens <= 0:
            raise SchedulerError("seq.invalid_max_new_tokens")
        self.id = seq_id
        self.tokens: List[int] = [int(t) for t in prompt]
        self.prompt_len = len(self.tokens)
        self.params = params
        self.processed = 0
        self.scheduled = 0
        self.status = WAITING
        self.finish_reason: Optional[str] = None

    @property
    def completion_len(self) -> int:
        return len(self.tokens) - self.prompt_len

    @property
    def completion(self) -> List[int]:
        return self.tokens[self.prompt_len:]

    @property
    def schedulable(self) -> int:
        return len(self.tokens) - self.processed - self.scheduled

    @property
    def is_finished(self) -> bool:
        return self.status == FINISHED

    def evaluate_stop(self, eos: Optional[int]) -> Optional[str]:
        if self.completion_len == 0:
            return None
        if not self.params.ignore_eos and eos is not None and self.tokens[-1] == eos:
            return "eos"
        if self.completion_len >= self.params.max_new_tokens:
            return "len_limit"
        return None


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
        self.waiting: Deque[Hashable] = deque()
        self.running: Deque[Hashable] = deque()
        self.active: Optional[ScheduledBatch] = None
        self._next_batch = 0
        self._on_admit = on_admit or cache.admit
        self._on_release = on_release or cache.release

    # ---- budget
    def _budget_tokens(self, seq: Sequence) -> int:
        return seq.prompt_len + seq.params.max_new_tokens - 1

    def _budget_pages(self, seq: Sequence) -> Dict[str, int]:
        return {name: self.cache.worst_case_pages(name, self._budget_tokens(seq)) for name in self.cache.groups}

    def fits_cache(self, seq: Sequence) -> bool:
        need = self._budget_pages(seq)
        return all(need[name] <= g.num_pages for name, g in self.cache.groups.items())

    # ---- admission
    def try_add(self, seq: Sequence) -> str:
        if self.active is not None:
            raise SchedulerError("batch_in_flight")
        if seq.id in self.sequences:
            raise SchedulerError("duplicate_sequence_id", repr(seq.id))
        if seq.status != WAITING or seq.processed or seq.scheduled or len(seq.tokens) != seq.prompt_len:
            raise SchedulerError("invalid_sequence_state", repr(seq.id))
        if not self.fits_cache(seq):
            return TOO_LARGE
        if len(self.waiting) + len(self.running) >= self.config.max_sequences:
            return DEFERRED
        need = self._budget_pages(seq)
        for name, g in self.cache.groups.items():
            available = g.num_pages
            for sid in list(self.waiting) + list(self.running):
                available -= self._budget_pages(self.sequences[sid])[name]
            if need[name] > available:
                return DEFERRED
        try:
            self._on_admit(seq.id)
            self.cache.reserve(seq.id, 1)
        except CacheError as e:
            self._on_release(seq.id)
            raise SchedulerError("block_manager_failure", str(e)) from None
        self.sequences[seq.id] = seq
        self.waiting.append(seq.id)
        return ADMITTED

    def add(self, seq: Sequence) -> None:
        result = self.try_add(seq)
        if result == TOO_LARGE:
            raise SchedulerError("sequence_too_large", repr(seq.id))
        if result == DEFERRED:
            raise SchedulerError("capacity_deferred", repr(seq.id))

    # ---- one step
    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def schedule(self) -> ScheduledBatch:
        if self.active is not None:
            raise SchedulerError("batch_in_flight")
        if not self.has_work():
            raise SchedulerError("no_runnable_sequences")
        cfg = self.config
        batch = ScheduledBatch(self._next_batch)
        used = 0
        try:
            for sid in self.running:
                if len(batch.items) >= cfg.max_sequences or used >= cfg.max_batch_tokens:
                    break
                seq = self.sequences[sid]
                if seq.schedulable != 1:
                    raise SchedulerError("invalid_sequence_state", f"running sequence {sid!r} has "
                                         f"{seq.schedulable} tokens to run")
                self._reserve(seq, 1)
                batch.items.append(ScheduledItem(sid, seq.processed, 1, True))
                seq.scheduled = 1
                used += 1
            contended = len(self.waiting) > 1 or bool(self.running)
            quantum = cfg.prefill_chunk_tokens if contended else cfg.max_batch_tokens
            for sid in self.waiting:
                if len(batch.items) >= cfg.max_sequences or used >= cfg.max_batch_tokens:
                    break
                seq = self.sequences[sid]
                available = seq.schedulable
                if available <= 0:
                    raise SchedulerError("invalid_sequence_state", f"waiting sequence {sid!r} has nothing to run")
                count = min(available, quantum, cfg.max_batch_tokens - used)
                self._reserve(seq, count)
                batch.items.append(ScheduledItem(sid, seq.processed, count, count == available))
                seq.scheduled = count
                used += count
        except SchedulerError:
            self._rollback(batch)
            raise
        if not batch.items:
            raise SchedulerError("no_runnable_sequences")
        self.active = batch
        self._next_batch += 1
        return batch

    def _reserve(self, seq: Sequence, count: int) -> None:
        try:
            self.cache.reserve(seq.id, seq.processed + count)
        except CacheError as e:
            if e.code == "capacity_exhausted":
                raise SchedulerError("cache_capacity_exhausted", str(e)) from None
            raise SchedulerError("block_manager_failure", str(e)) from None

    def _rollback(self, batch: ScheduledBatch) -> None:
        for item in batch.items:
            self.sequences[item.seq_id].scheduled = 0

    def complete(self, batch_id: int, sampled: Sequence[int]) -> List[SequenceUpdate]:
        if self.active is None:
            raise SchedulerError("no_batch_in_flight")
        batch = self.active
        if batch_id != batch.batch_id:
            raise SchedulerError("batch_id_mismatch")
        if len(sampled) != batch.sample_count:
            raise SchedulerError("result_count_mismatch",
                                 f"{len(sampled)} samples for {batch.sample_count} sampling items")
        updates: List[SequenceUpdate] = []
        k = 0
        for item in batch.items:
            seq = self.sequences[item.seq_id]
            seq.processed += seq.scheduled
            seq.scheduled = 0
            was_waiting = seq.status == WAITING
            (self.waiting if was_waiting else self.running).remove(item.seq_id)
            if not item.sample:
                self.waiting.append(item.seq_id)
                continue
            if was_waiting:
                seq.status = RUNNING
            seq.tokens.append(int(sampled[k]))
            k += 1
            reason = seq.evaluate_stop(self.eos_token)
            if reason is not None:
                seq.status = FINISHED
                seq.finish_reason = reason
                self._on_release(item.seq_id)
            else:
                self.running.append(item.seq_id)
            updates.append(SequenceUpdate(item.seq_id, seq.tokens[-1], reason))
        self.active = None
        return updates

    def abort(self, batch_id: int) -> None:
        """Undo the token reservations of the batch in flight; pages stay, so a
        retry schedules the same batch (src/scheduler.cc:431-452)."""
        if self.active is None:
            raise SchedulerError("no_batch_in_flight")
        if batch_id != self.active.batch_id:
            raise SchedulerError("batch_id_mismatch")
        self._rollback(self.active)
        self.active = None

    def cancel(self, seq_id: Hashable) -> None:
        if self.active is not None:
            raise SchedulerError("batch_in_flight")
        seq = self.sequences.get(seq_id)
        if seq is None:
            raise SchedulerError("unknown_sequence", repr(seq_id))
        if seq.is_finished:
            return
        for q in (self.waiting, self.running):
            if seq_id in q:
                q.remove(seq_id)
        seq.status = FINISHED
        seq.finish_reason = "cancelled"
        seq.scheduled = 0
        self._on_release(seq_id)

    def remove(self, seq_id: Hashable) -> Sequence:
        seq = self.sequences.get(seq_id)
        if seq is None:
            raise SchedulerError("unknown_sequence", repr(seq_id))
        if not seq.is_finished:
            raise SchedulerError("sequence_not_finished", repr(seq_id))
        return self.sequences.pop(seq_id)

    def check_invariants(self) -> None:
        live = list(self.waiting) + list(self.running)
        assert len(live) == len(set(live)), "a sequence is queued twice"
        for sid, seq in self.sequences.items():
            assert 0 <= seq.processed <= seq.processed + seq.scheduled <= len(seq.tokens)
            if seq.status == WAITING:
                assert sid in self.waiting
            elif seq.status == RUNNING:
                assert sid in self.running and seq.schedulable + seq.scheduled == 1
            else:
                assert sid not in live
