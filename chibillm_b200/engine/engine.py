"""The generation loop: schedule, build the batch, run the step, sample,
complete (src/inference_engine.cc:73-118), with the reference's rule that a
failure after scheduling aborts the batch and leaves the sequences untouched,
so the same batch can be retried (src/inference_engine.cc:140-151).  A step
is run provisionally: the cache's lengths and the fixed-size state of its
requests are taken back if anything fails before the tokens are accepted.

Requests that the scheduler defers wait in a first-in first-out queue; a later
request never passes a deferred one (src/serving_runtime.cc:243-247).
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Sequence as Seq

import torch

from ..sampling.sampler import Sampler, SamplingParams
from .batch import StepEntry
from .runner import ModelRunner
from .scheduler import (ADMITTED, DEFERRED, TOO_LARGE, Scheduler, SchedulerConfig, SchedulerError,
                        Sequence, SequenceUpdate)


@dataclass
class RequestMetrics:
    """Per-request figures with the reference's definitions
    (src/generation_metrics.cc:71-90): prefill tok/s = processed prompt tokens /
    seconds of the steps that processed them; decode tok/s = (output tokens - 1) /
    (time of the last token - time of the first)."""

    prompt_tokens: int = 0
    output_tokens: int = 0
    prefill_seconds: float = 0.0
    submitted_at: float = 0.0
    first_token_at: Optional[float] = None
    last_token_at: Optional[float] = None
    finish_reason: Optional[str] = None

    def as_dict(self) -> dict:
        ttft = None if self.first_token_at is None else self.first_token_at - self.submitted_at
        decode_tps = None
        if self.output_tokens > 1 and self.last_token_at and self.last_token_at > self.first_token_at:
            decode_tps = (self.output_tokens - 1) / (self.last_token_at - self.first_token_at)
        return {
            "schema_version": 1,
            "prompt_tokens": self.prompt_tokens,
            "output_tokens": self.output_tokens,
            "prefill_seconds": self.prefill_seconds,
            "prefill_tokens_per_second": (self.prompt_tokens / self.prefill_seconds
                                          if self.prefill_seconds > 0 else None),
            "time_to_first_token_seconds": ttft,
            "decode_tokens_per_second": decode_tps,
            "finish_reason": self.finish_reason,
        }


class InferenceEngine:
    def __init__(self, runner: ModelRunner, config: Optional[SchedulerConfig] = None):
        self.runner = runner
        self.config = config or SchedulerConfig(max_sequences=runner.cache.max_requests)
        if self.config.max_sequences > runner.cache.max_requests:
            raise SchedulerError("invalid_configuration",
                                 f"max_sequences {self.config.max_sequences} exceeds the cache's "
                                 f"{runner.cache.max_requests} request slots")
        self.scheduler = Scheduler(self.config, runner.cache, runner.spec.eos_token_id,
                                   on_admit=runner.admit, on_release=runner.end)
        self.sampler = Sampler(runner.runtime)
        self.run_ahead = True          # launch the next decode step before this one's tokens are on the host
        self.pending: Deque[Sequence] = deque()
        self.metrics: Dict[Hashable, RequestMetrics] = {}
        self._keys: Dict[Hashable, int] = {}
        self._next_key = 0

    # ---- requests
    def add(self, seq_id: Hashable, prompt: Seq[int], params: Optional[SamplingParams] = None,
            sample_key: Optional[int] = None) -> str:
        """Queue a request.  Returns "admitted" or "deferred" (it waits in line);
        raises if it can never fit.  ``sample_key`` names the request to the
        sampler: with the same seed, key and temperature a request samples the
        same tokens whatever else runs (default: a running number)."""
        params = params or SamplingParams()
        limit = self.runner.max_context_tokens
        if len(prompt) + 1 > limit:
            raise SchedulerError("sequence_too_large",
                                 f"a prompt of {len(prompt)} tokens leaves no room in a context of {limit}")
        seq = Sequence(seq_id, prompt, params)
        if seq_id in self.scheduler.sequences or any(p.id == seq_id for p in self.pending):
            raise SchedulerError("duplicate_sequence_id", repr(seq_id))
        if not self.scheduler.fits_cache(seq):
            raise SchedulerError("sequence_too_large", f"request {seq_id!r} can never fit the cache")
        self.metrics[seq_id] = RequestMetrics(prompt_tokens=len(prompt), submitted_at=time.perf_counter())
        self._keys[seq_id] = self._next_key if sample_key is None else int(sample_key)
        self._next_key += 1
        self.pending.append(seq)
        self._admit_pending()
        return ADMITTED if seq_id in self.scheduler.sequences else DEFERRED

    def _admit_pending(self) -> None:
        while self.pending:
            result = self.scheduler.try_add(self.pending[0])
            if result != ADMITTED:
                break
            self.pending.popleft()

    def is_finished(self) -> bool:
        return not self.pending and not self.scheduler.has_work()

    def find_sequence(self, seq_id: Hashable) -> Optional[Sequence]:
        return self.scheduler.sequences.get(seq_id)

    def cancel(self, seq_id: Hashable) -> None:
        for p in list(self.pending):
            if p.id == seq_id:
                self.pending.remove(p)
                return
        self.scheduler.cancel(seq_id)
        self._admit_pending()

    def remove(self, seq_id: Hashable) -> Sequence:
        return self.scheduler.remove(seq_id)

    # ---- the loop
    def step(self) -> List[SequenceUpdate]:
        sched = self.scheduler
        batch = sched.schedule()
        started = time.perf_counter()
        try:
            entries = []
            for item in batch.items:
                seq = sched.sequences[item.seq_id]
                if item.first != self.runner.length(item.seq_id):
                    raise SchedulerError("inconsistent_batch",
                                         f"request {item.seq_id!r}: the scheduler continues at token {item.first}, "
                                         f"the cache holds {self.runner.length(item.seq_id)}")
                toks = seq.slice(item.first, item.count)
                entries.append(StepEntry(item.seq_id, toks, [item.count - 1] if item.sample else []))
            kernels = self.runner.runtime.kernels
            deferred_check = hasattr(kernels, "error_word_async")
            # provisional: the cache's lengths advance now (a step launched ahead builds on them),
            # but they are taken back if the error word or the tokens say that the step failed
            logits = self.runner.step(entries, check=not deferred_check, provisional=True)
            if deferred_check:
                kernels.error_word_async()        # read together with the tokens, below
            sampled: List[int] = []
            if batch.sample_count:
                rows = [sched.sequences[i.seq_id] for i in batch.items if i.sample]
                pending = self.sampler.launch(
                    logits, [s.params for s in rows], [self._keys[s.id] for s in rows],
                    [s.completion_len for s in rows])
                # While the tokens travel to the host, the device already runs the step that
                # follows if all of these requests go on (the usual case in steady decoding).
                ahead = self.run_ahead and self._next_step_is_the_same(batch, rows) \
                    and self.runner.run_ahead([s.id for s in rows], pending.device_ids)
                sampled = pending.result()
                if ahead:
                    self.runner.confirm_ahead(sampled)
            elif deferred_check and self.runner.runtime.device.type == "cuda":
                torch.cuda.current_stream().synchronize()
            if deferred_check:
                kernels.check_error_copy()
            if len(sampled) != batch.sample_count:
                raise SchedulerError("result_count_mismatch")
            self.runner.settle_step()
        except Exception:
            # the step did not happen: lengths and state go back, a step launched ahead is
            # dropped, the scheduler's reservations are cancelled; pages stay, so a retry
            # runs the same tokens at the same places (src/inference_engine.cc:140-151)
            self.runner.rollback_step()
            sched.abort(batch.batch_id)
            raise
        now = time.perf_counter()
        for item in batch.items:
            if sched.sequences[item.seq_id].status == "waiting":
                self.metrics[item.seq_id].prefill_seconds += now - started
        updates = sched.complete(batch.batch_id, sampled)
        for u in updates:
            m = self.metrics[u.seq_id]
            m.output_tokens += 1
            m.first_token_at = m.first_token_at or now
            m.last_token_at = now
            m.finish_reason = u.finish_reason
        self._admit_pending()
        return updates

    def _next_step_is_the_same(self, batch, rows) -> bool:
        """Whether the next step can be foretold: every item of this one is a single
        decoded token, nobody waits to be admitted or to be prefilled, and no request
        reaches its token limit with the token being chosen (an end-of-sequence
        token cannot be foretold: then the step that ran ahead is dropped)."""
        if self.pending or self.scheduler.waiting or len(rows) != len(batch.items):
            return False
        for item, seq in zip(batch.items, rows):
            if item.count != 1 or seq.completion_len + 1 >= seq.params.max_new_tokens:
                return False
        return True

    def generate(self, prompts: Seq[Seq[int]], params=None) -> List[List[int]]:
        """Run the prompts to completion; returns the generated ids of each."""
        if params is None or isinstance(params, SamplingParams):
            params = [params or SamplingParams()] * len(prompts)
        ids = []
        for i, (prompt, p) in enumerate(zip(prompts, params)):
            sid = ("generate", self._next_key, i)
            ids.append(sid)
            self.add(sid, prompt, p, sample_key=i)
        while not self.is_finished():
            self.step()
        out = []
        for sid in ids:
            out.append(self.scheduler.remove(sid).completion)
        return out
