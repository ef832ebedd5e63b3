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

import math
import sys
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


def latency_summary(samples: List[float]) -> dict:
    """samples, p50 and p95 with the reference's rank rule: the value at
    ceil(fraction * n) - 1 of the sorted samples (src/generation_metrics.cc:12-23)."""
    if not samples:
        return {"samples": 0, "p50_seconds": None, "p95_seconds": None}
    ordered = sorted(samples)
    pick = lambda fraction: ordered[max(0, math.ceil(fraction * len(ordered)) - 1)]
    return {"samples": len(ordered), "p50_seconds": pick(0.50), "p95_seconds": pick(0.95)}


@dataclass
class RequestMetrics:
    """Per-request figures with the reference's definitions
    (src/generation_metrics.cc:40-90): prefill tok/s = processed prompt tokens /
    seconds of the steps that processed them; decode tok/s = (output tokens - 1) /
    (time of the last token - time of the first); decode-step latencies are the
    durations of the steps that decoded a token of this request, inter-token
    latencies the gaps between its tokens."""

    prompt_tokens: int = 0
    output_tokens: int = 0
    requested_tokens: int = 0
    processed_prompt_tokens: int = 0
    prefill_batches: int = 0
    prefill_seconds: float = 0.0
    decode_seconds: float = 0.0
    submitted_at: float = 0.0
    admitted_at: Optional[float] = None
    first_token_at: Optional[float] = None
    last_token_at: Optional[float] = None
    finish_reason: Optional[str] = None
    decode_samples: List[float] = field(default_factory=list)
    inter_token_samples: List[float] = field(default_factory=list)

    def record_batch(self, prefill: bool, prompt_count: int, seconds: float) -> None:
        if prefill:
            self.prefill_batches += 1
            self.processed_prompt_tokens += prompt_count
            self.prefill_seconds += seconds
        else:
            self.decode_seconds += seconds
            self.decode_samples.append(seconds)

    def record_token(self, at: float) -> None:
        if self.last_token_at is not None:
            self.inter_token_samples.append(at - self.last_token_at)
        else:
            self.first_token_at = at
        self.last_token_at = at
        self.output_tokens += 1

    def as_dict(self) -> dict:
        ttft = None if self.first_token_at is None else self.first_token_at - self.submitted_at
        engine_ttft = None
        if self.first_token_at is not None and self.admitted_at is not None:
            engine_ttft = self.first_token_at - self.admitted_at
        decode_tps = None
        if self.output_tokens > 1 and self.last_token_at and self.last_token_at > self.first_token_at:
            decode_tps = (self.output_tokens - 1) / (self.last_token_at - self.first_token_at)
        end_to_end = None if self.last_token_at is None else self.last_token_at - self.submitted_at
        return {
            "schema_version": 1,
            "type": "request",
            "stop_reason": self.finish_reason,
            "finish_reason": self.finish_reason,
            "prompt_tokens": self.prompt_tokens,
            "cached_prompt_tokens": 0,
            "processed_prompt_tokens": self.processed_prompt_tokens,
            "output_tokens": self.output_tokens,
            "requested_tokens": self.requested_tokens,
            "prefill_batches": self.prefill_batches,
            "prefill_seconds": self.prefill_seconds,
            "decode_engine_seconds": self.decode_seconds,
            "engine_ttft_seconds": engine_ttft,
            "time_to_first_token_seconds": ttft,
            "end_to_end_seconds": end_to_end,
            "prefill_tokens_per_second": (self.processed_prompt_tokens / self.prefill_seconds
                                          if self.prefill_seconds > 0 else None),
            "decode_tokens_per_second": decode_tps,
            "decode_step": latency_summary(self.decode_samples),
            "inter_token": latency_summary(self.inter_token_samples),
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
        self.profile_passes = False    # with a profiler on the kernels: one [cuda-pass] line per step
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
        self.metrics[seq_id] = RequestMetrics(prompt_tokens=len(prompt), requested_tokens=params.max_new_tokens,
                                              submitted_at=time.perf_counter())
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
            self.metrics[self.pending[0].id].admitted_at = time.perf_counter()
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
        profiler = getattr(self.runner.runtime.kernels, "profiler", None)
        if profiler is not None:
            profiler.begin_step()
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
        if profiler is not None:
            record = profiler.end_step(sum(item.count for item in batch.items))
            if self.profile_passes:
                print("[cuda-pass] tokens={tokens} launches={launches} encode_ms={encode_ms:.3f} "
                      "wait_ms={wait_ms:.3f} gpu_ms={gpu_ms:.3f} total_ms={total_ms:.3f}".format(**record),
                      file=sys.stderr)
        now = time.perf_counter()
        for item in batch.items:
            prefill = sched.sequences[item.seq_id].status == "waiting"
            self.metrics[item.seq_id].record_batch(prefill, item.count if prefill else 0, now - started)
        updates = sched.complete(batch.batch_id, sampled)
        for u in updates:
            m = self.metrics[u.seq_id]
            m.record_token(now)
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
