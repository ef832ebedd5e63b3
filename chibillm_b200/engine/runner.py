"""The step function: runs a batch of (request, its next tokens) from the cache
and returns the logits at the wanted places.

The reference's counterpart is ``qwen_model_runner::execute``
(src/qwen/qwen_model_runner.cc:198-239): metadata, embedding, layers, output on
the sampled rows, one wait.  Differences: a batch may mix portions of prompts
with single decoded tokens, any place of an entry may be wanted, and the
logits themselves are returned (the reference returns only the arg max).

A step runs only the tokens it is given.  Everything earlier comes from the
pages that former steps wrote.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Hashable, List, Optional, Sequence

import torch

from ..cache import native
from ..cache.manager import CacheError, CacheManager
from ..cache.storage import CacheStorage, FixedStateView, plan_cache
from ..config.registry import load_config
from ..parts.base import Runtime
from ..weights.loader import load_weights
from .batch import BatchError, StepContext, StepEntry, Workspace
from .model import DecoderModel

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
           "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype {name} is not supported (bfloat16 or float32)")
        return name
    try:
        return _DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"dtype '{name}' is not supported (bfloat16 or float32)") from None


def make_runtime(dtype, device="cuda:0", kernels=None, spec=None) -> Runtime:
    """The product's runtime: a CUDA device and this package's kernels.  A test
    may pass a stand-in for the kernels (then any device is allowed).  With the
    model's ``spec`` the libraries it will load are built together first."""
    device = torch.device(device)
    if kernels is None:
        from ..kernels.ops import CudaKernels
        if spec is not None:
            from ..csrc import build
            head_dims = {getattr(layer.mixer, "head_dim", 0) for layer in spec.layers}
            build.prepare(head_dims, bfloat16=parse_dtype(dtype) == torch.bfloat16)
        kernels = CudaKernels(device)
    return Runtime(device=device, dtype=parse_dtype(dtype), kernels=kernels)


def _align4(n: int) -> int:
    return (n + 3) & ~3


class ModelRunner:
    def __init__(self, model: DecoderModel, runtime: Runtime, page_size: int, pool_tokens: int,
                 max_requests: int):
        self.model = model
        self.spec = model.spec
        self.runtime = runtime
        self.page_size = page_size
        plan = plan_cache(model.cache_needs(), model.cache_sources(), page_size, pool_tokens,
                          model.spec.max_positions)
        self.plan = plan
        self.cache = CacheManager(plan.groups, max_requests)
        self.storage = CacheStorage(plan, runtime, max_requests)
        self.workspace = Workspace(runtime.device)
        self._meta_host: Optional[torch.Tensor] = None
        self._meta_dev: Optional[torch.Tensor] = None
        self._meta_copied = None      # event: the last copy out of the pinned array is done
        self.last_meta_bytes = 0      # bytes the last step sent to the device
        self.steps_run = 0
        self._meta_epoch = 0
        self.use_graphs = runtime.device.type == "cuda"
        self._graphs: Dict[tuple, tuple] = {}
        self._graphs_warm = set()
        self._graphs_epoch = None
        self.graph_replays = 0
        # a decode step launched ahead of the tokens that decide whether it is wanted
        self._ahead: Optional[dict] = None
        self.steps_ahead_used = 0
        self.steps_ahead_dropped = 0
        self._has_state = any(isinstance(v, FixedStateView) for v in self.storage.views)
        # the last step, if it was run with ``provisional=True`` and is neither settled nor rolled
        # back yet: (request ids, lengths before, saved rows of the fixed-size state)
        self._provisional: Optional[tuple] = None

    # ------------------------------------------------------------ construction
    @classmethod
    def from_folder(cls, model_dir: str, dtype="bfloat16", device="cuda:0", page_size: int = 16,
                    pool_tokens: int = 4096, max_requests: int = 4, kernels=None) -> "ModelRunner":
        _, _, spec = load_config(model_dir)
        runtime = make_runtime(dtype, device, kernels, spec)
        model = DecoderModel(spec, runtime)
        load_weights(model, model_dir, runtime)
        return cls(model, runtime, page_size, pool_tokens, max_requests)

    @classmethod
    def from_random(cls, config_object: dict, seed: int = 0, dtype="bfloat16", device="cuda:0",
                    page_size: int = 16, pool_tokens: int = 4096, max_requests: int = 4,
                    kernels=None, num_layers: Optional[int] = None) -> "ModelRunner":
        """A model of the architecture and sizes that ``config_object`` (the
        content of a config.json) names, with random weights made on the device.
        ``num_layers`` runs only the first layers (for measurements that must fit
        a time or memory limit; every layer keeps its full size)."""
        from ..config.registry import find_architecture
        from ..weights.random_init import bind_random_weights
        if num_layers is not None:
            config_object = dict(config_object, num_hidden_layers=num_layers)
        arch = find_architecture(config_object)
        spec = arch.model_spec(arch.read_config(config_object))
        runtime = make_runtime(dtype, device, kernels, spec)
        model = DecoderModel(spec, runtime)
        bind_random_weights(model, seed, runtime)
        return cls(model, runtime, page_size, pool_tokens, max_requests)

    @property
    def max_context_tokens(self) -> int:
        """min(model's positions, what the smallest pool holds)
        (src/qwen/qwen_model_runner.cc:128-134)."""
        pool = min((g.num_pages * g.page_size for g in self.plan.groups), default=self.spec.max_positions)
        return min(self.spec.max_positions, pool)

    # ------------------------------------------------------------ requests
    def admit(self, request_id: Hashable) -> None:
        rc = self.cache.admit(request_id)
        self.storage.zero_state_slot(rc.state_slot)

    def end(self, request_id: Hashable) -> None:
        if self._ahead is not None and request_id in self._ahead["ids"]:
            self._ahead = None              # its logits belong to a request that no longer exists
            self.steps_ahead_dropped += 1
        self.cache.release(request_id)

    def has(self, request_id: Hashable) -> bool:
        return self.cache.has(request_id)

    def length(self, request_id: Hashable) -> int:
        return self.cache.length(request_id)

    # ------------------------------------------------------------ metadata
    META_CAPACITY = 1 << 20      # int32 values; allocated once so that its address never changes

    def _meta_buffers(self, count: int):
        if self._meta_host is None or self._meta_host.numel() < count:
            cap = max(self.META_CAPACITY, 2 * count)
            pin = self.runtime.device.type == "cuda"
            self._meta_host = torch.empty(cap, dtype=torch.int32, pin_memory=pin)
            self._meta_dev = torch.empty(cap, dtype=torch.int32, device=self.runtime.device)
            self._meta_epoch += 1
        return self._meta_host, self._meta_dev

    def _build_context(self, entries: Sequence[StepEntry], fixed_update_capacity: bool):
        """Make room for the entries' tokens, flatten them, send the packed
        metadata to the device and hand back what brings the device's block tables
        up to date.  The checks, the reservations and the packing are one call into
        the C++ runtime, which writes straight into the pinned array.  With
        ``fixed_update_capacity`` the layout of the packed array depends only on the
        numbers of tokens, sequences and wanted rows (what a captured graph needs);
        the third value returned says whether the table updates of this step fitted
        that layout."""
        cache = self.cache
        S = len(entries)
        groups = cache.group_order()
        G = len(groups)
        q_lens = [len(e.tokens) for e in entries]
        want_lens = [len(e.want) for e in entries]
        T, R = sum(q_lens), sum(want_lens)
        ids = (ctypes.c_longlong * S)(*[cache.number_of(e.request_id) for e in entries])
        n_tokens = (ctypes.c_int * S)(*q_lens)
        n_want = (ctypes.c_int * S)(*want_lens)
        try:
            tokens = (ctypes.c_int * max(T, 1))(*[int(t) for e in entries for t in e.tokens])
            want = (ctypes.c_int * max(R, 1))(*[int(w) for e in entries for w in e.want])
        except (OverflowError, TypeError) as exc:
            raise BatchError(f"token ids and wanted places must be integers that fit 32 bits: {exc}") from None
        info = (ctypes.c_int * (13 + 2 * G))()
        words = 3 * _align4(max(T, 1)) + _align4(S + 1) + 2 * _align4(S) + _align4(max(R, 1)) \
            + G * _align4(1 + 6 * S) + 64
        while True:
            host, dev = self._meta_buffers(words)
            if self._meta_copied is not None:
                self._meta_copied.synchronize()     # the pinned array may still be read by the last copy
            status = native.runtime().chibi_pack_step(
                cache.handle, S, ids, n_tokens, tokens, n_want, want, self.spec.vocab_size,
                self.spec.max_positions, 1 if fixed_update_capacity else 0, host.data_ptr(), host.numel(),
                info, len(info))
            if status == 0:
                break
            code = native.ERROR_CODES.get(status)
            if code == "buffer_too_small" and words < (1 << 28):
                words *= 4                          # many table updates at once: a larger array
                continue
            message = native.error_message()
            if code in ("batch", "unknown_request"):
                raise BatchError(message)
            raise CacheError(code or f"status {status}", message)
        cursor, max_ctx, fixed = info[3], info[4], bool(info[5])
        offsets = dict(zip(("tokens", "positions", "seq_of_token", "q_start", "ctx_len", "state_slots",
                            "logit_rows"), info[6:13]))
        dev[:cursor].copy_(host[:cursor], non_blocking=True)
        if dev.is_cuda:
            if self._meta_copied is None:
                self._meta_copied = torch.cuda.Event()
            self._meta_copied.record()
        self.last_meta_bytes = cursor * 4

        def view(name, n):
            o = offsets[name]
            return dev[o:o + n]

        ctx_lens = host[offsets["ctx_len"]:offsets["ctx_len"] + S].tolist()
        slots = host[offsets["state_slots"]:offsets["state_slots"] + S].tolist()
        ctx = StepContext(
            num_tokens=T, num_seqs=S, tokens=view("tokens", T), positions=view("positions", T),
            seq_of_token=view("seq_of_token", T), q_start=view("q_start", S + 1),
            ctx_len=view("ctx_len", S), state_slots=view("state_slots", S),
            logit_rows=view("logit_rows", R), tables=self.storage.tables, workspace=self.workspace,
            request_ids=[e.request_id for e in entries], q_lens=q_lens, ctx_lens=ctx_lens,
            slot_list=slots, max_q_len=max(q_lens), min_q_len=min(q_lens), max_ctx_len=max_ctx)
        update_views = {}
        for g, name in enumerate(groups):
            o, cap = info[13 + g], info[13 + G + g]
            update_views[name] = (dev[o:o + 1 + 3 * cap], cap)
        return ctx, update_views, fixed

    def _run_model(self, ctx: StepContext, update_views) -> Optional[torch.Tensor]:
        k = self.runtime.kernels
        for name, (view, cap) in update_views.items():
            if cap > 0:
                k.apply_table_updates(self.storage.tables[name], view, cap)
        return self.model.forward(ctx, self.storage.views)

    # ------------------------------------------------------------ graphs
    def _graph_epoch(self):
        k = self.runtime.kernels
        return (self.workspace.generation, getattr(k, "scratch_generation", 0), self._meta_epoch)

    def _graph_key(self, ctx: StepContext):
        """What a captured decode step depends on besides the data in the packed
        array, or None if this step cannot be replayed from a graph."""
        if not self.use_graphs or ctx.max_q_len != 1 or not getattr(self.runtime.kernels, "supports_graphs", False):
            return None
        launch = self.model.launch_key(ctx)
        if launch is None:
            return None
        return (ctx.num_seqs, ctx.logit_rows.numel(), launch)

    def _step_with_graph(self, key, ctx, update_views) -> Optional[torch.Tensor]:
        epoch = self._graph_epoch()
        if epoch != self._graphs_epoch:
            self._graphs.clear()
            self._graphs_warm.clear()
            self._graphs_epoch = epoch
        entry = self._graphs.get(key)
        k = self.runtime.kernels
        if entry is None:
            if key not in self._graphs_warm:
                # first time: run as usual, so that every array and library exists
                self._graphs_warm.add(key)
                logits = self._run_model(ctx, update_views)
                if self._graph_epoch() != epoch:        # something was allocated: start over later
                    self._graphs_warm.discard(key)
                return logits
            graph = torch.cuda.CUDAGraph()
            before = k.launches
            torch.cuda.synchronize()
            with torch.cuda.graph(graph):
                logits = self._run_model(ctx, update_views)
            entry = (graph, logits, k.launches - before)
            k.launches = before
            self._graphs[key] = entry
        graph, logits, launches = entry
        graph.replay()
        k.launches += launches
        self.graph_replays += 1
        return logits

    # ------------------------------------------------------------ running ahead
    def run_ahead(self, request_ids: Sequence[Hashable], device_tokens: torch.Tensor) -> bool:
        """Launch now the decode step that follows if every one of these requests
        goes on with the token just chosen for it (``device_tokens[i]``, still on the
        device), so that the device does not wait while the host reads the tokens
        and decides.  The next ``step`` returns its logits if it asks for exactly
        this (same requests in this order, one token each, the tokens given to
        ``confirm_ahead``, logits of each); any other ``step`` drops it.  Only a
        step that is replayed from a captured graph runs ahead, and only a model
        whose requests hold nothing but paged keys and values (a fixed-size state
        would be advanced by a step that may not be wanted).  Returns whether the
        step was launched."""
        if self._ahead is not None or not self.use_graphs or self._has_state:
            return False
        S = len(request_ids)
        if S == 0 or S > self.cache.max_requests or device_tokens.numel() != S \
                or device_tokens.dtype != torch.int32 or not device_tokens.is_cuda:
            return False
        for rid in request_ids:
            if not self.cache.has(rid) or self.cache.length(rid) + 1 > self.spec.max_positions:
                return False
        try:
            for rid in request_ids:
                self.cache.reserve(rid, self.cache.length(rid) + 1)
        except Exception:
            return False                      # no page left: the ordinary step will say so
        entries = [StepEntry(rid, [0], [0]) for rid in request_ids]      # the tokens come from the device
        ctx, update_views, fixed = self._build_context(entries, True)
        key = self._graph_key(ctx) if fixed else None
        entry = self._graphs.get(key) if key is not None and self._graph_epoch() == self._graphs_epoch else None
        if entry is None:
            # the table updates of this step have been taken from the manager: apply them now
            k = self.runtime.kernels
            for name, (view, cap) in update_views.items():
                if cap > 0:
                    k.apply_table_updates(self.storage.tables[name], view, cap)
            return False
        ctx.tokens.copy_(device_tokens)
        graph, logits, launches = entry
        graph.replay()
        self.runtime.kernels.launches += launches
        self.graph_replays += 1
        self._ahead = {"ids": tuple(request_ids), "logits": logits, "ctx_lens": list(ctx.ctx_lens), "tokens": None}
        return True

    def confirm_ahead(self, tokens: Sequence[int]) -> None:
        """The tokens that the step launched by ``run_ahead`` used, now that the host has them."""
        if self._ahead is not None:
            self._ahead["tokens"] = [int(t) for t in tokens]

    def _matches_ahead(self, ahead: dict, entries: Sequence[StepEntry]) -> bool:
        if ahead["tokens"] is None or len(entries) != len(ahead["ids"]):
            return False
        for e, rid, tok, new_len in zip(entries, ahead["ids"], ahead["tokens"], ahead["ctx_lens"]):
            if e.request_id != rid or len(e.tokens) != 1 or int(e.tokens[0]) != tok or list(e.want) != [0]:
                return False
            if not self.cache.has(rid) or self.cache.length(rid) + 1 != new_len:
                return False
        return True

    # ------------------------------------------------------------ taking a step back
    def _begin_provisional(self, entries: Sequence[StepEntry], old_lengths: Sequence[int]) -> None:
        saved = []
        if self._has_state:
            slots = torch.tensor([self.cache.state_slot(e.request_id) for e in entries], dtype=torch.long,
                                 device=self.runtime.device)
            for view in self.storage.views:
                if isinstance(view, FixedStateView):
                    for t in view.arrays.values():
                        saved.append((t, slots, t.index_select(0, slots)))
        self._provisional = ([e.request_id for e in entries], list(old_lengths), saved)

    def settle_step(self) -> None:
        """The last provisional step stands: windows give their pages back, the
        saved state is dropped."""
        if self._provisional is None:
            return
        ids, _, _ = self._provisional
        self._provisional = None
        self.cache.settle_many([r for r in ids if self.cache.has(r)])

    def rollback_step(self) -> None:
        """The last provisional step did not happen: its requests hold what they
        held before it (lengths and fixed-size state; pages stay reserved, and what
        the step wrote past the old lengths is written again by the retry), so the
        same entries can be run again with the same result
        (src/qwen/qwen3_5_model_state.cc:284-370 is the reference's counterpart for
        its recurrent state).  A step launched ahead of it is dropped."""
        if self._ahead is not None:
            self._ahead = None
            self.steps_ahead_dropped += 1
        if self._provisional is None:
            return
        ids, old_lengths, saved = self._provisional
        self._provisional = None
        for array, slots, rows in saved:
            array.index_copy_(0, slots, rows)
        keep = [(r, n) for r, n in zip(ids, old_lengths) if self.cache.has(r)]
        self.cache.rollback_many([r for r, _ in keep], [n for _, n in keep])

    # ------------------------------------------------------------ the step
    def step(self, entries: Sequence[StepEntry], check: bool = True,
             provisional: bool = False) -> Optional[torch.Tensor]:
        """Run one batch.  Returns float32 logits [wanted, vocab] on the device in
        the order of the entries and of their ``want`` (None if nothing is
        wanted).  The array is reused by the next step.

        A step in which every request brings one token is captured into a CUDA
        graph the second time its shape is seen and replayed from then on; what
        changes between replays (tokens, positions, lengths, table updates,
        wanted rows) travels in the packed metadata array.

        With ``provisional`` the caller decides afterwards whether the step
        counts: ``settle_step()`` or ``rollback_step()`` must follow before the
        next provisional step (the generation loop reads the device's error word
        and the sampled tokens in between)."""
        if not entries:
            raise BatchError("a step needs at least one entry")
        if self._provisional is not None:
            raise BatchError("the last step is neither settled nor rolled back")
        ahead, self._ahead = self._ahead, None
        if ahead is not None:
            if self._matches_ahead(ahead, entries):
                ids = [e.request_id for e in entries]
                if provisional:
                    self._begin_provisional(entries, [n - 1 for n in ahead["ctx_lens"]])
                self.cache.commit_many(ids, ahead["ctx_lens"], hold=provisional)
                self.steps_run += 1
                self.steps_ahead_used += 1
                if check and hasattr(self.runtime.kernels, "check_error_word"):
                    self.runtime.kernels.check_error_word()
                return ahead["logits"]
            # Not wanted after all.  Nothing is undone: the step wrote keys and values one place
            # past what its requests hold (a place that the step which does reach it writes
            # again), and the pages it reserved stay reserved to their requests.
            self.steps_ahead_dropped += 1
        if len(entries) > self.cache.max_requests:
            raise BatchError(f"{len(entries)} entries in one step; at most {self.cache.max_requests} "
                             f"requests are live at a time")
        for e in entries:
            if not self.cache.has(e.request_id):
                self.admit(e.request_id)
        decode_only = all(len(e.tokens) == 1 for e in entries)
        ctx, update_views, fixed = self._build_context(entries, decode_only and self.use_graphs)
        if provisional:
            self._begin_provisional(entries, [n - q for n, q in zip(ctx.ctx_lens, ctx.q_lens)])
        key = self._graph_key(ctx) if fixed else None
        try:
            if key is not None:
                logits = self._step_with_graph(key, ctx, update_views)
            else:
                logits = self._run_model(ctx, update_views)
        except Exception:
            if provisional:
                self.rollback_step()        # lengths are unchanged; the fixed-size state goes back
            raise
        self.cache.commit_many([e.request_id for e in entries], ctx.ctx_lens, hold=provisional)
        self.steps_run += 1
        if check and hasattr(self.runtime.kernels, "check_error_word"):
            self.runtime.kernels.check_error_word()
        return logits
