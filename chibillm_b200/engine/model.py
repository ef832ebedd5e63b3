"""A decoder put together from a ModelSpec: embedding (and the adapters that
follow it at once), blocks in run order, final norm, vocabulary projection on
the wanted rows (and the adapters of the logits).

The class is the same for every architecture; what differs is the spec that
the architecture's configuration produced.  The vocabulary projection uses the
output matrix if the checkpoint holds one, else the embedding table (chosen by
the file's contents: src/qwen/qwen_weights.h:36-40, src/qwen/qwen_weights.cc:
157-160,192-200).
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Sequence

import torch

from ..config.spec import ModelSpec
from ..parts.base import Block, Runtime, TensorSpec, make_adapter, make_block, make_norm
from .batch import StepContext


class DecoderModel:
    def __init__(self, spec: ModelSpec, runtime: Runtime):
        self.spec = spec
        self.runtime = runtime
        self.blocks: List[Block] = [make_block(layer, runtime) for layer in spec.layers]
        self.final_norm = make_norm(spec.final_norm, spec.final_norm_name, runtime)
        self.input_adapters = [make_adapter(a, runtime) for a in spec.input_adapters]
        self.logit_adapters = [make_adapter(a, runtime) for a in spec.logit_adapters]
        self.embedding: torch.Tensor = None
        self.output: torch.Tensor = None
        for i, step in enumerate(spec.run_order):
            if not (0 <= step.layer < len(self.blocks)):
                raise ValueError(f"run step {i} names layer {step.layer}; the model has {len(self.blocks)}")

    # ---- weights
    def expected_tensors(self, available: Optional[Iterable[str]] = None) -> List[TensorSpec]:
        """All tensors of the model.  ``available``: names in the checkpoint; the
        output matrix is expected if it is there or if the embeddings are not tied."""
        s = self.spec
        out = [TensorSpec(s.embedding_name, (s.vocab_size, s.hidden_size))]
        out += self.final_norm.expected_tensors()
        has_output = available is not None and s.output_name in set(available)
        if has_output or not s.tie_output_to_embedding:
            out.append(TensorSpec(s.output_name, (s.vocab_size, s.hidden_size)))
        for b in self.blocks:
            out += b.expected_tensors()
        for a in self.input_adapters + self.logit_adapters:
            out += a.expected_tensors()
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        self.embedding = tensors[s.embedding_name].contiguous()
        self.output = tensors[s.output_name].contiguous() if s.output_name in tensors else self.embedding
        self.final_norm.bind(tensors)
        for b in self.blocks:
            b.bind(tensors)
        for a in self.input_adapters + self.logit_adapters:
            a.bind(tensors)

    # ---- cache
    def cache_needs(self) -> List[object]:
        return [self.blocks[step.layer].mixer.cache_need() for step in self.spec.run_order]

    def cache_sources(self) -> List[Optional[int]]:
        return [step.cache_of for step in self.spec.run_order]

    def launch_key(self, ctx: StepContext):
        """What the parts decide on the host from this batch's values (beyond its
        numbers of tokens, sequences and wanted rows), as a hashable; None if any
        part cannot promise that a captured step stays valid."""
        keys = []
        for a in self.input_adapters + self.logit_adapters:
            key = a.launch_key(ctx)
            if key is None:
                return None
            keys.append(key)
        for step in self.spec.run_order:
            block = self.blocks[step.layer]
            key = block.launch_key(ctx)
            if key is None:
                return None
            keys.append(key)
        return tuple(keys)

    # ---- run
    def forward(self, ctx: StepContext, cache_views: Sequence[object]) -> Optional[torch.Tensor]:
        """Run the tokens of ``ctx``; returns 32-bit logits [R, vocab] of the
        wanted rows (None when nothing is wanted)."""
        rt = self.runtime
        k = rt.kernels
        T = ctx.num_tokens
        hidden = self.spec.hidden_size
        residual = ctx.workspace.get("model.residual", (T, hidden), torch.float32)
        k.embed(ctx.tokens, self.embedding, residual)
        for a in self.input_adapters:
            a.forward(residual, ctx)
        pending = None      # a last product that a block left to be added to the residual
        for i, step in enumerate(self.spec.run_order):
            pending = self.blocks[step.layer].forward(residual, ctx, cache_views[i], pending)
        if pending is not None:
            pending.add_into(residual)
        R = ctx.logit_rows.numel()
        if R == 0:
            return None
        rows = ctx.workspace.get("model.rows", (R, hidden), torch.float32)
        k.gather_rows(residual, ctx.logit_rows, rows)
        normed = ctx.workspace.get("model.rows_normed", (R, hidden), rt.dtype)
        self.final_norm.forward(rows, normed)
        logits = ctx.workspace.get("model.logits", (R, self.spec.vocab_size), torch.float32)
        k.linear(normed, self.output, logits)
        for a in self.logit_adapters:
            a.forward(logits, ctx)
        return logits
