"""Architecture-neutral description of a decoder: parts, layers and run order.

A configuration class (one per architecture) turns the keys of its own
``config.json`` into a :class:`ModelSpec`.  Everything below the configuration
(weights loader, parts, cache manager, step function) reads only the spec, so
no part knows which model it is in.

Every size and constant is a field of a spec; nothing here has a default that
stands for a model's value.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    """A normalisation over the last ``size`` features.

    ``kind`` names a registered norm part ("rmsnorm").  ``weight_offset`` is
    added to the stored weight before use (0 for plain RMSNorm, 1 for the
    zero-centred variant).
    """

    kind: str
    size: int
    eps: float
    weight_offset: float = 0.0


@dataclass(frozen=True)
class PositionSpec:
    """Position encoding applied inside a mixer.

    ``kind`` "rope": split-half rotation of the first ``rotary_dim`` features
    of every head with ``inv_freq[j] = theta ** (-2j / rotary_dim)``.
    ``kind`` "none": nothing is applied.
    """

    kind: str
    head_dim: int = 0
    rotary_dim: int = 0
    theta: float = 0.0


@dataclass(frozen=True)
class MixerSpec:
    """Base of all token mixers; ``kind`` names a registered mixer part."""

    kind: str


@dataclass(frozen=True)
class AttentionSpec(MixerSpec):
    """Causal grouped-query attention over a paged key/value cache.

    ``window`` None means every earlier key is visible; an integer W means the
    W most recent keys, the query's own included.  ``scale`` multiplies the
    scores after the dot product.
    """

    hidden_size: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    scale: float = 0.0
    window: Optional[int] = None
    qk_norm: Optional[NormSpec] = None
    position: PositionSpec = PositionSpec(kind="none")


@dataclass(frozen=True)
class FeedForwardSpec:
    """Base of all feed-forward parts; ``kind`` names a registered part."""

    kind: str


@dataclass(frozen=True)
class GatedMLPSpec(FeedForwardSpec):
    """Dense gated feed-forward: down(act(gate(x)) * up(x))."""

    hidden_size: int = 0
    intermediate_size: int = 0
    activation: str = "silu"


@dataclass(frozen=True)
class LayerSpec:
    """One block: how mixer, feed-forward and norms are arranged.

    ``arrangement`` names a registered block ("prenorm": x + mixer(norm(x)),
    then x + ff(norm(x))).  ``weight_prefix`` is the checkpoint prefix of the
    block's tensors.  ``weight_names`` maps the part-local tensor roles to
    checkpoint names under that prefix.
    """

    arrangement: str
    mixer: MixerSpec
    feed_forward: FeedForwardSpec
    mixer_norm: NormSpec
    feed_forward_norm: NormSpec
    weight_prefix: str
    weight_names: Tuple[Tuple[str, str], ...] = ()

    def names(self) -> dict:
        return dict(self.weight_names)


@dataclass(frozen=True)
class RunStep:
    """One entry of the run order.

    ``layer`` indexes ``ModelSpec.layers`` (a layer may be named twice: its
    weights are shared, every run has a cache of its own).  ``cache_of`` names
    an earlier run step whose cache this step reads instead of writing one.
    """

    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class AdapterSpec:
    """A part at one of the decoder's ends: after the token embedding (it
    changes the residual stream in place: a learned or absolute position table,
    a scale of the embeddings) or on the logits of the wanted rows (a soft cap,
    a bias).  ``kind`` names a registered adapter part; ``weight_names`` maps
    its tensor roles to checkpoint names; ``params`` are its constants."""

    kind: str
    weight_names: Tuple[Tuple[str, str], ...] = ()
    params: Tuple[Tuple[str, float], ...] = ()

    def names(self) -> dict:
        return dict(self.weight_names)

    def constants(self) -> dict:
        return dict(self.params)


@dataclass(frozen=True)
class ModelSpec:
    """A whole decoder: embedding, what follows it at once, layers, run order,
    final norm, output, what is done to the logits."""

    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    layers: Tuple[LayerSpec, ...]
    run_order: Tuple[RunStep, ...]
    final_norm: NormSpec
    embedding_name: str
    final_norm_name: str
    output_name: str
    tie_output_to_embedding: bool
    eos_token_id: Optional[int] = None
    bos_token_id: Optional[int] = None
    extra: dict = field(default_factory=dict, compare=False)
    input_adapters: Tuple[AdapterSpec, ...] = ()      # run on the residual right after the embedding
    logit_adapters: Tuple[AdapterSpec, ...] = ()      # run on the 32-bit logits of the wanted rows
