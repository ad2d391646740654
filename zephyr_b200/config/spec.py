"""Architecture-neutral description of a model: what the parts are built from.

An architecture's typed configuration (for instance ``Qwen3Config``) turns
itself into a ``ModelSpec``.  Everything below the configuration layer
(parts, cache manager, step function, trace replay, bench) reads only the
spec, so a new architecture adds a configuration class and, where it needs
them, new parts; nothing else changes.

Every size and constant of a part travels in its spec.  A part never asks
which model it belongs to.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping


@dataclass(frozen=True)
class NormSpec:
    """A normalisation over the last dimension."""

    kind: str          # key in parts.NORMS, e.g. "rmsnorm"
    size: int
    eps: float
    weight: str        # full tensor name of the scale


@dataclass(frozen=True)
class PositionSpec:
    """A position encoding applied to queries and keys inside a mixer."""

    kind: str          # key in parts.POSITION_ENCODINGS, e.g. "rope_neox" or "none"
    head_dim: int
    max_positions: int
    params: Mapping[str, Any] = field(default_factory=dict)   # e.g. {"theta": 1e6}


@dataclass(frozen=True)
class MixerSpec:
    """The token mixer of a layer (attention here).

    ``params`` holds everything the mixer kind needs (head counts, head size,
    window, the names of its tensors).  ``position`` is the encoding it applies.
    """

    kind: str          # key in parts.MIXERS, e.g. "attention"
    params: Mapping[str, Any]
    position: PositionSpec | None = None


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str          # key in parts.FEED_FORWARDS, e.g. "swiglu"
    params: Mapping[str, Any]


@dataclass(frozen=True)
class LayerSpec:
    """One layer: which block arrangement, and the parts placed in it.

    ``norms`` holds the layer's norms under the names the block arrangement gives them: the pre-norm
    residual block wants "mixer" and "feed_forward"; an arrangement with norms after its parts as
    well would name four."""

    block: str         # key in parts.BLOCKS, e.g. "prenorm_residual"
    mixer: MixerSpec
    feed_forward: FeedForwardSpec
    norms: Mapping[str, NormSpec]


@dataclass(frozen=True)
class InputSpec:
    """What turns a step's token ids into the first hidden states (a table lookup here)."""

    kind: str          # key in parts.INPUTS, e.g. "embedding"
    params: Mapping[str, Any]


@dataclass(frozen=True)
class OutputSpec:
    """What turns the last hidden states of the wanted tokens into float32 logits."""

    kind: str          # key in parts.OUTPUTS, e.g. "norm_head"
    params: Mapping[str, Any]


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.

    ``layer`` indexes ``ModelSpec.layers`` (a layer may be named twice: its
    weights run again).  ``cache`` names the cache this call's mixer uses;
    calls with equal ``cache`` share it.  Only a call with ``writes_cache``
    stores new entries; a call without it reads what an earlier call of the
    same step stored (a layer that reads another layer's cache).
    """

    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_seq_len: int
    input: InputSpec
    layers: tuple[LayerSpec, ...]
    run_order: tuple[LayerCall, ...]
    output: OutputSpec
    eos_token_ids: tuple[int, ...] = ()
    ignorable_weights: tuple[str, ...] = ()   # names a checkpoint may carry that are not read

    @property
    def num_caches(self) -> int:
        return 1 + max(call.cache for call in self.run_order)

    def validate(self) -> None:
        from .errors import ConfigError

        if not self.layers or not self.run_order:
            raise ConfigError("a model needs at least one layer and one run-order entry")
        writers: dict[int, int] = {}
        for index, call in enumerate(self.run_order):
            if not 0 <= call.layer < len(self.layers):
                raise ConfigError(f"run_order[{index}] names layer {call.layer}, which does not exist")
            if call.cache < 0:
                raise ConfigError(f"run_order[{index}] has a negative cache id")
            if call.writes_cache:
                if call.cache in writers:
                    raise ConfigError(
                        f"cache {call.cache} is written by run_order[{writers[call.cache]}] and run_order[{index}]")
                writers[call.cache] = index
            elif call.cache not in writers:
                raise ConfigError(f"run_order[{index}] reads cache {call.cache} before any call has written it")
        if sorted(writers) != list(range(self.num_caches)):
            raise ConfigError("cache ids must be 0..n-1, each written by exactly one call")
