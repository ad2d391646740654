"""What every part is, the registries that name the kinds, and what a step hands to the parts.

A part is built from its spec (all sizes and constants), the loaded tensors it named in
``weight_decls`` and the engine's dtype.  It never learns which model it is in.

Registering a new kind is one call, from anywhere (a test included):

    register_mixer("my_mixer", MyMixer)

with the interface of the matching base class below.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping

import torch

from ..cache import CacheStorage, PagedCacheSpec, StateCacheSpec
from ..config.errors import ConfigError
from ..config.spec import FeedForwardSpec, InputSpec, LayerCall, MixerSpec, NormSpec, OutputSpec, PositionSpec
from ..weights.loader import WeightDecl


@dataclass
class StepContext:
    """One step's batch, as the parts see it.  Index tensors are int32 on the device.

    The new tokens of all rows (requests) lie behind one another in one stream of ``num_tokens``
    tokens; row ``r`` owns tokens ``row_q_start[r] .. row_q_start[r] + row_q_len[r]`` and had
    ``row_ctx[r]`` tokens in the cache before this step, so its first new token sits at position
    ``row_ctx[r]``."""

    num_tokens: int
    num_rows: int
    token_ids: torch.Tensor            # [T]
    positions: torch.Tensor            # [T] absolute position of each token in its request
    token_row: torch.Tensor            # [T] row of each token
    row_q_start: torch.Tensor          # [R]
    row_q_len: torch.Tensor            # [R]
    row_ctx: torch.Tensor              # [R]
    state_slots: torch.Tensor          # [R] state slot of each row's request
    block_tables: list[torch.Tensor]   # per cache group: [R, max_blocks]
    group_of_cache: Mapping[int, int]  # cache id -> group
    logit_tokens: torch.Tensor         # [n] stream indices of the tokens whose logits are wanted
    decode_rows: torch.Tensor          # [n_dec] rows with exactly one new token
    num_decode_rows: int
    max_decode_context: int            # longest context among decode rows, the new token included
    tiles: dict[tuple[int, str], tuple[torch.Tensor, torch.Tensor]]   # (tile_tokens, which) -> (tile_row, tile_q0)
    caches: CacheStorage
    status: torch.Tensor
    dtype: torch.dtype
    # Host copies for parts that plan on the host.
    host_q_len: list[int] = field(default_factory=list)
    host_ctx: list[int] = field(default_factory=list)
    host_slots: list[int] = field(default_factory=list)

    def block_table(self, cache_id: int) -> torch.Tensor:
        return self.block_tables[self.group_of_cache[cache_id]]


class Part:
    """Common ground of all parts."""

    # True if ``forward`` only launches work whose shapes depend on the step's sizes, and reads the
    # step's values (positions, tables, slots) on the device.  Steps of a model whose parts are all
    # graph-safe may be captured once and replayed.  A part that plans with host values of the
    # step (``StepContext.host_*``) must leave this False.
    graph_safe = False

    @staticmethod
    def weight_decls(spec) -> dict[str, WeightDecl]:
        """Full tensor names this part reads, with shapes and roles."""
        return {}

    def weights_read(self) -> list[torch.Tensor]:
        """The weight tensors one forward pass reads.  Some may share memory (the query rows of a fused
        q/k/v matrix); whoever adds up bytes counts a piece of memory once."""
        return [value for value in vars(self).values() if isinstance(value, torch.Tensor) and value.is_floating_point()]


class Norm(Part):
    def __init__(self, spec: NormSpec, weights: Mapping[str, torch.Tensor], dtype: torch.dtype): ...

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """Normalise the last dimension of ``x`` ([T, size])."""
        raise NotImplementedError

    def add_forward(self, residual: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
        """``residual += delta`` in place, then the norm of the sum.  The default does the two steps
        apart; a kind with a fused kernel overrides it."""
        residual.add_(delta)
        return self.forward(residual)

    def as_rms_scale(self) -> tuple[torch.Tensor, float] | None:
        """(scale vector, eps) if this norm is y = x * rsqrt(mean(x^2) + eps) * scale, so that a
        fused kernel may apply it; None for any other norm."""
        return None


class PositionEncoding(Part):
    def __init__(self, spec: PositionSpec, dtype: torch.dtype, device: torch.device | str): ...

    def apply(self, x: torch.Tensor, heads: int, positions: torch.Tensor, status: torch.Tensor) -> torch.Tensor:
        """Encode positions into ``x`` [T, heads*head_dim] in place and return it."""
        raise NotImplementedError

    def as_rotation_tables(self) -> tuple[torch.Tensor | None, torch.Tensor | None] | None:
        """What a kernel that encodes positions itself needs.  (cos, sin), float32
        [max_positions, head_dim/2] on the device, if the encoding rotates the pairs (i, i + head_dim/2)
        of every head by the angle of the token's position; (None, None) if it leaves queries and keys
        as they are; None for anything else, which is then applied through ``apply``."""
        return None

    def as_score_slopes(self) -> torch.Tensor | None:
        """None, or float32 [heads] on the device for an encoding that is a bias on the attention
        scores, linear in the distance: query head h adds slopes[h] * (key position - query position).
        The attention part then takes the general kernel, the only one with that door."""
        return None


class Mixer(Part):
    def __init__(self, spec: MixerSpec, weights: Mapping[str, torch.Tensor], dtype: torch.dtype,
                 device: torch.device | str): ...

    @staticmethod
    def cache_spec(spec: MixerSpec) -> PagedCacheSpec | StateCacheSpec | None:
        """What this mixer stores per request: pages, a fixed state, or nothing."""
        return None

    @staticmethod
    def tile_requests(spec: MixerSpec) -> list[tuple[int, str]]:
        """Tilings of the new tokens this mixer wants in ``StepContext.tiles``: (tokens per tile,
        "all" rows, only "multi"-token rows, or only "single"-token rows)."""
        return []

    def forward(self, x: torch.Tensor, ctx: StepContext, call: LayerCall) -> torch.Tensor:
        """x [T, hidden] -> [T, hidden], reading and (if ``call.writes_cache``) writing cache ``call.cache``."""
        raise NotImplementedError

    # A mixer of the form  out_weight( core( in_weight(x) ) )  may say so: a block can then run the
    # two plain products inside a fused chain of products and call ``core`` in between.
    def projections(self, call: LayerCall) -> tuple[torch.Tensor, torch.Tensor] | None:
        """(in_weight [P, hidden], out_weight [hidden, Q]) for this call, or None."""
        return None

    def core(self, projected: torch.Tensor, ctx: StepContext, call: LayerCall) -> torch.Tensor:
        """[T, P] -> [T, Q]: what lies between the two products."""
        raise NotImplementedError


class FeedForward(Part):
    def __init__(self, spec: FeedForwardSpec, weights: Mapping[str, torch.Tensor], dtype: torch.dtype): ...

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def as_gated_products(self) -> tuple[torch.Tensor, torch.Tensor] | None:
        """(gate_up weight [2I, hidden] in blocks of 8 gate rows and their 8 up rows, down weight
        [hidden, I]) if this part is down(silu(gate(x)) * up(x)); None otherwise."""
        return None


@dataclass
class ResidualStream:
    """The hidden states between blocks: the stream itself and a summand not yet added, which the
    next norm adds in the same pass that normalises."""

    hidden: torch.Tensor
    pending: torch.Tensor | None = None

    def flush(self) -> torch.Tensor:
        if self.pending is not None:
            self.hidden.add_(self.pending)
            self.pending = None
        return self.hidden


class Block(Part):
    """The arrangement of a layer's parts around the residual stream."""

    # The names of the norms this arrangement places, in ``LayerSpec.norms``.
    norm_names: tuple[str, ...] = ()

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, norms: Mapping[str, Norm]): ...

    def forward(self, stream: ResidualStream, ctx: StepContext, call: LayerCall) -> ResidualStream:
        raise NotImplementedError

    def chain_plan(self):
        """What a fused chain of small products needs of this block (``fused.BlockPlan``), or None
        if the block is not of the pre-norm residual form over parts that offer it."""
        return None


class InputPart(Part):
    """Token ids to the first hidden states."""

    def __init__(self, spec: InputSpec, weights: Mapping[str, torch.Tensor], dtype: torch.dtype): ...

    def forward(self, ctx: StepContext) -> torch.Tensor:
        """[T, hidden] in the model's type for the step's tokens (``ctx.token_ids``)."""
        raise NotImplementedError


class OutputPart(Part):
    """The last hidden states of the wanted tokens to logits."""

    def __init__(self, spec: OutputSpec, weights: Mapping[str, torch.Tensor], dtype: torch.dtype): ...

    def forward(self, stream: ResidualStream, ctx: StepContext) -> torch.Tensor:
        """float32 logits [wanted, vocab] for the tokens ``ctx.logit_tokens`` names (indices into the
        step's token stream), in that order.  ``stream`` may carry a pending summand."""
        raise NotImplementedError


NORMS: dict[str, type] = {}
INPUTS: dict[str, type] = {}
OUTPUTS: dict[str, type] = {}
POSITION_ENCODINGS: dict[str, type] = {}
MIXERS: dict[str, type] = {}
FEED_FORWARDS: dict[str, type] = {}
BLOCKS: dict[str, type] = {}


def _register(table: dict[str, type], what: str, kind: str, cls: type, replace: bool) -> None:
    if kind in table and not replace:
        raise ConfigError(f"{what} kind '{kind}' is already registered")
    table[kind] = cls


def register_norm(kind: str, cls: type, replace: bool = False) -> None:
    _register(NORMS, "norm", kind, cls, replace)


def register_position_encoding(kind: str, cls: type, replace: bool = False) -> None:
    _register(POSITION_ENCODINGS, "position encoding", kind, cls, replace)


def register_mixer(kind: str, cls: type, replace: bool = False) -> None:
    _register(MIXERS, "mixer", kind, cls, replace)


def register_feed_forward(kind: str, cls: type, replace: bool = False) -> None:
    _register(FEED_FORWARDS, "feed-forward", kind, cls, replace)


def register_block(kind: str, cls: type, replace: bool = False) -> None:
    _register(BLOCKS, "block", kind, cls, replace)


def register_input(kind: str, cls: type, replace: bool = False) -> None:
    _register(INPUTS, "input part", kind, cls, replace)


def register_output(kind: str, cls: type, replace: bool = False) -> None:
    _register(OUTPUTS, "output part", kind, cls, replace)


def lookup(table: dict[str, type], what: str, kind: str) -> type:
    if kind not in table:
        raise ConfigError(f"unknown {what} kind '{kind}'; registered: {', '.join(sorted(table)) or 'none'}")
    return table[kind]
