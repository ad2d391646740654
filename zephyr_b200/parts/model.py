"""A model put together from parts, as its spec says: an input part (token ids to hidden states),
the layers in their run order, and an output part (hidden states of the wanted tokens to float32
logits).  For the one architecture built here these are the embedding, the decoder layers, and the
final norm with the vocabulary projection (reference forward: src/model/causal_lm/qwen3.cpp:152-181).
"""

from __future__ import annotations

import dataclasses
from typing import Mapping

import torch

from ..cache import PagedCacheSpec, StateCacheSpec
from ..config.errors import ConfigError
from ..config.spec import LayerSpec, ModelSpec
from ..kernels import ops
from ..weights.loader import WeightDecl, WeightStore, load_weights
from .base import (BLOCKS, FEED_FORWARDS, INPUTS, MIXERS, NORMS, OUTPUTS, ResidualStream, StepContext, lookup)
from .fused import DecodeChains


def _layer_classes(layer: LayerSpec):
    block = lookup(BLOCKS, "block", layer.block)
    wanted, given = set(getattr(block, "norm_names", ())), set(layer.norms)
    if wanted and wanted != given:
        raise ConfigError(f"block '{layer.block}' places the norms {sorted(wanted)}, the layer brings {sorted(given)}")
    return (block, lookup(MIXERS, "mixer", layer.mixer.kind),
            lookup(FEED_FORWARDS, "feed-forward", layer.feed_forward.kind),
            {name: lookup(NORMS, "norm", norm.kind) for name, norm in layer.norms.items()})


def expected_weights(spec: ModelSpec) -> dict[str, WeightDecl]:
    """Every tensor the model reads, by full name.  A name declared by two parts (a head tied to the
    embedding) must have one shape; it keeps the role of its first declaration."""
    decls: dict[str, WeightDecl] = {}

    def merge(new: dict[str, WeightDecl]) -> None:
        for name, decl in new.items():
            if name in decls:
                if decls[name].shape != decl.shape:
                    raise ConfigError(f"tensor '{name}' is declared twice with different shapes")
                continue
            decls[name] = decl

    merge(lookup(INPUTS, "input part", spec.input.kind).weight_decls(spec.input))
    for layer in spec.layers:
        _, mixer, ffn, norms = _layer_classes(layer)
        merge(mixer.weight_decls(layer.mixer))
        merge(ffn.weight_decls(layer.feed_forward))
        for name, norm in norms.items():
            merge(norm.weight_decls(layer.norms[name]))
    merge(lookup(OUTPUTS, "output part", spec.output.kind).weight_decls(spec.output))
    return decls


def cache_specs(spec: ModelSpec) -> list[PagedCacheSpec | StateCacheSpec | None]:
    """What each cache id needs, taken from the mixer of the call that writes it."""
    out: list = [None] * spec.num_caches
    for call in spec.run_order:
        layer = spec.layers[call.layer]
        mixer = lookup(MIXERS, "mixer", layer.mixer.kind)
        need = mixer.cache_spec(layer.mixer)
        if call.writes_cache:
            out[call.cache] = need
        elif out[call.cache] != need:
            raise ConfigError(f"layer {call.layer} reads cache {call.cache}, whose shape does not fit its mixer")
    return out


def tile_requests(spec: ModelSpec) -> list[tuple[int, str]]:
    wanted: list[tuple[int, str]] = []
    for layer in spec.layers:
        for request in lookup(MIXERS, "mixer", layer.mixer.kind).tile_requests(layer.mixer):
            if request not in wanted:
                wanted.append(request)
    return wanted


class Model:
    def __init__(self, spec: ModelSpec, weights: Mapping[str, torch.Tensor], dtype: torch.dtype,
                 device: torch.device | str):
        spec.validate()
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        self.input = lookup(INPUTS, "input part", spec.input.kind)(spec.input, weights, dtype)
        self.output = lookup(OUTPUTS, "output part", spec.output.kind)(spec.output, weights, dtype)
        self.layers = []
        for layer in spec.layers:
            block, mixer, ffn, norms = _layer_classes(layer)
            self.layers.append(block(mixer(layer.mixer, weights, dtype, device), ffn(layer.feed_forward, weights, dtype),
                                     {name: cls(layer.norms[name], weights, dtype) for name, cls in norms.items()}))
        self.cache_specs = cache_specs(spec)
        parts = [self.input, self.output]
        for block in self.layers:
            parts += [block, block.mixer, block.feed_forward, *getattr(block, "norms", {}).values(),
                      getattr(block.mixer, "position", None)]
        self.graph_safe = all(getattr(part, "graph_safe", False) for part in parts if part is not None)
        self.tile_requests = tile_requests(spec)
        # Steps of a few tokens run as fused chains of products where every block offers its pieces.
        self.chains = DecodeChains.build(self.layers, spec.run_order, spec.hidden_size, dtype)
        self.use_chains = True
        # A decode step of a small model is bound by latency: a layer's chain of small products waits on
        # barriers while the memory system idles, and its attention streams the cache while the tensor
        # cores idle.  Two halves of the batch, each on half the SMs and on a stream of its own, fill each
        # other's pauses.  It pays where the cache a layer reads outweighs the layer's weights (which are
        # then read twice) and each half still has rows enough to keep its SMs busy: measured on the
        # Qwen3-0.6B shape at context 4096, 16 requests gain 9 % (2.53 -> 2.29 ms a step), 8 lose 5 %.
        self.lanes_min_rows = 12
        self.lanes_max_layer_bytes = 64 << 20
        self._lanes_ok = (self.chains is not None and self.graph_safe
                          and all(getattr(block.mixer, "fast_decode", False) for block in self.layers))
        self._layer_bytes = None
        self._side_stream = None

    @classmethod
    def load(cls, spec: ModelSpec, store: WeightStore, dtype: torch.dtype, device: torch.device | str) -> "Model":
        weights = load_weights(store, expected_weights(spec), dtype, device, spec.ignorable_weights)
        return cls(spec, weights, dtype, device)

    def weight_bytes_read_per_step(self) -> int:
        """Bytes of weights one step reads when every matrix is used once (an embedding table is only
        gathered from, unless it also serves as the head)."""
        by_storage: dict[int, dict[tuple[int, int], int]] = {}     # storage -> {(address, bytes) of a tensor}
        sizes: dict[int, int] = {}

        def add(t: torch.Tensor) -> None:
            storage = t.untyped_storage()
            sizes[storage.data_ptr()] = storage.nbytes()
            by_storage.setdefault(storage.data_ptr(), {})[(t.data_ptr(), t.numel() * t.element_size())] = 1

        for part in (self.input, self.output):
            for tensor in part.weights_read():
                add(tensor)
        for call in self.spec.run_order:
            block = self.layers[call.layer]
            for part in (block.mixer, block.feed_forward, *getattr(block, "norms", {}).values()):
                for tensor in part.weights_read():
                    add(tensor)
        # Tensors that share a storage overlap (a matrix and a view of its first rows): such a storage
        # counts once, and never for more than it holds.
        return sum(min(sizes[storage], sum(size for _, size in tensors)) for storage, tensors in by_storage.items())

    def _lane_split(self, ctx: StepContext) -> int:
        """How many of the step's rows go to the first of two lanes; 0 if the step runs as one."""
        rows = ctx.num_rows
        if (not self._lanes_ok or rows < self.lanes_min_rows or ctx.num_decode_rows != rows or ctx.num_tokens != rows):
            return 0
        if self._layer_bytes is None:
            self._layer_bytes = (self.weight_bytes_read_per_step() - sum(
                t.numel() * t.element_size() for t in self.output.weights_read())) // max(len(self.spec.run_order), 1)
        if self._layer_bytes > self.lanes_max_layer_bytes:
            return 0
        first = (rows + 1) // 2
        return first if self.chains.supports(first) and self.chains.supports(rows - first) else 0

    @staticmethod
    def _rows_of(ctx: StepContext, r0: int, r1: int) -> StepContext:
        """The rows r0..r1 of a step in which every row brings one token, as a step of their own: a
        row's number is then also its token's place in the stream, so the first n entries of the index
        vectors that count rows or tokens serve any n rows."""
        n = r1 - r0
        return dataclasses.replace(
            ctx, num_tokens=n, num_rows=n, token_ids=ctx.token_ids[r0:r1], positions=ctx.positions[r0:r1],
            token_row=ctx.token_row[:n], row_q_start=ctx.row_q_start[:n], row_q_len=ctx.row_q_len[r0:r1],
            row_ctx=ctx.row_ctx[r0:r1], state_slots=ctx.state_slots[r0:r1],
            block_tables=[table[r0:r1] for table in ctx.block_tables], logit_tokens=ctx.logit_tokens[:0],
            decode_rows=ctx.decode_rows[:n], num_decode_rows=n, host_q_len=ctx.host_q_len[r0:r1],
            host_ctx=ctx.host_ctx[r0:r1], host_slots=ctx.host_slots[r0:r1])

    def _forward_in_two_lanes(self, hidden: torch.Tensor, ctx: StepContext, first: int):
        main = torch.cuda.current_stream(self.device)
        if self._side_stream is None:
            self._side_stream = torch.cuda.Stream(device=self.device)
        side = self._side_stream
        sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        rows = ctx.num_rows
        side.wait_stream(main)
        with ops.lane(0, sms // 2):
            head = self.chains.forward(hidden[:first], self._rows_of(ctx, 0, first))
        with torch.cuda.stream(side), ops.lane(1, sms - sms // 2):
            tail = self.chains.forward(hidden[first:], self._rows_of(ctx, first, rows))
        main.wait_stream(side)
        return torch.cat([head[0], tail[0]]), torch.cat([head[1], tail[1]])

    def forward(self, ctx: StepContext) -> torch.Tensor:
        """Run the step's tokens through the model; float32 logits [wanted, vocab]."""
        hidden = self.input.forward(ctx)
        if self.use_chains and self.chains is not None and self.chains.supports(ctx.num_tokens):
            first = self._lane_split(ctx)
            if first:
                stream = ResidualStream(*self._forward_in_two_lanes(hidden, ctx, first))
            else:
                stream = ResidualStream(*self.chains.forward(hidden, ctx))
        else:
            stream = ResidualStream(hidden)
            for call in self.spec.run_order:
                stream = self.layers[call.layer].forward(stream, ctx, call)
        return self.output.forward(stream, ctx)
