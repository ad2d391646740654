"""A model put together from parts, as its spec says: embedding, the layers in their run order,
final norm, and the vocabulary projection for the tokens whose logits are wanted
(reference forward: src/model/causal_lm/qwen3.cpp:152-181).

Differences from the reference's order of work, none of which changes the math: the final norm
runs on the wanted rows only (it is row-wise; the reference norms every token and selects after,
qwen3.cpp:173-174), and the logits come out in float32 whatever the model's type (the reference
stores them in the model's type, qwen3.cpp:175-180).
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..cache import PagedCacheSpec, StateCacheSpec
from ..config.errors import ConfigError
from ..config.spec import LayerSpec, ModelSpec
from ..kernels import ops
from ..weights.loader import ROLE_EMBEDDING, ROLE_LINEAR, WeightDecl, WeightStore, load_weights
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, ResidualStream, StepContext, lookup)
from .fused import DecodeChains


def _layer_classes(layer: LayerSpec):
    return (lookup(BLOCKS, "block", layer.block), lookup(MIXERS, "mixer", layer.mixer.kind),
            lookup(FEED_FORWARDS, "feed-forward", layer.feed_forward.kind),
            lookup(NORMS, "norm", layer.mixer_norm.kind), lookup(NORMS, "norm", layer.feed_forward_norm.kind))


def expected_weights(spec: ModelSpec) -> dict[str, WeightDecl]:
    """Every tensor the model reads, by full name."""
    decls: dict[str, WeightDecl] = {
        spec.embedding_weight: WeightDecl((spec.vocab_size, spec.hidden_size), ROLE_EMBEDDING)}
    if not spec.tied_head:
        decls[spec.lm_head_weight] = WeightDecl((spec.vocab_size, spec.hidden_size), ROLE_LINEAR)

    def merge(new: dict[str, WeightDecl]) -> None:
        for name, decl in new.items():
            if name in decls and decls[name] != decl:
                raise ConfigError(f"tensor '{name}' is declared twice with different shapes")
            decls[name] = decl

    for layer in spec.layers:
        _, mixer, ffn, norm1, norm2 = _layer_classes(layer)
        merge(mixer.weight_decls(layer.mixer))
        merge(ffn.weight_decls(layer.feed_forward))
        merge(norm1.weight_decls(layer.mixer_norm))
        merge(norm2.weight_decls(layer.feed_forward_norm))
    merge(lookup(NORMS, "norm", spec.final_norm.kind).weight_decls(spec.final_norm))
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
        self.embedding = weights[spec.embedding_weight]
        self.lm_head = self.embedding if spec.tied_head else weights[spec.lm_head_weight]
        self.layers = []
        for layer in spec.layers:
            block, mixer, ffn, norm1, norm2 = _layer_classes(layer)
            self.layers.append(block(mixer(layer.mixer, weights, dtype, device),
                                     ffn(layer.feed_forward, weights, dtype),
                                     norm1(layer.mixer_norm, weights, dtype),
                                     norm2(layer.feed_forward_norm, weights, dtype)))
        self.final_norm = lookup(NORMS, "norm", spec.final_norm.kind)(spec.final_norm, weights, dtype)
        self.cache_specs = cache_specs(spec)
        parts = [self.final_norm]
        for block in self.layers:
            parts += [block, block.mixer, block.feed_forward, block.mixer_norm, block.feed_forward_norm,
                      getattr(block.mixer, "position", None)]
        self.graph_safe = all(getattr(part, "graph_safe", False) for part in parts if part is not None)
        self.tile_requests = tile_requests(spec)
        # Steps of a few tokens run as fused chains of products where every block offers its pieces.
        self.chains = DecodeChains.build(self.layers, spec.run_order, spec.hidden_size, dtype)
        self.use_chains = True

    @classmethod
    def load(cls, spec: ModelSpec, store: WeightStore, dtype: torch.dtype, device: torch.device | str) -> "Model":
        weights = load_weights(store, expected_weights(spec), dtype, device, spec.ignorable_weights)
        return cls(spec, weights, dtype, device)

    def weight_bytes_read_per_step(self) -> int:
        """Bytes of weights one step reads when every matrix is used once (the embedding table is
        only gathered from, unless it also serves as the head)."""
        by_storage: dict[int, dict[tuple[int, int], int]] = {}     # storage -> {(address, bytes) of a tensor}
        sizes: dict[int, int] = {}

        def add(t: torch.Tensor) -> None:
            storage = t.untyped_storage()
            sizes[storage.data_ptr()] = storage.nbytes()
            by_storage.setdefault(storage.data_ptr(), {})[(t.data_ptr(), t.numel() * t.element_size())] = 1

        add(self.lm_head)
        for tensor in self.final_norm.weights_read():
            add(tensor)
        for call in self.spec.run_order:
            block = self.layers[call.layer]
            for part in (block.mixer, block.feed_forward, block.mixer_norm, block.feed_forward_norm):
                for tensor in part.weights_read():
                    add(tensor)
        # Tensors that share a storage overlap (a matrix and a view of its first rows): such a storage
        # counts once, and never for more than it holds.
        return sum(min(sizes[storage], sum(size for _, size in tensors)) for storage, tensors in by_storage.items())

    def forward(self, ctx: StepContext) -> torch.Tensor:
        """Run the step's tokens through the model; float32 logits [wanted, vocab]."""
        hidden = ops.embedding(self.embedding, ctx.token_ids, ctx.status)
        if self.use_chains and self.chains is not None and self.chains.supports(ctx.num_tokens):
            stream = ResidualStream(*self.chains.forward(hidden, ctx))
        else:
            stream = ResidualStream(hidden)
            for call in self.spec.run_order:
                stream = self.layers[call.layer].forward(stream, ctx, call)
        wanted = ctx.logit_tokens
        if wanted.numel() == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.device)
        rows = ops.gather_rows(stream.hidden, wanted, ctx.status)
        if stream.pending is not None:
            normed = self.final_norm.add_forward(rows, ops.gather_rows(stream.pending, wanted, ctx.status))
        else:
            normed = self.final_norm.forward(rows)
        return ops.linear(normed, self.lm_head, out_dtype=torch.float32)
