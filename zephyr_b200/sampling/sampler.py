"""Choosing the next token from float32 logits.

``SamplingParams`` carries the reference's names (src/include/sampler/sampler.hpp:20-34).  Built:
greedy (temperature < 1e-7: argmax, lowest index among equals, the generator is not advanced) and
temperature sampling over the whole vocabulary (p = softmax((x - max) / T), inclusive prefix sums
in index order, the first index whose sum exceeds u * total; one draw
u = (next 64 random bits >> 40) * 2^-24 per sampled token from the request's own MT19937-64;
src/sampler/sampler.cpp:316-333, src/sampler/sampler.cu:82-83,150-167).  The reference's other
filters (top-k, top-p, min-p, penalties, logit bias, logprobs) are refused with a clear error.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Mapping, Sequence

import torch

from ..config.errors import InvalidArgumentError
from ..kernels import ops
from .mt19937_64 import MT19937_64

GREEDY_TEMPERATURE = 1e-7


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    repetition_penalty: float = 1.0
    logits_bias: Mapping[int, float] = field(default_factory=dict)
    top_logprobs: int | None = None

    @property
    def greedy(self) -> bool:
        return self.temperature < GREEDY_TEMPERATURE

    def validate(self, vocab_size: int) -> None:
        """The checks of ValidateSamplingParams (src/sampler/sampler.cpp:278-294), then this engine's
        own: filters it does not implement are refused rather than ignored."""
        numbers = (self.temperature, self.top_p, self.min_p, self.frequency_penalty, self.presence_penalty,
                   self.repetition_penalty)
        if any(not math.isfinite(v) for v in numbers) or self.temperature < 0.0 or self.repetition_penalty <= 0.0:
            raise InvalidArgumentError(
                "sampling parameters must be finite, with nonnegative temperature and positive repetition penalty")
        for token, bias in self.logits_bias.items():
            if not 0 <= token < vocab_size or math.isnan(bias) or bias == math.inf:
                raise InvalidArgumentError("logits bias requires a valid token and a finite or negative-infinite bias")
        unsupported = []
        if self.top_k > 0:
            unsupported.append("top_k")
        if 0.0 < self.top_p < 1.0:
            unsupported.append("top_p")
        if 0.0 < self.min_p < 1.0:
            unsupported.append("min_p")
        if self.frequency_penalty != 0.0 or self.presence_penalty != 0.0 or self.repetition_penalty != 1.0:
            unsupported.append("penalties")
        if self.logits_bias:
            unsupported.append("logits_bias")
        if self.top_logprobs is not None:
            unsupported.append("top_logprobs")
        if unsupported:
            raise InvalidArgumentError(
                "this engine samples greedily or by temperature over the whole vocabulary; not supported: "
                + ", ".join(unsupported))


class Sampler:
    """Selects tokens on the device; only the chosen ids come back to the host."""

    def __init__(self, device: torch.device | str):
        self.device = torch.device(device)
        self.status = ops.new_status(self.device)

    def sample_async(self, logits: torch.Tensor, params: Sequence[SamplingParams],
                     generators: Sequence[MT19937_64 | None]) -> torch.Tensor:
        """Launch the selection; returns int32 ids on the device.  Draws are taken in row order, one per
        non-greedy row."""
        rows = logits.shape[0]
        if rows != len(params) or rows != len(generators):
            raise InvalidArgumentError("one SamplingParams and one generator per row of logits")
        if all(p.greedy for p in params):
            return ops.sample(logits, None, None, self.status)
        temperature = [0.0 if p.greedy else float(p.temperature) for p in params]
        uniform = []
        for p, g in zip(params, generators):
            if p.greedy:
                uniform.append(0.0)
            else:
                if g is None:
                    raise InvalidArgumentError("a sampled row needs a generator")
                uniform.append(g.next_uniform())
        host = torch.tensor([temperature, uniform], dtype=torch.float32).pin_memory()
        device = host.to(self.device, non_blocking=True)
        return ops.sample(logits, device[0], device[1], self.status)

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams],
               generators: Sequence[MT19937_64 | None]) -> list[int]:
        ids = self.sample_async(logits, params, generators).tolist()
        ops.check_status(self.status, "sampling")
        return ids
