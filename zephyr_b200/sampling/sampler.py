"""Choosing the next token from float32 logits.

``SamplingParams`` carries the reference's names and meanings (src/include/sampler/sampler.hpp:20-34,
python/zephyr/_C.pyi:405-442).  Built, all on the device (kernels/ops.sample_rows, csrc/sampling.cu):
  * penalties and biases from the request's history (src/sampler/sampler.cpp:112-139,
    src/sampler/sampler.cu:28-56);
  * greedy (temperature < 1e-7: argmax, lowest index among equals, the generator is not advanced);
  * temperature sampling, p = softmax((x - max) / T), with top-k, top-p and min-p
    (src/sampler/sampler.cu:99-118): rows with top-k or top-p draw over the tokens ranked by
    probability, the others over the vocabulary in index order; one draw
    u = (next 64 random bits >> 40) * 2^-24 per sampled token from the request's own MT19937-64
    (src/sampler/sampler.cpp:316-333);
  * ``top_logprobs``: the chosen token's log-probability and the n most probable tokens, measured
    after penalties and temperature and before the filters (src/sampler/sampler.cu:178-194).
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
    top_k: int = -1
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
        """The checks of ValidateSamplingParams (src/sampler/sampler.cpp:278-294)."""
        numbers = (self.temperature, self.top_p, self.min_p, self.frequency_penalty, self.presence_penalty,
                   self.repetition_penalty)
        if any(not math.isfinite(v) for v in numbers) or self.temperature < 0.0 or self.repetition_penalty <= 0.0:
            raise InvalidArgumentError(
                "sampling parameters must be finite, with nonnegative temperature and positive repetition penalty")
        for token, bias in self.logits_bias.items():
            if not 0 <= token < vocab_size or math.isnan(bias) or bias == math.inf:
                raise InvalidArgumentError("logits bias requires a valid token and a finite or negative-infinite bias")
        if self.top_logprobs is not None and self.top_logprobs < 0:
            raise InvalidArgumentError("top_logprobs must not be negative")

    @property
    def uses_history(self) -> bool:
        return self.frequency_penalty != 0.0 or self.presence_penalty != 0.0 or self.repetition_penalty != 1.0


@dataclass(frozen=True)
class TokenLogprob:
    token_id: int
    logprob: float


@dataclass(frozen=True)
class SamplingLogprobs:
    """The chosen token's log-probability and the most probable tokens, best first."""

    logprob: float
    top_logprobs: tuple[TokenLogprob, ...] = ()


@dataclass(frozen=True)
class SamplingResult:
    token_id: int
    logprobs: SamplingLogprobs | None = None


class Sampler:
    """Selects tokens on the device; only the chosen ids (and the reports asked for) come back."""

    def __init__(self, device: torch.device | str, status: torch.Tensor | None = None):
        """``status``: the device status word the kernels report into; one of its own unless given
        (sharing the model runner's lets a single read per step cover both)."""
        self.device = torch.device(device)
        self.status = status if status is not None else ops.new_status(self.device)
        self._pinned_rings: dict = {}

    def _launch(self, logits: torch.Tensor, params: Sequence[SamplingParams],
                generators: Sequence[MT19937_64 | None], histories: Sequence[Sequence[int]] | None,
                prompt_lengths: Sequence[int] | None) -> ops.SampleOutput:
        rows, vocab = logits.shape
        if rows != len(params) or rows != len(generators):
            raise InvalidArgumentError("one SamplingParams and one generator per row of logits")
        if all(p.greedy and p.top_logprobs is None and not p.uses_history and not p.logits_bias for p in params):
            return ops.sample_rows(logits, None, self.status)
        records, adjustments = [], []
        # Draws are taken in row order, one per non-greedy row (src/sampler/sampler.cpp:326-333).
        for r, (p, g) in enumerate(zip(params, generators)):
            uniform = 0.0
            if not p.greedy:
                if g is None:
                    raise InvalidArgumentError("a sampled row needs a generator")
                uniform = g.next_uniform()
            records.append(ops.SampleRow(
                temperature=float(p.temperature), uniform=uniform,
                top_k=min(p.top_k, vocab) if p.top_k > 0 else 0,
                top_p=float(p.top_p) if not p.greedy and 0.0 < p.top_p < 1.0 else 0.0,
                min_p=float(p.min_p) if not p.greedy and 0.0 < p.min_p < 1.0 else 0.0,
                num_logprobs=-1 if p.top_logprobs is None else min(int(p.top_logprobs), vocab),
                frequency_penalty=float(p.frequency_penalty), presence_penalty=float(p.presence_penalty),
                repetition_penalty=float(p.repetition_penalty)))
            # History and biases merge into one record per token (src/sampler/sampler.cpp:112-139):
            # how often the token was generated, whether it occurs at all, and its bias.
            merged: dict[int, list] = {}
            if p.uses_history:
                if histories is None or prompt_lengths is None:
                    raise InvalidArgumentError("penalties need the request's token history and prompt length")
                history, prompt_length = histories[r], prompt_lengths[r]
                if prompt_length > len(history):
                    raise InvalidArgumentError("sampling history must include the complete prompt")
                for position, token in enumerate(history):
                    if not 0 <= token < vocab:
                        continue
                    entry = merged.setdefault(token, [0, False, 0.0])
                    entry[1] = True
                    if position >= prompt_length:
                        entry[0] += 1
            for token, bias in p.logits_bias.items():
                merged.setdefault(int(token), [0, False, 0.0])[2] = float(bias)
            adjustments.extend(ops.TokenAdjustment(r, token, count, seen, bias)
                               for token, (count, seen, bias) in merged.items())
        return ops.sample_rows(logits, records, self.status, adjustments)

    def sample_async(self, logits: torch.Tensor, params: Sequence[SamplingParams],
                     generators: Sequence[MT19937_64 | None], histories: Sequence[Sequence[int]] | None = None,
                     prompt_lengths: Sequence[int] | None = None) -> torch.Tensor:
        """Launch the selection; returns the rows' chosen ids, int32, on the device.  For rows that
        ask for no report.  Penalties and biases change ``logits`` in place."""
        if any(p.top_logprobs is not None for p in params):
            raise InvalidArgumentError("sample_async returns ids only; use sample() for rows that report")
        return self._launch(logits, params, generators, histories, prompt_lengths).ids

    def launch(self, logits: torch.Tensor, params: Sequence[SamplingParams],
               generators: Sequence[MT19937_64 | None], histories: Sequence[Sequence[int]] | None = None,
               prompt_lengths: Sequence[int] | None = None) -> "PendingSample":
        """Launch the selection and the copy of its results to the host; ``finish`` waits for them.
        Between the two the host is free while the device works."""
        for p in params:
            p.validate(logits.shape[1])
        out = self._launch(logits, params, generators, histories, prompt_lengths)
        # One wait brings the ids and the status word: every wait for the device costs the step time.
        # Both are copied into one pinned buffer taken from a small ring (no kernel, no allocation).
        count, words = out.ids.numel(), self.status.numel()
        host_ids = self._pinned("ids", count + words, out.ids.dtype)
        host_ids[:count].copy_(out.ids, non_blocking=True)
        host_ids[count:].copy_(self.status, non_blocking=True)
        host_values = None
        if out.logprobs is not None:
            host_values = self._pinned("values", out.logprobs.numel(), out.logprobs.dtype)
            host_values.copy_(out.logprobs.reshape(-1), non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        return PendingSample(list(params), out.offsets, logits.shape[1], host_ids, host_values, done, out.ids)

    PINNED_RING = 4       # selections that may be under way or unread at a time (the engine keeps at most two)

    def _pinned(self, what: str, numel: int, dtype: torch.dtype) -> torch.Tensor:
        """A pinned host buffer of ``numel`` elements: the ring's next one, grown when too small."""
        ring = self._pinned_rings.setdefault((what, dtype), {"turn": 0, "buffers": [None] * self.PINNED_RING})
        turn = ring["turn"]
        ring["turn"] = (turn + 1) % self.PINNED_RING
        buffer = ring["buffers"][turn]
        if buffer is None or buffer.numel() < numel:
            buffer = ring["buffers"][turn] = torch.empty(max(numel, 64), dtype=dtype, pin_memory=True)
        return buffer[:numel]

    def finish(self, pending: "PendingSample") -> list[SamplingResult]:
        """Wait for a launched selection; one ``SamplingResult`` per row."""
        pending.done.synchronize()
        ids = pending.host_ids.tolist()
        if ids[-4] != 0:
            ops.check_status(self.status, "step")
        del ids[-4:]
        values = pending.host_values.tolist() if pending.host_values is not None else None
        results = []
        for p, at in zip(pending.params, pending.offsets):
            report = None
            if p.top_logprobs is not None:
                n = min(int(p.top_logprobs), pending.vocab)
                report = SamplingLogprobs(values[at], tuple(TokenLogprob(ids[at + 1 + k], values[at + 1 + k])
                                                             for k in range(n)))
            results.append(SamplingResult(ids[at], report))
        return results

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams],
               generators: Sequence[MT19937_64 | None], histories: Sequence[Sequence[int]] | None = None,
               prompt_lengths: Sequence[int] | None = None) -> list[SamplingResult]:
        """One ``SamplingResult`` per row.  ``histories`` (prompt and generated tokens) and
        ``prompt_lengths`` are needed for rows with penalties.  Penalties and biases change
        ``logits`` in place."""
        return self.finish(self.launch(logits, params, generators, histories, prompt_lengths))


@dataclass
class PendingSample:
    """A selection that has been launched: its results are on their way to the host."""

    params: list
    offsets: list
    vocab: int
    host_ids: torch.Tensor
    host_values: torch.Tensor | None
    done: "torch.cuda.Event"
    device_ids: torch.Tensor          # the rows' results on the device (a row's chosen id at its offset)
