"""Continuous batching above the step function: admit, cut prompts into portions under a token
budget, decode, finish and free; pure host code.

State machine and rules come from the reference's ``PagedScheduler``
(src/scheduler/paged_scheduler.cpp): FIFO admission that reserves the whole prompt's pages
(:84-142), portions bounded by ``max_num_batched_tokens`` and ``max_prefill_chunk_tokens``
(:37-43,189-217), decoders served oldest first (:231-256), recompute-style preemption of the
youngest sequence when pages run out, with the victim put at the FRONT of the waiting queue and
its generated tokens kept in its history (:161-169), and rejection of a prompt that could never
fit (:95-98).  The difference: the reference returns either a prefill batch or a decode batch and
alternates (``IsDecodeDue`` :45-82); this scheduler builds ONE mixed step: first every resident
decoder's single token, then prompt portions in the token budget that is left.

When pages run out:
  * a decoder cannot grow      -> the youngest running sequence is preempted (itself, if it is the
                                  youngest); it frees everything and will recompute from its tokens;
  * a waiting prompt has no room -> it waits at the head of the queue (nothing behind it overtakes);
  * a prompt needs more pages than the whole pool -> REJECTED, never admitted.
"""

from __future__ import annotations

import enum
from collections import deque
from dataclasses import dataclass, field
from typing import Hashable, Protocol

from ..config.errors import ConfigError, InvalidArgumentError


class SequenceState(enum.Enum):
    WAITING = "waiting"
    PREFILL = "prefill"
    DECODE = "decode"
    FINISHED = "finished"
    ERROR = "error"
    REJECTED = "rejected"


@dataclass
class Sequence:
    """Append-only token history of one choice of a request (src/include/scheduler/sequence.hpp:23-45)."""

    id: Hashable
    token_ids: list[int]
    prompt_length: int = 0
    num_computed_tokens: int = 0
    state: SequenceState = SequenceState.WAITING
    error_message: str = ""
    arrival: int = 0
    num_preemptions: int = 0

    def __post_init__(self) -> None:
        if not self.prompt_length:
            self.prompt_length = len(self.token_ids)

    @property
    def is_terminal(self) -> bool:
        return self.state in (SequenceState.FINISHED, SequenceState.ERROR, SequenceState.REJECTED)


@dataclass(frozen=True)
class PagedSchedulerConfig:
    """Names and defaults of the reference (src/include/engine/engine.hpp:36-39).
    ``max_decode_steps_before_prefill`` is accepted for compatibility and unused: decoders and
    prompt portions share every step here, so neither has to wait for the other."""

    max_num_seqs: int = 8
    max_num_batched_tokens: int = 512
    max_prefill_chunk_tokens: int = 512
    max_decode_steps_before_prefill: int = 8

    def validate(self) -> None:
        if min(self.max_num_seqs, self.max_num_batched_tokens, self.max_prefill_chunk_tokens,
               self.max_decode_steps_before_prefill) <= 0:
            raise ConfigError("Scheduler sequence and token budgets must be positive")


class CacheFacade(Protocol):
    """What the scheduler needs of the cache manager (``CacheManager`` or the runner offers it)."""

    def add_request(self, request_id: Hashable, reserve_tokens: int = 0, step_tokens: int = 1) -> bool: ...
    def ensure_capacity(self, request_id: Hashable, length: int) -> bool: ...
    def free_request(self, request_id: Hashable) -> None: ...
    def fits_at_all(self, length: int, step_tokens: int) -> bool: ...


@dataclass(frozen=True)
class ScheduledSequence:
    sequence_id: Hashable
    start_token: int
    num_tokens: int
    sample: bool          # the portion ends the sequence's known tokens: its last logits pick the next token


@dataclass
class ScheduledStep:
    sequences: list[ScheduledSequence] = field(default_factory=list)
    preempted: list[Hashable] = field(default_factory=list)
    rejected: list[Hashable] = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return sum(s.num_tokens for s in self.sequences)


class Scheduler:
    def __init__(self, config: PagedSchedulerConfig, sequences: dict[Hashable, Sequence], cache: CacheFacade):
        config.validate()
        self.config = config
        self.sequences = sequences
        self.cache = cache
        self.waiting: deque[Hashable] = deque()
        self.running: list[Hashable] = []       # in order of admission
        self._arrivals = 0
        self._decode_cursor = 0
        self.num_preemptions = 0

    # ---------------------------------------------------------------- requests
    def add(self, sequence_id: Hashable) -> None:
        sequence = self.sequences[sequence_id]
        if (sequence.state != SequenceState.WAITING or sequence.num_computed_tokens != 0 or not sequence.token_ids
                or sequence_id in self.waiting or sequence_id in self.running):
            raise InvalidArgumentError("scheduling requires a fresh, nonempty sequence with a unique id")
        sequence.arrival = self._arrivals
        self._arrivals += 1
        self.waiting.append(sequence_id)

    def finish(self, sequence_id: Hashable, state: SequenceState = SequenceState.FINISHED, message: str = "") -> None:
        """Retire a sequence (finished, cancelled or failed) and give back what it holds.  Safe to repeat."""
        sequence = self.sequences[sequence_id]
        if sequence_id in self.running:
            self.running.remove(sequence_id)
            self.cache.free_request(sequence_id)
        elif sequence_id in self.waiting:
            self.waiting.remove(sequence_id)
        if not sequence.is_terminal:
            sequence.state = state
            sequence.error_message = message

    @property
    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    # -------------------------------------------------------------- scheduling
    def _preempt(self, sequence_id: Hashable, step: ScheduledStep) -> None:
        sequence = self.sequences[sequence_id]
        self.running.remove(sequence_id)
        self.cache.free_request(sequence_id)
        sequence.num_computed_tokens = 0
        sequence.state = SequenceState.WAITING
        sequence.num_preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(sequence_id)
        step.preempted.append(sequence_id)
        step.sequences[:] = [s for s in step.sequences if s.sequence_id != sequence_id]

    def _schedule_decoders(self, step: ScheduledStep) -> int:
        """Every resident decoder gets its one token, oldest first; returns the tokens used."""
        decoders = sorted((i for i in self.running if self.sequences[i].state == SequenceState.DECODE),
                          key=lambda i: self.sequences[i].arrival)
        budget = self.config.max_num_batched_tokens
        if len(decoders) > budget:      # more decoders than budget: take turns
            count = len(decoders)
            start = self._decode_cursor % count
            decoders = (decoders[start:] + decoders[:start])[:budget]
            self._decode_cursor = (start + budget) % count
        used = 0
        for sequence_id in decoders:
            if sequence_id not in self.running:      # preempted a moment ago to make room for an older one
                continue
            sequence = self.sequences[sequence_id]
            while not self.cache.ensure_capacity(sequence_id, len(sequence.token_ids)):
                victim = max(self.running, key=lambda i: self.sequences[i].arrival)
                self._preempt(victim, step)
                if victim == sequence_id:
                    break
            else:
                step.sequences.append(ScheduledSequence(sequence_id, len(sequence.token_ids) - 1, 1, True))
                used += 1
        return used

    def _admit(self, step: ScheduledStep) -> None:
        chunk = min(self.config.max_prefill_chunk_tokens, self.config.max_num_batched_tokens)
        while self.waiting and len(self.running) < self.config.max_num_seqs:
            sequence_id = self.waiting[0]
            sequence = self.sequences[sequence_id]
            length = len(sequence.token_ids)
            if not self.cache.fits_at_all(length, chunk):
                self.waiting.popleft()
                sequence.state = SequenceState.REJECTED
                sequence.error_message = "Sequence exceeds the total usable KV cache capacity"
                step.rejected.append(sequence_id)
                continue
            if sequence_id in step.preempted:
                break           # preempted in this very step: it waits for the next one
            if not self.cache.add_request(sequence_id, reserve_tokens=length, step_tokens=chunk):
                break           # FIFO: nothing overtakes the head of the queue
            self.waiting.popleft()
            sequence.state = SequenceState.PREFILL
            self.running.append(sequence_id)

    def _schedule_prefill(self, step: ScheduledStep, budget: int) -> None:
        for sequence_id in list(self.running):
            if budget <= 0:
                break
            sequence = self.sequences[sequence_id]
            if sequence.state != SequenceState.PREFILL:
                continue
            remaining = len(sequence.token_ids) - sequence.num_computed_tokens
            count = min(remaining, self.config.max_prefill_chunk_tokens, budget)
            if count <= 0 or not self.cache.ensure_capacity(sequence_id, sequence.num_computed_tokens + count):
                continue
            step.sequences.append(ScheduledSequence(sequence_id, sequence.num_computed_tokens, count,
                                                    count == remaining))
            budget -= count

    def schedule(self) -> ScheduledStep:
        """Choose the next step's work.  The caller runs it, then calls ``commit`` with the result."""
        step = ScheduledStep()
        for sequence_id in [i for i in self.running if self.sequences[i].is_terminal]:
            self.finish(sequence_id)
        used = self._schedule_decoders(step)
        self._admit(step)
        self._schedule_prefill(step, self.config.max_num_batched_tokens - used)
        return step

    def commit(self, step: ScheduledStep) -> None:
        """The step ran: its tokens are in the cache.  A sequence whose tokens are all computed decodes next."""
        for scheduled in step.sequences:
            sequence = self.sequences[scheduled.sequence_id]
            sequence.num_computed_tokens = max(sequence.num_computed_tokens,
                                               scheduled.start_token + scheduled.num_tokens)
            if sequence.state == SequenceState.PREFILL and sequence.num_computed_tokens == len(sequence.token_ids):
                sequence.state = SequenceState.DECODE
