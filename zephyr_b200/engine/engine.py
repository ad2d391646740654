"""The Python entry point: ``Engine(model_dir, ...).generate(token_ids, ...)``.

Option names and meanings follow the reference's ``EngineConfig`` and ``Engine``
(python/zephyr/engine/config.py:30-54, python/zephyr/engine/engine.py:50-117): ``dtype``,
``max_seq_len`` (0 = the model's limit), ``gpu_memory_utilization``, ``scheduler``
(``PagedSchedulerConfig``), ``kv_cache`` (``KvCacheOptions``), ``eos_token_ids``.  Prompts are
token ids; there is no tokenizer here, so text prompts are refused.

The loop is the reference's control loop without its thread (src/engine/engine.cpp:525-589,
src/engine/generation.cpp:13-101): schedule, run one step, sample where a sequence's known tokens
end, apply the finish rules, retire finished sequences.
"""

from __future__ import annotations

import json
import logging
import time
from dataclasses import dataclass, replace
from pathlib import Path
from typing import Any, Iterable, Sequence

import torch

from ..config import ConfigError, InvalidArgumentError, load_model_config
from ..kernels import ops
from ..parts import Model
from ..sampling import MT19937_64, Sampler, SamplingParams
from ..weights import Checkpoint
from .params import (Choice, FinishReason, GenerationOutput, GenerationParams, KvCacheOptions, RequestStatus, Usage)
from .runner import ModelRunner, StepEntry
from .scheduler import PagedSchedulerConfig, ScheduledStep, Scheduler, Sequence as Seq, SequenceState

_LOGGER = logging.getLogger("zephyr_b200")
_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "bf16": torch.bfloat16, "fp32": torch.float32}


def resolve_dtype(dtype: str | torch.dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype in (torch.bfloat16, torch.float32):
            return dtype
    elif dtype in _DTYPES:
        return _DTYPES[dtype]
    raise ConfigError(f"dtype must be 'bfloat16' or 'float32', not {dtype!r}")


@dataclass
class _Request:
    request_id: int
    prompt: tuple[int, ...]
    params: GenerationParams
    sampling: SamplingParams
    max_new_tokens: int
    sequence_ids: list[tuple[int, int]]
    finish_reasons: dict[int, FinishReason | None]
    stop_reasons: dict[int, int | None]
    error_message: str = ""


@dataclass
class EngineStats:
    steps: int = 0
    prefill_tokens: int = 0
    generated_tokens: int = 0
    preemptions: int = 0
    step_seconds: float = 0.0


@dataclass
class _Flight:
    """A step that has been launched: its plan, the sequences it samples for, the selection under way."""

    plan: Any
    sampled: list
    pending: Any


class Engine:
    """One model on one GPU; synchronous batch generation."""

    def __init__(self, model: str | Path, *, dtype: str | torch.dtype = "bfloat16", max_seq_len: int = 0,
                 gpu_memory_utilization: float = 0.9, scheduler: PagedSchedulerConfig | None = None,
                 kv_cache: KvCacheOptions | None = None, eos_token_ids: Sequence[int] | None = None,
                 devices: Sequence[int] = (0,), weights: Any = None, model_config: Any = None):
        if not torch.cuda.is_available():
            raise ops.KernelError("zephyr_b200 needs a CUDA device (sm_100a); there is no CPU path")
        if len(tuple(devices)) != 1:
            raise ConfigError("this engine runs on exactly one GPU")
        if not 0.0 < gpu_memory_utilization <= 1.0:
            raise ConfigError("gpu_memory_utilization must be in (0, 1]")
        self.device = torch.device("cuda", tuple(devices)[0])
        torch.cuda.set_device(self.device)
        self.dtype = resolve_dtype(dtype)
        self.scheduler_config = scheduler or PagedSchedulerConfig()
        self.scheduler_config.validate()
        kv_cache = kv_cache or KvCacheOptions()

        started = time.perf_counter()
        if model_config is None:
            model_config = load_model_config(model)
        self.model_config = model_config
        spec = model_config.to_model_spec()
        self.generation_defaults = self._read_generation_defaults(model) if model is not None else {}
        store = weights if weights is not None else Checkpoint(model)
        self.model = Model.load(spec, store, self.dtype, self.device)
        torch.cuda.empty_cache()        # loading may hold copies (fused matrices) that it no longer needs
        _LOGGER.info("model ready: %s, %s, %.2f s", spec.architecture, self.dtype, time.perf_counter() - started)

        limit = spec.max_seq_len if max_seq_len in (0, None) else min(max_seq_len, spec.max_seq_len)
        num_pages = self._size_cache(kv_cache, gpu_memory_utilization, limit)
        self.runner = ModelRunner(self.model, kv_cache.block_size, num_pages, self.scheduler_config.max_num_seqs,
                                  max_seq_len=limit)
        self.max_seq_len = limit
        self.vocab_size = spec.vocab_size

        eos = eos_token_ids
        if eos is None:
            eos = self.generation_defaults.get("eos_token_id")
        if eos is None:
            eos = spec.eos_token_ids
        if isinstance(eos, int):
            eos = [eos]
        self.eos_token_ids = tuple(int(e) for e in (eos or ()))
        for token in self.eos_token_ids:
            if not 0 <= token < self.vocab_size:
                raise ConfigError(f"eos token id {token} lies outside the vocabulary")

        self.sampler = Sampler(self.device, status=self.runner.status)
        self.sequences: dict[tuple[int, int], Seq] = {}
        self.scheduler = Scheduler(self.scheduler_config, self.sequences, _RunnerCache(self.runner))
        self._requests: dict[int, _Request] = {}
        self._generators: dict[tuple[int, int], MT19937_64] = {}
        self._logprobs: dict[tuple[int, int], list] = {}
        self._seed_source = MT19937_64(0)     # seeds for requests that bring none (engine.hpp:162)
        self._next_request_id = 0
        self.stats = EngineStats()
        self._closed = False
        # While the device runs a step of decoders only, the host plans and describes the next one
        # (all but its tokens): ``look_ahead`` turns that off.
        self.look_ahead = True
        self.launch_ahead = True                # ... and launches it where its tokens can stay on the device
        self._flight = None                     # the step launched ahead: its plan and its selection under way
        self._ahead = None                      # (plan, prepared) of the step after this one
        self._placeholders: set[tuple[int, int]] = set()   # sequences whose last token is still on the device

    # ------------------------------------------------------------------- set-up
    @staticmethod
    def _read_generation_defaults(model: str | Path) -> dict[str, Any]:
        path = Path(model) / "generation_config.json"
        if not path.exists():
            return {}
        data = json.loads(path.read_text(encoding="utf-8"))
        if not isinstance(data, dict):
            raise ConfigError(f"{path}: the generation configuration must be a JSON object")
        supported = {"temperature", "top_k", "top_p", "min_p", "repetition_penalty", "max_new_tokens", "max_length",
                     "do_sample", "eos_token_id"}
        return {k: v for k, v in data.items() if k in supported}

    def _size_cache(self, kv_cache: KvCacheOptions, utilization: float, max_seq_len: int) -> int:
        """Number of pages: given, or what ``memory_bytes`` buys, or what is left of
        ``gpu_memory_utilization`` x total memory after the weights and after what a step needs at its
        peak.  That peak is measured, as the reference measures its own (src/executor/causal_lm.cpp:
        301-425,495-537): ``_profile_step_peak`` runs the largest prompt portion and the largest decode
        batch the scheduler may form and reads the allocator's high-water mark."""
        block = kv_cache.block_size
        if block <= 0 or block & (block - 1):
            raise ConfigError("kv_cache.block_size must be a power of two")
        self.profiled_step_bytes = None
        if kv_cache.num_blocks is not None:
            pages = int(kv_cache.num_blocks)
        else:
            if kv_cache.memory_bytes is not None:
                budget = int(kv_cache.memory_bytes)
            else:
                self.profiled_step_bytes = self._profile_step_peak(block, max_seq_len)
                torch.cuda.empty_cache()        # what loading and profiling left cached goes back first
                free, total = torch.cuda.mem_get_info(self.device)
                used = total - free
                # Twice the measured peak: a step that runs launch by launch and the same step's captured
                # graph (all graphs share one memory pool) each hold their activations.  Beside it the
                # selection's buffers (a few rows of the vocabulary per sequence) and a fixed reserve.
                transient = 2 * self.profiled_step_bytes \
                    + 4 * self.scheduler_config.max_num_seqs * self.model.spec.vocab_size * 4 + (256 << 20)
                budget = min(free - max(512 << 20, total // 50), int(utilization * total) - used) - transient
            pages = ModelRunner.pages_for_memory(self.model, block, max(budget, 0))
            # No use holding more pages than every resident sequence at full length can fill.
            pages = min(pages, self.scheduler_config.max_num_seqs * -(-max_seq_len // block))
        pages += 1      # the null page
        if pages < 2:
            raise ConfigError("the cache pool has no room for a single page; lower max_seq_len or free memory")
        return pages

    def _profile_step_peak(self, block: int, max_seq_len: int) -> int:
        """Bytes the allocator holds at the peak of a step beyond what is resident: the largest prompt
        step the scheduler may form (``max_num_batched_tokens`` tokens, spread over as many sequences
        as it takes when one sequence cannot be that long), then one decode step of ``max_num_seqs``
        sequences, on a throw-away pool just large enough for them."""
        seqs = self.scheduler_config.max_num_seqs
        portion = max(1, min(self.scheduler_config.max_prefill_chunk_tokens, max_seq_len))
        tokens = max(1, min(self.scheduler_config.max_num_batched_tokens, seqs * portion))
        portions = [portion] * (tokens // portion) + ([tokens % portion] if tokens % portion else [])
        pages = sum(-(-n // block) for n in portions) + seqs + 2
        runner = ModelRunner(self.model, block, pages, seqs + 1, max_seq_len=max_seq_len, use_cuda_graphs=False)
        torch.cuda.synchronize(self.device)
        torch.cuda.reset_peak_memory_stats(self.device)
        base = torch.cuda.memory_allocated(self.device)
        rows = [("profile", index) for index in range(seqs)]
        for row in rows[:len(portions)]:
            runner.add_request(row)
        runner.step([StepEntry(row, [0] * n, (n - 1,)) for row, n in zip(rows, portions)])
        for row in rows[:len(portions)]:
            runner.free_request(row)
        for row in rows:
            runner.add_request(row)
        runner.step([StepEntry(row, [0], (0,)) for row in rows])
        runner.check()
        peak = torch.cuda.max_memory_allocated(self.device) - base
        _LOGGER.info("a step of %d tokens holds %.1f MiB at its peak", tokens, peak / 2**20)
        return max(int(peak), 0)

    # ---------------------------------------------------------------- requests
    def add_request(self, prompt: Sequence[int], params: GenerationParams | None = None) -> int:
        """Queue one request and return its id.  ``step()`` makes progress; ``take_output`` collects."""
        params = params or GenerationParams()
        tokens = [int(t) for t in prompt]
        if not tokens or len(tokens) > self.max_seq_len:
            raise ValueError(f"Input must contain between 1 and {self.max_seq_len} tokens")
        if any(not 0 <= t < self.vocab_size for t in tokens):
            raise ValueError("Input contains a token ID outside the model vocabulary")
        remaining = self.max_seq_len - len(tokens)
        if remaining <= 0:
            raise ValueError("The prompt must leave room for generation within max_seq_len")
        defaults = self.generation_defaults
        maximum = params.max_tokens
        if maximum is None:
            maximum = defaults.get("max_new_tokens")
            if maximum is None and defaults.get("max_length") is not None:
                maximum = defaults["max_length"] - len(tokens)
            maximum = min(remaining, maximum) if maximum is not None else remaining
        if type(maximum) is not int or not 0 < maximum <= remaining:
            raise ValueError(f"max_tokens must be between 1 and {remaining} for this prompt")
        sampling: dict[str, Any] = {}
        for name in ("temperature", "top_k", "top_p", "min_p", "frequency_penalty", "presence_penalty",
                     "repetition_penalty"):
            value = getattr(params, name)
            if value is None:
                value = defaults.get(name)
            if value is not None:
                sampling[name] = value
        if params.temperature is None and defaults.get("do_sample") is False:
            sampling["temperature"] = 0.0
        sampling_params = SamplingParams(**sampling, logits_bias=dict(params.logit_bias or {}),
                                         top_logprobs=params.top_logprobs)
        sampling_params.validate(self.vocab_size)
        for token in params.stop_token_ids:
            if not 0 <= int(token) < self.vocab_size:
                raise ValueError("stop_token_ids contains a token outside the vocabulary")

        request_id = self._next_request_id
        self._next_request_id += 1
        request = _Request(request_id, tuple(tokens), params, sampling_params, maximum, [], {}, {})
        for choice in range(params.n):
            key = (request_id, choice)
            self.sequences[key] = Seq(key, list(tokens))
            seed = params.seed + choice if params.seed is not None else self._seed_source.next_u64()
            self._generators[key] = MT19937_64(seed)
            request.sequence_ids.append(key)
            request.finish_reasons[choice] = None
            request.stop_reasons[choice] = None
            self.scheduler.add(key)
        self._requests[request_id] = request
        return request_id

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished

    # -------------------------------------------------------------------- step
    def step(self) -> int:
        """Schedule and run one step; returns the number of tokens it computed (0: nothing to do).
        The step may have been launched already, during the call before (see ``_launch_ahead``)."""
        started = time.perf_counter()
        flight = self._settle_flight()
        if flight is None:
            flight = self._run_step()
            if flight is None:
                return 0
        plan = flight.plan
        if flight.pending is not None:
            # Host work while the device runs the step: the next step is planned and described, and,
            # where its tokens can go from this step's selection to its input on the device, launched.
            ahead = self._plan_ahead(plan)
            if ahead is not None and ahead[1] is not None:
                self._flight = self._launch_ahead(flight, ahead)
                if self._flight is not None:
                    ahead = None
            results = self.sampler.finish(flight.pending)        # also reads the step's status
            for item, result in zip(flight.sampled, results):
                sequence = self.sequences.get(item.sequence_id)
                if sequence is None or sequence.is_terminal:
                    continue        # ended or cancelled while its step was under way
                if result.logprobs is not None:
                    self._logprobs.setdefault(item.sequence_id, []).append(result.logprobs)
                self._append_token(item.sequence_id, int(result.token_id))
                self.stats.generated_tokens += 1
            self._ahead = ahead
        self.stats.steps += 1
        self.stats.preemptions = self.scheduler.num_preemptions
        self.stats.step_seconds += time.perf_counter() - started
        return plan.num_tokens

    def _run_step(self) -> "_Flight | None":
        """Schedule a step (or take the plan made ahead), run it and launch its selection."""
        plan, prepared = self._take_ahead()
        if plan is None:
            plan = self.scheduler.schedule()
        for key in plan.rejected:
            request = self._requests[key[0]]
            request.error_message = self.sequences[key].error_message
            request.finish_reasons[key[1]] = FinishReason.ERROR
        if not plan.sequences:
            if self.scheduler.has_unfinished and not plan.preempted and not plan.rejected:
                raise RuntimeError("the scheduler made no progress although sequences are unfinished")
            return None
        logits = self.runner.step(self._entries(plan), prepared)
        self.scheduler.commit(plan)
        self.stats.prefill_tokens += sum(i.num_tokens for i in plan.sequences if i.num_tokens > 1 or not i.sample)
        sampled = [item for item in plan.sequences if item.sample]
        return _Flight(plan, sampled, self._launch_selection(logits, sampled) if sampled else None)

    def _launch_selection(self, logits: torch.Tensor, sampled):
        params = [self._requests[i.sequence_id[0]].sampling for i in sampled]
        generators = [self._generators[i.sequence_id] for i in sampled]
        sequences = [self.sequences[i.sequence_id] for i in sampled]
        return self.sampler.launch(logits, params, generators, [s.token_ids for s in sequences],
                                   [s.prompt_length for s in sequences])

    def _entries(self, plan) -> list[StepEntry]:
        entries = []
        for item in plan.sequences:
            sequence = self.sequences[item.sequence_id]
            tokens = sequence.token_ids[item.start_token:item.start_token + item.num_tokens]
            entries.append(StepEntry(item.sequence_id, tokens, (item.num_tokens - 1,) if item.sample else ()))
        return entries

    # ------------------------------------------------------------ one step ahead
    def _plan_ahead(self, plan):
        """Called between the launch of a step's selection and the wait for its tokens.  If the step
        after this one is known but for its tokens (every resident sequence is decoding and got its
        token in this step, nothing waits for admission, no sequence reaches a length limit with the
        token on its way), schedule it now and let the runner describe it: when the tokens arrive only
        they are missing.  A sequence that then ends on its token (end of sequence, a stop token) or
        anything else that changes the picture makes ``_take_ahead`` drop the plan; the scheduler is
        asked again and decides on what it finds, as it always does."""
        scheduler = self.scheduler
        if (not self.look_ahead or scheduler.waiting or len(plan.sequences) != len(scheduler.running)
                or len(plan.sequences) > self.scheduler_config.max_num_batched_tokens
                or not all(item.sample for item in plan.sequences)):
            return None
        for item in plan.sequences:
            sequence = self.sequences[item.sequence_id]
            request = self._requests[item.sequence_id[0]]
            if (sequence.state != SequenceState.DECODE or item.sequence_id not in scheduler.running
                    or len(sequence.token_ids) - sequence.prompt_length + 1 >= request.max_new_tokens
                    or len(sequence.token_ids) >= self.max_seq_len - 1):
                return None
        for item in plan.sequences:
            self.sequences[item.sequence_id].token_ids.append(-1)      # stands for the token on its way
            self._placeholders.add(item.sequence_id)
        ahead = scheduler.schedule()
        if ahead.preempted or ahead.rejected or not ahead.sequences:
            return (ahead, None)
        return (ahead, self.runner.prepare(self._entries(ahead)))

    def _launch_ahead(self, flight: "_Flight", ahead) -> "_Flight | None":
        """Launch the step after ``flight`` before ``flight``'s tokens have reached the host: they go
        from its selection's output to the next step's input on the device.  The device then never
        waits for the host between two decode steps.  Only where nothing about the next step depends
        on the tokens' values: the same sequences in the same order, one row of ids each, no
        penalties (they need the history on the host).  A sequence that turns out to have ended on
        its token has computed one token in vain; ``_settle_flight`` drops it."""
        plan, prepared = ahead
        sampled = flight.sampled
        if (not self.launch_ahead or [i.sequence_id for i in plan.sequences] != [i.sequence_id for i in sampled]
                or flight.pending.offsets != list(range(len(sampled)))
                or any(self._requests[i.sequence_id[0]].sampling.uses_history for i in plan.sequences)):
            return None
        entries = self._entries(plan)
        if not self.runner.holds(prepared, entries):
            return None
        logits = self.runner.step(entries, prepared, device_tokens=flight.pending.device_ids)
        return _Flight(plan, list(plan.sequences), self._launch_selection(logits, plan.sequences))

    def _settle_flight(self) -> "_Flight | None":
        """The step launched ahead, now that the tokens of the step before it are known: sequences
        that ended meanwhile fall out of it (their row was computed in vain); None if no step is
        under way or none of its sequences is left."""
        flight, self._flight = self._flight, None
        if flight is None:
            return None
        alive = [item for item in flight.plan.sequences
                 if item.sequence_id in self.sequences and self.sequences[item.sequence_id].state == SequenceState.DECODE
                 and item.sequence_id in self.scheduler.running]
        keep = {item.sequence_id for item in alive}
        # The selection's rows stay as they were launched; rows of sequences that ended are skipped
        # when the results are read (``step`` looks at the sequence's state).
        plan = ScheduledStep(sequences=alive, preempted=flight.plan.preempted, rejected=flight.plan.rejected)
        self.scheduler.commit(plan)
        if not keep:
            self.sampler.finish(flight.pending)      # nobody wants them, but the status word is looked at
            return None
        return _Flight(plan, flight.sampled, flight.pending)

    def _take_ahead(self):
        """(plan, prepared) for this step from the plan made one step ahead, or (None, None).  The
        plan is used as it is if it is still what the scheduler would choose: every sequence in it
        decodes on, and nobody waits for admission but those the plan itself preempted.  Otherwise
        the scheduler is asked again; what the dropped plan preempted or rejected has happened and
        is reported with the new plan."""
        ahead, self._ahead = self._ahead, None
        if ahead is None:
            return None, None
        plan, prepared = ahead
        scheduler = self.scheduler
        clean = set(scheduler.waiting) <= set(plan.preempted)
        for item in plan.sequences:
            sequence = self.sequences.get(item.sequence_id)
            if (sequence is None or sequence.state != SequenceState.DECODE or item.sequence_id not in scheduler.running
                    or item.start_token + item.num_tokens != len(sequence.token_ids)):
                clean = False
        if clean:
            return plan, prepared
        fresh = scheduler.schedule()
        fresh.preempted[:0] = plan.preempted
        fresh.rejected[:0] = plan.rejected
        return fresh, None

    def _append_token(self, key: tuple[int, int], token: int) -> None:
        """The finish rules in the reference's order (src/engine/generation.cpp:81-99).  The sampled
        token enters the history now; its cache entry is made by the next step."""
        sequence = self.sequences[key]
        request = self._requests[key[0]]
        if key in self._placeholders:          # the plan made ahead already counts this token
            self._placeholders.discard(key)
            sequence.token_ids.pop()
        reason = None
        if not request.params.ignore_eos and token in self.eos_token_ids:
            reason = FinishReason.EOS
        elif token in request.params.stop_token_ids:
            reason = FinishReason.STOP_TOKEN
            request.stop_reasons[key[1]] = token
        elif len(sequence.token_ids) - sequence.prompt_length + 1 >= request.max_new_tokens:
            reason = FinishReason.LENGTH
        elif len(sequence.token_ids) >= self.max_seq_len:
            reason = FinishReason.MODEL_LENGTH
        sequence.token_ids.append(token)
        if reason is not None:
            request.finish_reasons[key[1]] = reason
            self.scheduler.finish(key)

    def cancel(self, request_id: int) -> None:
        request = self._requests[request_id]
        for key in request.sequence_ids:
            if not self.sequences[key].is_terminal:
                request.finish_reasons[key[1]] = FinishReason.CANCELED
                self.scheduler.finish(key)

    def is_finished(self, request_id: int) -> bool:
        return all(self.sequences[key].is_terminal for key in self._requests[request_id].sequence_ids)

    def take_output(self, request_id: int) -> GenerationOutput:
        """The finished request's output; the engine forgets the request."""
        request = self._requests.pop(request_id)
        choices = []
        states = []
        for key in request.sequence_ids:
            sequence = self.sequences.pop(key)
            self._generators.pop(key, None)
            states.append(sequence.state)
            reports = self._logprobs.pop(key, None)
            choices.append(Choice(key[1], tuple(sequence.token_ids[sequence.prompt_length:]),
                                  request.finish_reasons[key[1]], request.stop_reasons[key[1]],
                                  logprobs=tuple(reports) if reports is not None else None))
        if any(s == SequenceState.REJECTED for s in states):
            status = RequestStatus.REJECTED
        elif any(s == SequenceState.ERROR for s in states):
            status = RequestStatus.ERROR
        elif any(c.finish_reason == FinishReason.CANCELED for c in choices):
            status = RequestStatus.CANCELED
        else:
            status = RequestStatus.COMPLETED
        usage = Usage(len(request.prompt), sum(len(c.token_ids) for c in choices))
        return GenerationOutput(request_id, request.prompt, tuple(choices), status, usage, request.error_message)

    # ---------------------------------------------------------------- generate
    def generate(self, prompts, params: GenerationParams | None = None, **kwargs: Any):
        """Generate for one prompt (a sequence of token ids) or a batch (a sequence of those); keyword
        arguments override ``params``.  Returns one ``GenerationOutput`` or a list in input order."""
        if self._closed:
            raise RuntimeError("the engine is closed")
        params = replace(params, **kwargs) if params is not None else GenerationParams(**kwargs)
        if isinstance(prompts, str) or (isinstance(prompts, Sequence) and prompts and isinstance(prompts[0], str)):
            raise ValueError("Text APIs require a tokenizer; this engine takes token ids")
        single = isinstance(prompts, Sequence) and bool(prompts) and isinstance(prompts[0], int)
        inputs: Iterable[Sequence[int]] = [prompts] if single else prompts
        ids = [self.add_request(prompt, params) for prompt in inputs]
        while any(not self.is_finished(i) for i in ids):
            self.step()
        outputs = [self.take_output(i) for i in ids]
        return outputs[0] if single else outputs

    def close(self) -> None:
        self._closed = True

    def __enter__(self) -> "Engine":
        return self

    def __exit__(self, *exc: Any) -> None:
        self.close()


class _RunnerCache:
    """The scheduler's view of the cache: the manager, with the runner's device-side duties
    (zeroing a new state slot, poisoning freed pages in tests) done on the way."""

    def __init__(self, runner: ModelRunner):
        self._runner = runner

    def add_request(self, request_id, reserve_tokens: int = 0, step_tokens: int = 1) -> bool:
        return self._runner.add_request(request_id, reserve_tokens, step_tokens)

    def ensure_capacity(self, request_id, length: int) -> bool:
        return self._runner.manager.ensure_capacity(request_id, length)

    def free_request(self, request_id) -> None:
        self._runner.free_request(request_id)

    def fits_at_all(self, length: int, step_tokens: int) -> bool:
        return self._runner.manager.fits_at_all(length, step_tokens)
