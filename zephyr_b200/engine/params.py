"""Request parameters and outputs of the Python entry point, with the reference's names
(python/zephyr/engine/inputs.py:16-41, python/zephyr/engine/outputs.py:139-162,
src/include/engine/output.hpp:15-16)."""

from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Mapping, Sequence


class FinishReason(enum.Enum):
    EOS = "eos"
    STOP_TOKEN = "stop_token"
    STOP_STRING = "stop_string"       # never produced here: there is no text front end
    LENGTH = "length"
    MODEL_LENGTH = "model_length"
    CANCELED = "canceled"
    ERROR = "error"


class RequestStatus(enum.Enum):
    COMPLETED = "completed"
    CANCELED = "canceled"
    REJECTED = "rejected"
    ERROR = "error"


@dataclass(frozen=True)
class KvCacheOptions:
    """``block_size`` tokens per page; ``memory_bytes`` for the pool, or None to size it from
    ``gpu_memory_utilization`` (src/include/executor/causal_lm.hpp:16-20).  ``num_blocks`` (this
    engine's addition) fixes the number of pages directly and wins over both."""

    block_size: int = 16
    memory_bytes: int | None = None
    num_blocks: int | None = None


@dataclass(frozen=True, kw_only=True)
class GenerationParams:
    """Per-request overrides.  ``max_tokens`` limits generated tokens, the terminating one included."""

    max_tokens: int | None = None
    n: int = 1
    temperature: float | None = None
    top_k: int | None = None
    top_p: float | None = None
    min_p: float | None = None
    frequency_penalty: float | None = None
    presence_penalty: float | None = None
    repetition_penalty: float | None = None
    logit_bias: Mapping[int, float] | None = None
    top_logprobs: int | None = None
    seed: int | None = None
    stop: str | Sequence[str] | None = None
    stop_token_ids: Sequence[int] = ()
    ignore_eos: bool = False
    include_stop_str_in_output: bool = False
    skip_special_tokens: bool = True

    def __post_init__(self) -> None:
        for name, value, minimum in (("n", self.n, 1), ("max_tokens", self.max_tokens, 1),
                                     ("top_logprobs", self.top_logprobs, 0), ("seed", self.seed, 0)):
            if value is not None and (type(value) is not int or value < minimum):
                raise ValueError(f"{name} must be an integer >= {minimum}")
        if self.seed is not None and self.seed >= 2**64:
            raise ValueError("seed must fit in an unsigned 64-bit integer")
        if self.stop:
            raise ValueError("stop strings need a tokenizer; this engine works on token ids (use stop_token_ids)")
        object.__setattr__(self, "stop_token_ids", tuple(self.stop_token_ids))
        if self.logit_bias is not None:
            object.__setattr__(self, "logit_bias", dict(self.logit_bias))


@dataclass(frozen=True)
class Usage:
    prompt_tokens: int = 0
    completion_tokens: int = 0


@dataclass(frozen=True)
class Choice:
    index: int
    token_ids: tuple[int, ...]
    finish_reason: FinishReason | None = None
    stop_reason: int | None = None
    text: str = ""                    # always empty: no tokenizer is loaded
    logprobs: tuple | None = None     # one SamplingLogprobs per generated token, if top_logprobs was set


@dataclass(frozen=True)
class GenerationOutput:
    request_id: int
    prompt_token_ids: tuple[int, ...]
    choices: tuple[Choice, ...]
    status: RequestStatus | None = None
    usage: Usage = field(default_factory=Usage)
    error_message: str = ""

    @property
    def token_ids(self) -> tuple[int, ...]:
        """The first choice's generated tokens."""
        return self.choices[0].token_ids if self.choices else ()
