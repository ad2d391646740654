"""Trace replay: given token ids, step by step, through the engine's own step function.

``TraceReplayer`` is what ``bin/trace_run`` runs.  It owns nothing but the bookkeeping of which
request ids it has seen: the model, the cache manager, the step function and the kernels are the
ones generation uses (``ModelRunner``).  It samples nothing.
"""

from __future__ import annotations

from pathlib import Path
from typing import Any, Mapping

import numpy as np
import torch

from ..config import InvalidArgumentError, load_model_spec
from ..kernels import ops
from ..parts import Model
from ..weights import Checkpoint
from .engine import resolve_dtype
from .runner import ModelRunner, StepEntry


class TraceReplayer:
    def __init__(self, model_dir: str | Path, dtype: str, max_tokens: int, page_size: int = 16,
                 max_requests: int = 8, device: int = 0):
        if max_tokens <= 0:
            raise InvalidArgumentError("max_tokens must be positive")
        if page_size <= 0 or page_size & (page_size - 1) or page_size > 64:
            raise InvalidArgumentError("the page size must be a power of two of at most 64")
        if not torch.cuda.is_available():
            raise ops.KernelError("trace replay needs a CUDA device; the engine has no CPU path")
        ops.library()       # compiles the kernels at the first call, with progress lines
        self.device = torch.device("cuda", device)
        spec = load_model_spec(model_dir)
        model = Model.load(spec, Checkpoint(model_dir), resolve_dtype(dtype), self.device)
        # The pool holds max_tokens tokens; each request's count is rounded up to whole pages by the
        # tables, and 64 is a multiple of every page size allowed here.
        pages = -(-max_tokens // page_size) + 1       # + the null page
        self.runner = ModelRunner(model, page_size, pages, max_requests)
        self.max_requests = max_requests

    def step(self, record: Mapping[str, Any]) -> np.ndarray | None:
        """Run one trace record; returns float32 logits [wanted, vocab], or None if none were wanted."""
        runner = self.runner
        entries = []
        for item in record.get("entries", []):
            if item["id"] not in runner.manager and not runner.add_request(item["id"]):
                raise InvalidArgumentError(
                    f"no state slot left for request {item['id']!r} (at most {self.max_requests} live requests)")
            entries.append(StepEntry(item["id"], item["tokens"], item.get("want", ())))
        result = None
        if entries:
            logits = runner.step(entries)
            if logits.shape[0]:
                result = logits.cpu().numpy().astype("<f4", copy=False)
            runner.check()
        for request_id in record.get("end", []):
            if request_id in runner.manager:
                runner.free_request(request_id)
        return result
