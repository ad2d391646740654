"""Building traces (the ways of cutting the same requests into steps) and checking replayed logits
against the plain implementation."""

from __future__ import annotations

import functools
import random
from pathlib import Path

import numpy as np
import torch

from plain_qwen3 import load_model_folder, plain_forward

FP32_TOL = 1e-4        # 32-bit path: max abs logit error, as a fraction of max(1, the row's largest |logit|)
# bfloat16: the bound on a row of logits is BF16_UNITS * 2^-8 * the row's largest |logit|.  2^-8 is one
# unit in the last place of a bfloat16 value below 2; the hidden state is rounded to bfloat16 about six
# times a layer, each rounding moves a logit by a random amount of about 2^-9 of the logits' spread, the
# movements add in quadrature (a factor of 3 to 13 for 2 to 28 layers) and the worst of a few hundred
# thousand logits lies four to five deviations out.  The worst ratio seen is printed by the tests
# (``pytest -s``); it stays below 4 on every configuration.
BF16_UNITS = 8.0
WORST: dict = {}       # (what, dtype) -> worst error seen, in units of its bound


def random_tokens(vocab: int, length: int, seed: int) -> list[int]:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(length)]


@functools.lru_cache(maxsize=64)
def _plain_cached(folder: str, tokens: tuple[int, ...]) -> np.ndarray:
    config, weights = load_model_folder(folder)
    return plain_forward(config, weights, list(tokens)).numpy()


def plain_logits(folder, tokens) -> np.ndarray:
    """[T, vocab] float64 logits of the whole sequence from the plain implementation."""
    return _plain_cached(str(folder), tuple(tokens))


def tolerance(dtype: str, expected_row: np.ndarray) -> float:
    """The bound on the largest error in one row of logits."""
    largest = float(np.abs(expected_row).max())
    if dtype == "float32":
        return FP32_TOL * max(1.0, largest)
    return BF16_UNITS * 2.0 ** -8 * largest


# ------------------------------------------------------------------------- traces
def trace_whole(requests: dict[str, list[int]]) -> list[dict]:
    """Each request alone and whole: one step, every position wanted."""
    steps = []
    for rid, tokens in requests.items():
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": tokens, "want": list(range(len(tokens)))}],
                      "end": [rid]})
    return steps


def trace_tail(requests: dict[str, list[int]], tail: int = 32) -> list[dict]:
    """Most of it in one step, then the last ``tail`` tokens one by one."""
    steps = []
    for rid, tokens in requests.items():
        head = max(1, len(tokens) - tail)
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": tokens[:head], "want": [head - 1]}],
                      "end": []})
        for index in range(head, len(tokens)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [tokens[index]], "want": [0]}],
                          "end": [rid] if index == len(tokens) - 1 else []})
        if head == len(tokens):
            steps[-1]["end"] = [rid]
    return steps


def trace_portions(requests: dict[str, list[int]], sizes=(7, 2, 5, 3, 2, 11, 2, 4, 1, 6)) -> list[dict]:
    """Portions of changing size, down to two tokens (and one), every position wanted."""
    steps = []
    for rid, tokens in requests.items():
        start, turn = 0, 0
        while start < len(tokens):
            count = min(sizes[turn % len(sizes)], len(tokens) - start)
            steps.append({"step": len(steps),
                          "entries": [{"id": rid, "tokens": tokens[start:start + count], "want": list(range(count))}],
                          "end": [rid] if start + count == len(tokens) else []})
            start += count
            turn += 1
    return steps


def trace_mixed(requests: dict[str, list[int]], max_live: int = 4, seed: int = 0, tail: int = 12,
                sizes=(9, 2, 6, 3, 13, 2, 5)) -> list[dict]:
    """Up to ``max_live`` requests at a time: portions of some beside single tokens of others; a
    request is sometimes left out of a step; as one ends the next starts, so its pages are used
    again.  Every position is wanted."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    live: dict[str, int] = {}       # id -> tokens fed so far
    turn: dict[str, int] = {}
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, _ = waiting.pop(0)
            live[rid] = 0
            turn[rid] = rng.randrange(len(sizes))
        entries, ended = [], []
        for rid in list(live):
            if len(live) > 1 and rng.random() < 0.2:
                continue        # left out of this step; goes on later
            tokens = requests[rid]
            done = live[rid]
            remaining = len(tokens) - done
            count = 1 if remaining <= tail else min(sizes[turn[rid] % len(sizes)], remaining - tail)
            turn[rid] += 1
            entries.append({"id": rid, "tokens": tokens[done:done + count], "want": list(range(count))})
            live[rid] = done + count
            if live[rid] == len(tokens):
                ended.append(rid)
        if not entries:
            continue
        for rid in ended:
            del live[rid]
        steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps


def trace_batched_tail(requests: dict[str, list[int]], max_live: int = 4, tail: int = 32) -> list[dict]:
    """Groups of up to ``max_live`` requests: each request's head in a step of its own, then the last
    ``tail`` tokens of the whole group decoded together, one token per request and step (a request
    that is shorter than the others ends first)."""
    steps = []
    names = list(requests)
    for start in range(0, len(names), max_live):
        group = names[start:start + max_live]
        fed = {}
        for rid in group:
            tokens = requests[rid]
            head = max(1, len(tokens) - tail)
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": tokens[:head], "want": [head - 1]}],
                          "end": [rid] if head == len(tokens) else []})
            fed[rid] = head
        while any(fed[rid] < len(requests[rid]) for rid in group):
            entries, ended = [], []
            for rid in group:
                if fed[rid] < len(requests[rid]):
                    entries.append({"id": rid, "tokens": [requests[rid][fed[rid]]], "want": [0]})
                    fed[rid] += 1
                    if fed[rid] == len(requests[rid]):
                        ended.append(rid)
            steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps


def peak_tokens(steps: list[dict], round_to: int = 64) -> int:
    """The most tokens live requests hold at any time, each rounded up to a multiple of ``round_to``."""
    held: dict[str, int] = {}
    peak = 0
    for step in steps:
        for entry in step["entries"]:
            held[entry["id"]] = held.get(entry["id"], 0) + len(entry["tokens"])
        peak = max(peak, sum(-(-n // round_to) * round_to for n in held.values()))
        for rid in step["end"]:
            held.pop(rid, None)
    return peak


# ----------------------------------------------------------------------- checking
def collect(steps: list[dict], outputs: dict[int, np.ndarray]) -> dict[tuple[str, int], np.ndarray]:
    """(request, position) -> logits row, from per-step outputs in the order of entries and want."""
    fed: dict[str, int] = {}
    rows: dict[tuple[str, int], np.ndarray] = {}
    for step in steps:
        cursor = 0
        out = outputs.get(step["step"])
        for entry in step["entries"]:
            base = fed.get(entry["id"], 0)
            for place in entry["want"]:
                assert out is not None, f"step {step['step']} wanted logits but produced none"
                rows[(entry["id"], base + place)] = out[cursor]
                cursor += 1
            fed[entry["id"]] = base + len(entry["tokens"])
        assert out is None or cursor == out.shape[0], "more logits rows than wanted places"
    return rows


def first_mismatch(rows, requests, folder, dtype, what: str = ""):
    """The earliest (request, position) whose logits differ from the plain implementation by more than
    the tolerance, with the error; None if all agree.  Also returns the largest error seen, and
    prints it in units of its bound."""
    worst, where, worst_ratio = 0.0, None, 0.0
    first = None
    for (rid, position), got in sorted(rows.items(), key=lambda kv: (kv[0][0], kv[0][1])):
        expected = plain_logits(folder, requests[rid])
        tol = tolerance(dtype, expected[position])
        assert np.isfinite(got).all(), f"non-finite logits for request {rid} position {position}"
        error = float(np.abs(got.astype(np.float64) - expected[position]).max())
        if error > worst:
            worst, where = error, (rid, position)
        worst_ratio = max(worst_ratio, error / tol)
        if error > tol and first is None:
            first = (rid, position, error, tol)
    key = (what or Path(str(folder)).name, dtype)
    WORST[key] = max(WORST.get(key, 0.0), worst_ratio)
    print(f"[logits] {key[0]} {dtype}: worst error {worst:.3e} at {where} = {worst_ratio:.2f} of its bound")
    return first, worst, where


def run_in_process(folder, dtype: str, steps: list[dict], page_size: int, max_tokens: int | None = None,
                   poison: bool = True, max_requests: int = 4, prepare=None) -> dict[int, np.ndarray]:
    """Replay with the engine's ``TraceReplayer`` (what bin/trace_run runs) in this process.
    ``prepare(replayer)`` may change the replayer before the first step."""
    from zephyr_b200.engine.replay import TraceReplayer

    replayer = TraceReplayer(folder, dtype, max_tokens or peak_tokens(steps, max(64, page_size)), page_size=page_size,
                             max_requests=max_requests)
    if prepare is not None:
        prepare(replayer)
    replayer.runner.poison_freed_pages = poison
    outputs = {}
    for step in steps:
        result = replayer.step(step)
        if result is not None:
            outputs[step["step"]] = result
        replayer.runner.manager.check_invariants()
    return outputs
