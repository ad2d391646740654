"""A plain, slow restatement of the reference's sampler in float64, for the tests.

Written from the reference's formulas (src/sampler/sampler.cpp, src/sampler/sampler.cu); it shares
no code with the package.  One function per step:

  adjust       penalties and biases of a request's history          sampler.cpp:112-139, sampler.cu:28-56
  scale        z = (x - max) / T, T = 1 for greedy rows             sampler.cu:82-83, sampler.cpp:97
  rank         descending by value, equal values by index           deps/ttl/include/ttl/ops/topk.hpp:27-29
  keep         top-k, top-p and min-p over the ranked candidates    sampler.cu:99-118
  draw         first positive candidate whose prefix sum exceeds    sampler.cu:150-167
               u * total, else the last positive one
  report       log-softmax of z over the whole vocabulary           sampler.cu:178-194, sampler.cpp:173-176

Every function also says how close its decision came to going the other way (a margin relative to
the total mass), so that a test can tell a fault from a fair difference in the last bits.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64
GREEDY_TEMPERATURE = 1e-7


def adjust(logits: torch.Tensor, history, prompt_length: int, frequency_penalty: float = 0.0,
           presence_penalty: float = 0.0, repetition_penalty: float = 1.0, bias=None) -> torch.Tensor:
    """The adjusted logits, computed in float32 as the reference does (one update per token)."""
    out = logits.clone().to(torch.float32)
    vocab = out.numel()
    generated: dict[int, int] = {}
    seen = set()
    if frequency_penalty != 0.0 or presence_penalty != 0.0 or repetition_penalty != 1.0:
        for position, token in enumerate(history):
            if not 0 <= token < vocab:
                continue
            seen.add(token)
            if position >= prompt_length:
                generated[token] = generated.get(token, 0) + 1
    f32 = lambda v: torch.tensor(v, dtype=torch.float32)
    for token in sorted(seen | set(bias or {})):
        score = out[token]
        if generated.get(token, 0) > 0:
            score = score - f32(frequency_penalty) * f32(float(generated[token]))
            score = score - f32(presence_penalty)
        if token in seen and repetition_penalty != 1.0:
            score = score / f32(repetition_penalty) if score > 0 else score * f32(repetition_penalty)
        score = score + f32((bias or {}).get(token, 0.0))
        out[token] = score
    return out


def scale(logits: torch.Tensor, temperature: float) -> torch.Tensor:
    """Formed in double and stored as float, as the reference does; later steps start from that value."""
    x = logits.to(F64)
    z = (x - x.max()) / (1.0 if temperature < GREEDY_TEMPERATURE else temperature)
    return z.to(torch.float32).to(F64)


def rank(values: torch.Tensor) -> torch.Tensor:
    """Indices by descending value, equal values by ascending index."""
    return torch.sort(values, descending=True, stable=True).indices


def draw(weights: torch.Tensor, uniform: float) -> tuple[int, float]:
    """Position of the drawn candidate and the margin of the draw."""
    cdf = torch.cumsum(weights, 0)
    total = float(cdf[-1])
    target = min(uniform * total, math.nextafter(total, 0.0))
    positive = weights > 0
    crossing = torch.nonzero(positive & (cdf > target))
    at = int(crossing[0]) if crossing.numel() else int(torch.nonzero(positive)[-1])
    low = float(cdf[at - 1]) if at > 0 else 0.0
    return at, min(target - low, float(cdf[at]) - target) / total


def sample(logits: torch.Tensor, temperature: float, uniform: float, top_k: int = -1, top_p: float = 1.0,
           min_p: float = 0.0) -> tuple[int, float]:
    """The chosen token and the smallest margin of the decisions that led to it."""
    z = scale(logits, temperature)
    if temperature < GREEDY_TEMPERATURE:
        return int(rank(z)[0]), 1.0
    vocab = z.numel()
    p = torch.exp(z)
    p = p / p.sum()
    top_p = top_p if 0.0 < top_p < 1.0 else 0.0
    min_p = min_p if 0.0 < min_p < 1.0 else 0.0
    margin = 1.0
    if top_k > 0 or top_p > 0.0:
        order = rank(p)
        k = min(top_k, vocab) if top_k > 0 else vocab
        weights = p[order].clone()
        keep = torch.arange(vocab) < k
        if top_p > 0.0:
            cdf = torch.cumsum(weights, 0)
            before = torch.cat([torch.zeros(1, dtype=F64), cdf[:-1]])
            threshold = top_p * cdf[k - 1]
            inside = before < threshold
            inside[0] = True
            margin = min(margin, float((before[1:k] - threshold).abs().min() / cdf[k - 1]) if k > 1 else 1.0)
            keep &= inside
        if min_p > 0.0:
            keep &= weights > min_p * p.max()
            margin = min(margin, float((weights - min_p * p.max()).abs().min() / p.max()))
        weights[~keep] = 0.0
        at, m = draw(weights, uniform)
        return int(order[at]), min(margin, m)
    weights = p.clone()
    if min_p > 0.0:
        weights[~(p > min_p * p.max())] = 0.0
        margin = min(margin, float((p - min_p * p.max()).abs().min() / p.max()))
    at, m = draw(weights, uniform)
    return at, min(margin, m)


def report(logits: torch.Tensor, temperature: float, token: int, count: int):
    """(log-probability of ``token``, [(token, log-probability)] of the ``count`` best)."""
    logp = torch.log_softmax(scale(logits, temperature), 0)
    best = rank(logp)[:count]
    return float(logp[token]), [(int(i), float(logp[i])) for i in best]
