"""A plain, slow implementation of the dense Qwen3 decoder, the yardstick of the tests.

It rests on the reference's formulas, cited function by function (paths are the reference
project's own).  The reference's model code is CUDA-only and cannot run on a CPU; its output on a
B200 for the tiny configuration B (greedy tokens and full rows of log-probabilities) is stored under
tests/golden/ with the script that made it, and tests/test_reference_anchor.py compares this
implementation with it.  Whole sequences, no cache, float64 arithmetic, one function per part, and no
code shared with the engine: this file imports nothing from ``zephyr_b200`` and reads model folders
with the ``safetensors`` package.

Where the reference rounds to the storage type between operations (after each norm, inside the
rotation, between silu and the product), this implementation does not round at all: it is the
exact value that both the reference and the engine approximate.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import numpy as np
import torch

F64 = torch.float64


# ------------------------------------------------------------------ model folder
def load_model_folder(model_dir) -> tuple[dict, dict[str, torch.Tensor]]:
    """config.json as a dict and every tensor of model.safetensors as float64."""
    from safetensors import safe_open

    model_dir = Path(model_dir)
    config = json.loads((model_dir / "config.json").read_text())
    tensors = {}
    with safe_open(str(model_dir / "model.safetensors"), framework="pt", device="cpu") as handle:
        for name in handle.keys():
            tensors[name] = handle.get_tensor(name).to(F64)
    return config, tensors


def head_dim_of(config: dict) -> int:
    """head_dim, or hidden_size / heads when absent or null (src/model/causal_lm/qwen3_config.cpp:53-57)."""
    if config.get("head_dim") is not None:
        return int(config["head_dim"])
    return int(config["hidden_size"]) // int(config["num_attention_heads"])


def layer_window(config: dict, layer: int) -> int:
    """0 for full attention, else the number of positions a query sees, its own included.  Qwen3 has
    none: the reference rejects windows (qwen3_config.cpp:63-80).  The tests' own windowed
    architecture names them per layer under ``layer_windows``."""
    windows = config.get("layer_windows")
    return int(windows[layer]) if windows is not None else 0


# ------------------------------------------------------------------------- parts
def plain_embedding(table: torch.Tensor, token_ids) -> torch.Tensor:
    """h[t, :] = E[id[t], :], no scaling (src/layer/embedding.cpp:17-31)."""
    return table[torch.as_tensor(list(token_ids), dtype=torch.long)]


def plain_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w over the last dimension; the weight multiplies after the
    normalisation (deps/ttl/src/kernels/normalization/normalization.cu:76-139, src/layer/normalization.cpp:15-18)."""
    mean_square = (x * x).mean(dim=-1, keepdim=True)
    return x / torch.sqrt(mean_square + eps) * weight


def plain_rope_tables(head_dim: int, num_positions: int, theta: float) -> tuple[torch.Tensor, torch.Tensor]:
    """inv_freq[i] = 1 / theta^(2i / hd) and angle = p * inv_freq[i], both in float32 as the
    reference computes them on the host (src/layer/rotary_embedding.cpp:36-55); then cos and sin of
    that float32 angle."""
    index = np.arange(head_dim // 2, dtype=np.float32)
    exponent = (np.float32(2.0) * index) / np.float32(head_dim)
    inv_freq = (np.float32(1.0) / np.power(np.float32(theta), exponent, dtype=np.float32)).astype(np.float32)
    angles = (np.arange(num_positions, dtype=np.float32)[:, None] * inv_freq[None, :]).astype(np.float32)
    angles64 = torch.from_numpy(angles.astype(np.float64))
    return torch.cos(angles64), torch.sin(angles64)


def plain_rope(x: torch.Tensor, positions, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """NeoX rotation of x [T, heads, hd]: pairs (i, i + hd/2); x' = x*c - y*s, y' = y*c + x*s
    (src/layer/rotary_embedding.cu:24-47)."""
    half = x.shape[-1] // 2
    index = torch.as_tensor(list(positions), dtype=torch.long)
    c = cos[index][:, None, :]
    s = sin[index][:, None, :]
    first, second = x[..., :half], x[..., half:]
    return torch.cat([first * c - second * s, second * c + first * s], dim=-1)


def plain_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int = 0) -> torch.Tensor:
    """Causal grouped-query attention over a whole sequence.  q [T, nh, hd], k and v [T, nkv, hd];
    query head j uses key/value head j // (nh / nkv); scale 1/sqrt(hd); a query at position t sees
    positions u <= t (and u > t - window with a window); softmax over the allowed keys
    (deps/ttl/src/kernels/attention/attention.cu:46-56,76-77,90-166; src/model/causal_lm/qwen3.cpp:35-37)."""
    T, nh, hd = q.shape
    nkv = k.shape[1]
    group = nh // nkv
    scale = 1.0 / math.sqrt(hd)
    out = torch.zeros_like(q)
    for head in range(nh):
        kv_head = head // group
        scores = (q[:, head, :] @ k[:, kv_head, :].T) * scale           # [T, T]
        t = torch.arange(T)[:, None]
        u = torch.arange(T)[None, :]
        allowed = u <= t
        if window > 0:
            allowed = allowed & (u > t - window)
        scores = scores.masked_fill(~allowed, float("-inf"))
        out[:, head, :] = torch.softmax(scores, dim=-1) @ v[:, kv_head, :]
    return out


def plain_self_attention(x: torch.Tensor, weights: dict, prefix: str, config: dict, layer: int, cos, sin) -> torch.Tensor:
    """Projections without bias, per-head RMSNorm of q and k with the layer eps before the rotation,
    attention, output projection (src/model/causal_lm/qwen3.cpp:39-69)."""
    T = x.shape[0]
    nh, nkv, hd = int(config["num_attention_heads"]), int(config["num_key_value_heads"]), head_dim_of(config)
    eps = float(config["rms_norm_eps"])
    q = (x @ weights[f"{prefix}.q_proj.weight"].T).view(T, nh, hd)
    k = (x @ weights[f"{prefix}.k_proj.weight"].T).view(T, nkv, hd)
    v = (x @ weights[f"{prefix}.v_proj.weight"].T).view(T, nkv, hd)
    q = plain_rmsnorm(q, weights[f"{prefix}.q_norm.weight"], eps)
    k = plain_rmsnorm(k, weights[f"{prefix}.k_norm.weight"], eps)
    positions = range(T)
    q = plain_rope(q, positions, cos, sin)
    k = plain_rope(k, positions, cos, sin)
    attended = plain_attention(q, k, v, layer_window(config, layer)).reshape(T, nh * hd)
    return attended @ weights[f"{prefix}.o_proj.weight"].T


def plain_silu(z: torch.Tensor) -> torch.Tensor:
    """silu(z) = z / (1 + exp(-z)) (src/layer/activation.cu:31-33)."""
    return z / (1.0 + torch.exp(-z))


def plain_mlp(x: torch.Tensor, weights: dict, prefix: str) -> torch.Tensor:
    """down(silu(gate(x)) * up(x)), no biases (src/layer/mlp.cpp:29-36)."""
    gate = x @ weights[f"{prefix}.gate_proj.weight"].T
    up = x @ weights[f"{prefix}.up_proj.weight"].T
    return (plain_silu(gate) * up) @ weights[f"{prefix}.down_proj.weight"].T


def plain_decoder_layer(x: torch.Tensor, weights: dict, config: dict, layer: int, cos, sin) -> torch.Tensor:
    """r = x + attn(norm(x)); x' = r + mlp(norm(r)) (src/model/causal_lm/qwen3.cpp:79-88)."""
    prefix = f"model.layers.{layer}"
    eps = float(config["rms_norm_eps"])
    attended = plain_self_attention(plain_rmsnorm(x, weights[f"{prefix}.input_layernorm.weight"], eps), weights,
                                    f"{prefix}.self_attn", config, layer, cos, sin)
    residual = x + attended
    return residual + plain_mlp(plain_rmsnorm(residual, weights[f"{prefix}.post_attention_layernorm.weight"], eps),
                                weights, f"{prefix}.mlp")


def plain_forward(config: dict, weights: dict, token_ids) -> torch.Tensor:
    """Logits [T, vocab] of a whole sequence: embedding, the layers, final norm, and the head, which
    is the embedding table when tie_word_embeddings is set (src/model/causal_lm/qwen3.cpp:152-181,134-136)."""
    hd = head_dim_of(config)
    cos, sin = plain_rope_tables(hd, len(token_ids), float(config.get("rope_theta", 1000000.0)))
    x = plain_embedding(weights["model.embed_tokens.weight"], token_ids)
    for layer in range(int(config["num_hidden_layers"])):
        x = plain_decoder_layer(x, weights, config, layer, cos, sin)
    x = plain_rmsnorm(x, weights["model.norm.weight"], float(config["rms_norm_eps"]))
    head = weights["model.embed_tokens.weight"] if config.get("tie_word_embeddings", False) else weights["lm_head.weight"]
    return x @ head.T


# ---------------------------------------------------------------------- sampling
def plain_argmax(logits: torch.Tensor) -> int:
    """The lowest index among equal maxima (deps/ttl/include reduction_operations.cuh:108-131)."""
    best = 0
    for index in range(1, logits.numel()):
        if logits[index] > logits[best]:
            best = index
    return best


def plain_sample(logits: torch.Tensor, temperature: float, uniform: float) -> tuple[int, float]:
    """p = softmax((x - max) / T); inclusive prefix sums in index order; the first index whose prefix
    sum exceeds u * total (src/sampler/sampler.cu:82-83,150-167).  Returns the index and how far
    u * total lies from the nearer edge of that index's interval, relative to the total (a small
    margin means float32 prefix sums may fairly pick a neighbour)."""
    z = (logits.to(F64) - logits.to(F64).max()) / temperature
    p = torch.exp(z)
    cdf = torch.cumsum(p, dim=0)
    total = cdf[-1]
    target = uniform * total
    index = int(torch.searchsorted(cdf, target, right=True))
    index = min(index, logits.numel() - 1)
    low = cdf[index - 1] if index > 0 else torch.tensor(0.0, dtype=F64)
    margin = float(torch.minimum(target - low, cdf[index] - target) / total)
    return index, margin


def plain_greedy_generate(config: dict, weights: dict, prompt, max_new_tokens: int) -> list[int]:
    """Greedy decoding by recomputing the whole sequence for every token."""
    tokens = list(prompt)
    for _ in range(max_new_tokens):
        tokens.append(plain_argmax(plain_forward(config, weights, tokens)[-1]))
    return tokens[len(prompt):]
