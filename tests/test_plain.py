"""The plain implementation checked against itself from other angles: each part against a
second, even plainer formulation, and the whole model against properties any causal decoder has."""

import cmath
import math

import pytest
import torch

from plain_qwen3 import (F64, load_model_folder, plain_argmax, plain_attention, plain_forward, plain_greedy_generate,
                         plain_mlp, plain_rmsnorm, plain_rope, plain_rope_tables, plain_sample, plain_silu)
from tiny_configs import TINY, tiny_config
from zephyr_b200.weights import write_random_model


def test_rmsnorm():
    x = torch.tensor([[3.0, 4.0]], dtype=F64)
    w = torch.tensor([2.0, 0.5], dtype=F64)
    rms = math.sqrt((9 + 16) / 2 + 1e-6)
    assert torch.allclose(plain_rmsnorm(x, w, 1e-6), torch.tensor([[3 / rms * 2, 4 / rms * 0.5]], dtype=F64))


def test_rope_is_a_rotation_of_the_pairs_by_position_times_frequency():
    hd, theta = 8, 10000.0
    cos, sin = plain_rope_tables(hd, 50, theta)
    x = torch.randn(3, 2, hd, dtype=F64, generator=torch.Generator().manual_seed(0))
    positions = [0, 7, 49]
    out = plain_rope(x, positions, cos, sin)
    assert torch.equal(out[0], x[0])                                   # position 0: no rotation
    for t, p in enumerate(positions):
        for i in range(hd // 2):
            angle = p / theta ** (2 * i / hd)
            z = complex(x[t, 1, i], x[t, 1, i + hd // 2]) * cmath.exp(1j * angle)
            assert abs(out[t, 1, i] - z.real) < 1e-4 and abs(out[t, 1, i + hd // 2] - z.imag) < 1e-4
    assert torch.allclose(out.norm(dim=-1), x.norm(dim=-1))           # a rotation keeps lengths
    # The scores depend on the distance only.
    q = plain_rope(x[:1].expand(2, -1, -1).clone(), [5, 30], cos, sin)
    k = plain_rope(x[1:2].expand(2, -1, -1).clone(), [2, 27], cos, sin)
    assert abs(float((q[0, 0] * k[0, 0]).sum() - (q[1, 0] * k[1, 0]).sum())) < 1e-5


def naive_attention(q, k, v, window):
    T, nh, hd = q.shape
    g = nh // k.shape[1]
    out = torch.zeros_like(q)
    for t in range(T):
        for h in range(nh):
            lo = max(0, t - window + 1) if window else 0
            weights = [math.exp(float(q[t, h] @ k[u, h // g]) / math.sqrt(hd)) for u in range(lo, t + 1)]
            total = sum(weights)
            for j, u in enumerate(range(lo, t + 1)):
                out[t, h] += weights[j] / total * v[u, h // g]
    return out


@pytest.mark.parametrize("window", [0, 3, 1])
def test_attention_against_a_naive_loop(window):
    g = torch.Generator().manual_seed(1)
    q, k, v = torch.randn(9, 6, 8, dtype=F64, generator=g), torch.randn(9, 3, 8, dtype=F64, generator=g), \
        torch.randn(9, 3, 8, dtype=F64, generator=g)
    assert torch.allclose(plain_attention(q, k, v, window), naive_attention(q, k, v, window), atol=1e-12)
    if window == 1:     # a window of one sees only itself
        assert torch.allclose(plain_attention(q, k, v, 1), v.repeat_interleave(2, dim=1))


def test_silu_and_mlp():
    z = torch.tensor([-2.0, 0.0, 3.0], dtype=F64)
    assert torch.allclose(plain_silu(z), z * torch.sigmoid(z))
    weights = {"m.gate_proj.weight": torch.eye(2, dtype=F64), "m.up_proj.weight": 2 * torch.eye(2, dtype=F64),
               "m.down_proj.weight": torch.tensor([[1.0, 1.0]], dtype=F64)}
    x = torch.tensor([[1.0, -1.0]], dtype=F64)
    expected = (plain_silu(x) * 2 * x).sum(-1, keepdim=True)
    assert torch.allclose(plain_mlp(x, weights, "m"), expected)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_model_properties(name, tmp_path):
    folder = write_random_model(tiny_config(name), TINY[name]["seed"], tmp_path)
    config, weights = load_model_folder(folder)
    vocab = config["vocab_size"]
    tokens = [(5 * i + 2) % vocab for i in range(40)]
    logits = plain_forward(config, weights, tokens)
    assert logits.shape == (40, vocab) and torch.isfinite(logits).all()
    # Causality: a prefix gives the same logits.
    assert torch.allclose(plain_forward(config, weights, tokens[:17]), logits[:17], atol=1e-10)
    # Changing a later token changes nothing before it, and something after it.
    changed = list(tokens)
    changed[20] = (changed[20] + 1) % vocab
    other = plain_forward(config, weights, changed)
    assert torch.allclose(other[:20], logits[:20], atol=1e-10) and not torch.allclose(other[20:], logits[20:])
    if name == "C":     # windows: layers 1 and 2 see 24 positions, layer 0 sees all
        assert config["layer_windows"] == [0, 24, 24]
        full = plain_forward({k: v for k, v in config.items() if k != "layer_windows"}, weights, tokens)
        assert torch.allclose(full[:24], logits[:24], atol=1e-10) and not torch.allclose(full[24:], logits[24:])
    generated = plain_greedy_generate(config, weights, tokens[:5], 3)
    assert len(generated) == 3 and generated[0] == int(plain_forward(config, weights, tokens[:5])[-1].argmax())


def test_selection():
    assert plain_argmax(torch.tensor([1.0, 3.0, 3.0, 2.0])) == 1        # the lowest index among equals
    logits = torch.log(torch.tensor([0.1, 0.2, 0.3, 0.4]))
    assert [plain_sample(logits, 1.0, u)[0] for u in (0.0, 0.09, 0.11, 0.31, 0.59, 0.61, 0.999)] == [0, 0, 1, 2, 2, 3, 3]
    assert plain_sample(logits, 0.01, 0.5)[0] == 3                       # a low temperature sharpens
