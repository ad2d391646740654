"""Each part of a layer alone against the plain function of the same part: norm, position encoding,
feed-forward, attention mixer (whole sequence, and cut in two steps), and the block arrangement."""

import pytest
import torch

from plain_qwen3 import (F64, load_model_folder, plain_decoder_layer, plain_mlp, plain_rmsnorm, plain_rope,
                         plain_rope_tables, plain_self_attention)
from replay_util import random_tokens
from tiny_configs import TINY, tiny_config

pytestmark = pytest.mark.gpu


def tol(dtype):
    return 2e-5 if dtype == "float32" else 2e-2


def load(model_folders, name, dtype, device):
    from zephyr_b200.config import load_model_spec
    from zephyr_b200.engine import ModelRunner
    from zephyr_b200.parts import Model
    from zephyr_b200.weights import Checkpoint

    folder = model_folders(name, dtype)
    model = Model.load(load_model_spec(folder), Checkpoint(folder), getattr(torch, dtype), device)
    runner = ModelRunner(model, TINY[name]["page_size"], 64, 4)
    config, weights = load_model_folder(folder)
    return model, runner, config, weights


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_norm_feed_forward_and_position(model_folders, cuda_device, name, dtype):
    from zephyr_b200.kernels import ops

    model, runner, config, weights = load(model_folders, name, dtype, cuda_device)
    block = model.layers[1]
    g = torch.Generator().manual_seed(0)
    x = torch.randn(13, config["hidden_size"], generator=g).to(model.dtype).to(cuda_device)
    x64 = x.double().cpu()
    eps = config["rms_norm_eps"]

    got = block.mixer_norm.forward(x)
    assert (got.double().cpu() - plain_rmsnorm(x64, weights["model.layers.1.input_layernorm.weight"], eps)).abs().max() \
        <= tol(dtype) * 4

    got = block.feed_forward.forward(x)
    expected = plain_mlp(x64, weights, "model.layers.1.mlp")
    assert (got.double().cpu() - expected).abs().max() <= tol(dtype) * max(1.0, float(expected.abs().max()))
    # As many rows as a long prompt portion brings (in bfloat16 the first product then runs on the
    # tcgen05 kernel with the activation in its epilogue, at widths that end inside its tiles).
    many = torch.randn(700, config["hidden_size"], generator=g).to(model.dtype).to(cuda_device)
    before = ops.LAUNCH_COUNTS.get("gemm_tc", 0)
    got = block.feed_forward.forward(many)
    assert dtype == "float32" or ops.LAUNCH_COUNTS.get("gemm_tc", 0) == before + 1
    expected = plain_mlp(many.double().cpu(), weights, "model.layers.1.mlp")
    assert (got.double().cpu() - expected).abs().max() <= tol(dtype) * max(1.0, float(expected.abs().max()))

    position = block.mixer.position
    nh, hd = config["num_attention_heads"], block.mixer.hd
    q = torch.randn(13, nh * hd, generator=g).to(model.dtype).to(cuda_device)
    positions = torch.tensor([0, 1, 2, 3, 50, 51, 99, 100, 101, 7, 7, 127, 64], dtype=torch.int32, device=cuda_device)
    q64 = q.double().cpu().view(13, nh, hd)
    status = ops.new_status(cuda_device)
    rotated = position.apply(q.clone(), nh, positions, status)
    ops.check_status(status)
    cos, sin = plain_rope_tables(hd, 128, config["rope_theta"])
    expected = plain_rope(q64, positions.tolist(), cos, sin)
    assert (rotated.double().cpu().view(13, nh, hd) - expected).abs().max() <= tol(dtype) * 4
    # The device tables are the float32 values of the plain tables.
    assert (position.cos.double().cpu()[:128] - cos).abs().max() <= 1e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_attention_mixer_and_block(model_folders, cuda_device, name, dtype):
    from zephyr_b200.config import LayerCall
    from zephyr_b200.engine import StepEntry
    from zephyr_b200.parts import ResidualStream

    model, runner, config, weights = load(model_folders, name, dtype, cuda_device)
    layer = 1
    block = model.layers[layer]
    call = LayerCall(layer, layer)
    T = 45
    g = torch.Generator().manual_seed(1)
    x = torch.randn(T, config["hidden_size"], generator=g).to(model.dtype).to(cuda_device)
    x64 = x.double().cpu()
    hd = block.mixer.hd
    cos, sin = plain_rope_tables(hd, T, config["rope_theta"])
    expected = plain_self_attention(x64, weights, f"model.layers.{layer}.self_attn", config, layer, cos, sin)
    tokens = random_tokens(config["vocab_size"], T, seed=2)

    # Whole sequence in one step.
    assert runner.add_request("whole")
    ctx = runner.build_context([StepEntry("whole", tokens)])
    got = block.mixer.forward(x, ctx, call)
    runner.check()
    scale = max(1.0, float(expected.abs().max()))
    assert (got.double().cpu() - expected).abs().max() <= tol(dtype) * scale

    # The same cut in two: 29 tokens, then 15 single tokens... then the last one; the cache carries over.
    assert runner.add_request("cut")
    ctx = runner.build_context([StepEntry("cut", tokens[:29])])
    first = block.mixer.forward(x[:29].contiguous(), ctx, call)
    runner.manager.commit("cut", 29)
    pieces = [first]
    for t in range(29, T):
        ctx = runner.build_context([StepEntry("cut", tokens[t:t + 1])])
        pieces.append(block.mixer.forward(x[t:t + 1].contiguous(), ctx, call))
        runner.manager.commit("cut", t + 1)
    runner.check()
    assert (torch.cat(pieces).double().cpu() - expected).abs().max() <= tol(dtype) * scale

    # The block: r = x + attn(norm(x)); x' = r + mlp(norm(r)).
    assert runner.add_request("block")
    ctx = runner.build_context([StepEntry("block", tokens)])
    stream = block.forward(ResidualStream(x.clone()), ctx, call)
    runner.check()
    after = stream.flush()
    expected = plain_decoder_layer(x64, weights, config, layer, cos, sin)
    assert (after.double().cpu() - expected).abs().max() <= tol(dtype) * max(1.0, float(expected.abs().max())) * 2


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_weight_bytes_of_a_step(model_folders, cuda_device, name):
    """What the roofline divides by: every matrix and scale a step reads, once (a fused q/k/v matrix
    and the view of its query rows are one piece of memory; a tied head is the embedding table)."""
    model, _, _, _ = load(model_folders, name, "bfloat16", cuda_device)
    c = TINY[name]["config"]
    h, i, v, layers = c["hidden_size"], c["intermediate_size"], c["vocab_size"], c["num_hidden_layers"]
    hd = c.get("head_dim") or h // c["num_attention_heads"]
    q, kv = c["num_attention_heads"] * hd, c["num_key_value_heads"] * hd
    matrices = 2 * (layers * ((q + 2 * kv) * h + h * q + 3 * i * h) + v * h)      # the head, or the table that serves as it
    scales = layers * (2 * h + 2 * hd) + h                                        # two or four bytes each, as stored
    assert matrices + 2 * scales <= model.weight_bytes_read_per_step() <= matrices + 4 * scales
