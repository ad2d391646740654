"""The engine against the plain implementation under every way of cutting the work, in 32-bit and
in bfloat16: each request alone and whole; most of it in one step and the last 32 tokens one by one;
portions of changing size down to two tokens; mixed, up to four live requests with so few pages that
they are used again (pages given back are filled with NaN, so a kernel that reads a page it should
not shows up as a non-finite logit); and the tails of several requests decoded together.  The
configurations are the tiny ones (A, B), the windowed test architecture (C, W), and D, E, F, which
have the head size and layer widths of the benchmarked models and so run the kernels those run."""

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from replay_util import (collect, first_mismatch, peak_tokens, random_tokens, run_in_process, trace_batched_tail,
                         trace_mixed, trace_portions, trace_tail, trace_whole)
from tiny_configs import TINY

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [70, 128, 45, 33, 100, 5, 17, 64], "B": [1, 9, 33, 70, 150, 256, 41, 96],
           "C": [60, 130, 250, 40, 90, 33, 17, 200], "W": [60, 130, 250, 40, 300, 33, 17, 200],
           "D": [300, 600, 129, 257, 64, 40, 513, 17], "E": [200, 520, 64, 129, 300, 33], "F": [300, 40, 130, 70]}
TRACES = {"whole": trace_whole, "tail": trace_tail, "portions": trace_portions, "mixed": trace_mixed,
          "batched": trace_batched_tail}
NAMES = ["A", "B", "C", "W", "D", "E", "F"]


def make_requests(name: str) -> dict[str, list[int]]:
    vocab = TINY[name]["config"]["vocab_size"]
    return {f"r{i}": random_tokens(vocab, n, seed=1000 * ord(name) + i) for i, n in enumerate(LENGTHS[name])}


@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed", "batched"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", NAMES)
def test_replay_matches_plain(model_folders, cuda_device, name, dtype, mode):
    folder = model_folders(name, dtype)
    requests = make_requests(name)
    steps = TRACES[mode](requests)
    outputs = run_in_process(folder, dtype, steps, TINY[name]["page_size"])
    rows = collect(steps, outputs)
    assert len(rows) >= sum(1 for _ in requests)
    first, worst, where = first_mismatch(rows, requests, folder, dtype, f"{name} {mode}")
    assert first is None, (f"{name} {dtype} {mode}: first wrong logits at request {first[0]} position {first[1]}: "
                           f"error {first[2]:.3e} > {first[3]:.1e}; worst {worst:.3e} at {where}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "D", "E"])
def test_cuttings_agree_with_each_other(model_folders, cuda_device, name, dtype):
    """The same (request, position) gives the same logits however the tokens were cut, beyond rounding
    (twice the bound of one run against the plain implementation)."""
    from replay_util import tolerance

    folder = model_folders(name, dtype)
    requests = make_requests(name)
    results = {}
    for mode, build in TRACES.items():
        steps = build(requests)
        results[mode] = collect(steps, run_in_process(folder, dtype, steps, TINY[name]["page_size"]))
    for key, row in results["whole"].items():
        for mode in ("portions", "mixed"):
            assert np.abs(results[mode][key] - row).max() <= 2 * tolerance(dtype, row), (mode, key)
    for mode in ("tail", "batched"):
        for key, row in results[mode].items():
            assert np.abs(results["whole"][key] - row).max() <= 2 * tolerance(dtype, row), (mode, key)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(model_folders, cuda_device, tmp_path, dtype):
    """bin/trace_run itself: a mixed trace through the program, files and ``done`` lines checked."""
    name = "A"
    folder = model_folders(name, dtype)
    requests = make_requests(name)
    steps = trace_mixed(requests, seed=3)
    root = Path(__file__).resolve().parent.parent
    out = tmp_path / "out"
    command = [sys.executable, str(root / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype, "--out",
               str(out), "--max-tokens", str(peak_tokens(steps)), "--page-size", str(TINY[name]["page_size"])]
    feed = "".join(json.dumps(step) + "\n" for step in steps)
    done = subprocess.run(command, input=feed, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    assert [line for line in done.stdout.splitlines() if line.startswith("done ")] == \
        [f"done {step['step']}" for step in steps]
    vocab = TINY[name]["config"]["vocab_size"]
    outputs = {}
    for step in steps:
        wanted = sum(len(e["want"]) for e in step["entries"])
        path = out / f"{step['step']}.f32"
        assert path.exists() == (wanted > 0)
        if wanted:
            outputs[step["step"]] = np.fromfile(path, dtype="<f4").reshape(wanted, vocab)
    first, worst, where = first_mismatch(collect(steps, outputs), requests, folder, dtype)
    assert first is None, f"trace_run {dtype}: {first}; worst {worst:.3e} at {where}"


def test_long_decoding(model_folders, cuda_device):
    """A short prompt, then 200 tokens one by one, across many page edges."""
    for name, dtype in (("B", "float32"), ("B", "bfloat16"), ("C", "bfloat16"), ("W", "bfloat16"), ("D", "bfloat16")):
        folder = model_folders(name, dtype)
        tokens = random_tokens(TINY[name]["config"]["vocab_size"], 230, seed=77)
        requests = {"long": tokens}
        steps = trace_tail(requests, tail=200)
        rows = collect(steps, run_in_process(folder, dtype, steps, TINY[name]["page_size"]))
        first, worst, where = first_mismatch(rows, requests, folder, dtype)
        assert first is None, f"{name} {dtype}: {first}; worst {worst:.3e} at {where}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_contexts_as_long_as_the_benchmarks(model_folders, cuda_device, dtype):
    """A prompt of 4100 tokens in portions of 2048, 1500 and 552, then 24 tokens one by one (the decode
    graph's bound goes from 4096 to the model's limit), beside a second request of 2300 tokens that
    decodes along: the prompt kernels' long rows of tiles, the decode kernel's items over hundreds of
    pages, and logits of positions beyond 4096."""
    name = "L"
    folder = model_folders(name, dtype)
    vocab = TINY[name]["config"]["vocab_size"]
    requests = {"long": random_tokens(vocab, 4124, seed=41), "other": random_tokens(vocab, 2324, seed=42)}
    steps, fed = [], {"long": 0, "other": 0}

    def feed(items, end=()):
        entries = []
        for rid, count, want in items:
            entries.append({"id": rid, "tokens": requests[rid][fed[rid]:fed[rid] + count], "want": want})
            fed[rid] += count
        steps.append({"step": len(steps), "entries": entries, "end": list(end)})

    feed([("long", 2048, [0, 2047])])
    feed([("long", 1500, [1499]), ("other", 2300, [2299])])
    feed([("long", 552, [0, 551])])
    for turn in range(24):
        feed([("long", 1, [0]), ("other", 1, [0])], end=("long", "other") if turn == 23 else ())
    rows = collect(steps, run_in_process(folder, dtype, steps, TINY[name]["page_size"]))
    assert ("long", 4123) in rows and ("other", 2323) in rows
    first, worst, where = first_mismatch(rows, requests, folder, dtype, f"{name} long contexts")
    assert first is None, f"{dtype}: {first}; worst {worst:.3e} at {where}"


@pytest.mark.parametrize("name", ["D", "E", "F"])
def test_a_step_of_more_than_a_thousand_rows(model_folders, cuda_device, name):
    """Four prompts of 270 to 300 tokens in ONE step (1140 rows: the feed-forward's first product runs on
    the tcgen05 kernel with the activation in its epilogue, through several tiles per CTA), then six
    decoded tokens each, against the plain implementation."""
    dtype = "bfloat16"
    folder = model_folders(name, dtype)
    vocab = TINY[name]["config"]["vocab_size"]
    lengths = {"a": 300, "b": 270, "c": 290, "d": 280}
    requests = {rid: random_tokens(vocab, n + 6, seed=50 + n) for rid, n in lengths.items()}
    steps = [{"step": 0, "end": [], "entries": [
        {"id": rid, "tokens": requests[rid][:n], "want": [0, n // 2, n - 1]} for rid, n in lengths.items()]}]
    for turn in range(6):
        steps.append({"step": turn + 1, "end": list(lengths) if turn == 5 else [], "entries": [
            {"id": rid, "tokens": [requests[rid][n + turn]], "want": [0]} for rid, n in lengths.items()]})
    from zephyr_b200.kernels import ops
    before = ops.LAUNCH_COUNTS.get("gemm_tc", 0)
    rows = collect(steps, run_in_process(folder, dtype, steps, TINY[name]["page_size"]))
    assert ops.LAUNCH_COUNTS.get("gemm_tc", 0) > before              # the kernel this test is about did run
    first, worst, where = first_mismatch(rows, requests, folder, dtype, f"{name} 1140 rows")
    assert first is None, f"{first}; worst {worst:.3e} at {where}"


@pytest.mark.parametrize("name", ["B", "D", "E"])
def test_without_the_vendor_library(model_folders, cuda_device, monkeypatch, name):
    """With ``ops.USE_LIBRARY_PRODUCTS`` off no product of the step goes to the vendor library: every
    bfloat16 product of more than a few rows runs on this package's tcgen05 kernel (the projections,
    the feed-forward, the head's logits of many wanted rows), and the logits still are the plain
    implementation's, whole prompts, portions and mixed steps alike."""
    import torch

    from zephyr_b200.kernels import ops
    dtype = "bfloat16"
    folder = model_folders(name, dtype)
    requests = make_requests(name)
    monkeypatch.setattr(ops, "USE_LIBRARY_PRODUCTS", False)

    def no_library(*args, **kwargs):
        raise AssertionError("a product went to the vendor library")
    monkeypatch.setattr(torch, "mm", no_library)
    before = ops.LAUNCH_COUNTS.get("gemm_tc", 0)
    for mode in ("whole", "portions", "mixed"):
        steps = TRACES[mode](requests)
        rows = collect(steps, run_in_process(folder, dtype, steps, TINY[name]["page_size"]))
        first, worst, where = first_mismatch(rows, requests, folder, dtype, f"{name} {mode}, own products")
        assert first is None, f"{mode}: {first}; worst {worst:.3e} at {where}"
    assert ops.LAUNCH_COUNTS.get("gemm_tc", 0) > before


@pytest.mark.parametrize("seed", [1, 7])
def test_random_configurations(cuda_device, tmp_path, seed):
    """Configurations drawn at random (head sizes in steps of 16 up to 256, any head and group counts,
    widths that are no multiple of 8, odd vocabularies, any page size), each replayed mixed, with a
    batched tail and in portions, in both types, against the plain implementation."""
    import random

    import torch

    from zephyr_b200.config import Qwen3Config
    from zephyr_b200.weights import write_random_model

    rng = random.Random(seed)
    for case in range(4):
        hd = rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 144, 256])
        nkv = rng.choice([1, 2, 3, 4])
        nh = nkv * (rng.choice([1, 2, 3, 4, 7]) if hd <= 128 else rng.choice([1, 2]))
        vocab, page = rng.choice([97, 130, 257, 1003]), rng.choice([4, 8, 16, 32])
        config = Qwen3Config(
            vocab_size=vocab, hidden_size=rng.choice([40, 72, 100, 136, 264, 96]),
            intermediate_size=rng.choice([56, 100, 136, 250, 328]), num_hidden_layers=rng.choice([1, 2, 3]),
            num_attention_heads=nh, num_key_value_heads=nkv, head_dim=hd, max_position_embeddings=320,
            rms_norm_eps=rng.choice([1e-6, 1e-5, 3e-6]), rope_theta=rng.choice([1e4, 1e6, 5e5]),
            tie_word_embeddings=rng.random() < 0.5)
        requests = {f"r{i}": random_tokens(vocab, n, seed=100 * case + i) for i, n in enumerate((45, 120, 33, 200, 70))}
        for dtype in ("bfloat16", "float32"):
            folder = write_random_model(config, case, tmp_path / f"{seed}_{case}_{dtype}", dtype=getattr(torch, dtype))
            for mode in ("mixed", "batched", "portions"):
                steps = TRACES[mode](requests)
                rows = collect(steps, run_in_process(folder, dtype, steps, page))
                first, worst, where = first_mismatch(rows, requests, folder, dtype, f"random {seed}.{case} {mode}")
                assert first is None, f"{config} page {page} {dtype} {mode}: {first}; worst {worst:.3e} at {where}"


def test_first_tokens(model_folders, cuda_device):
    """The first tokens of a sequence, one at a time from the very start (position 0 has one key)."""
    for name in ("A", "B", "C"):
        for dtype in ("float32", "bfloat16"):
            folder = model_folders(name, dtype)
            tokens = random_tokens(TINY[name]["config"]["vocab_size"], 6, seed=5)
            requests = {"s": tokens}
            steps = [{"step": i, "entries": [{"id": "s", "tokens": [t], "want": [0]}], "end": []}
                     for i, t in enumerate(tokens)]
            rows = collect(steps, run_in_process(folder, dtype, steps, TINY[name]["page_size"]))
            first, worst, where = first_mismatch(rows, requests, folder, dtype)
            assert first is None, f"{name} {dtype}: {first}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_repeated_step_shapes_replay_a_graph(model_folders, cuda_device, dtype):
    """Steps of one shape (a portion of 9 tokens beside a portion of 5 and a single token) come five
    times, with other requests, tokens, contexts and pages each time: the first runs launch by launch,
    the second is captured, the others replay the graph.  All agree with the plain implementation, and
    with a runner that never uses graphs bit for bit."""
    from zephyr_b200.engine.replay import TraceReplayer

    name = "B"
    folder = model_folders(name, dtype)
    vocab = TINY[name]["config"]["vocab_size"]
    requests = {f"r{i}": random_tokens(vocab, 40 + 7 * i, seed=300 + i) for i in range(3)}
    fed = {rid: 0 for rid in requests}
    steps = []
    # A first step that gives every request a different context, then the repeated shape.
    for rid, count in zip(requests, (3, 11, 6)):
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": requests[rid][:count], "want": [count - 1]}],
                      "end": []})
        fed[rid] = count
    order = list(requests)
    for turn in range(5):
        a, b, c = order[turn % 3], order[(turn + 1) % 3], order[(turn + 2) % 3]
        entries = []
        for rid, count, want in ((a, 9, [0, 8]), (b, 5, [4]), (c, 1, [0])):
            entries.append({"id": rid, "tokens": requests[rid][fed[rid]:fed[rid] + count], "want": want})
            fed[rid] += count
        steps.append({"step": len(steps), "entries": entries, "end": []})
    outputs = {}
    for graphs in (True, False):
        replayer = TraceReplayer(folder, dtype, peak_tokens(steps), page_size=TINY[name]["page_size"], max_requests=4)
        replayer.runner.use_cuda_graphs = graphs
        outputs[graphs] = {s["step"]: replayer.step(s) for s in steps}
        if graphs:
            shaped = [k for k in replayer.runner._graphs if not isinstance(k[0], int)]
            assert len(shaped) == 1 and replayer.runner._graphs[shaped[0]]["graph"] is not None
    for step in steps:
        assert np.array_equal(outputs[True][step["step"]], outputs[False][step["step"]]), f"step {step['step']}"
    rows = collect(steps, outputs[True])
    first, worst, where = first_mismatch(rows, {r: t[:fed[r]] for r, t in requests.items()}, folder, dtype)
    assert first is None, f"{dtype}: {first}; worst {worst:.3e} at {where}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prepared_steps_and_tokens_from_the_device(model_folders, cuda_device, dtype):
    """A decode step described ahead of its tokens (``prepare``), and one whose tokens never visit
    the host (``device_tokens``: the argmax of the step before, still on the device), give the
    logits of steps described the ordinary way, bit for bit; a prepared step that no longer holds is
    refused when it is given tokens on the device and ignored otherwise."""
    import torch

    from zephyr_b200.config import InvalidArgumentError
    from zephyr_b200.engine import StepEntry
    from zephyr_b200.engine.replay import TraceReplayer
    from zephyr_b200.kernels import ops

    name = "C"
    folder = model_folders(name, dtype)
    vocab = TINY[name]["config"]["vocab_size"]
    prompts = {f"p{i}": random_tokens(vocab, 11 + 6 * i, seed=500 + i) for i in range(3)}

    def decode(mode: str):
        runner = TraceReplayer(folder, dtype, 256, page_size=TINY[name]["page_size"], max_requests=4).runner
        tokens = {}
        for rid, prompt in prompts.items():
            assert runner.add_request(rid)
            logits = runner.step([StepEntry(rid, prompt, (len(prompt) - 1,))])
            tokens[rid] = int(logits[0].argmax())
        rows, device_ids = [], None
        for step in range(8):
            entries = [StepEntry(rid, [tokens[rid]], (0,)) for rid in prompts]
            if mode == "plain" or step < 2:          # the graph is captured by the first decode step
                logits = runner.step(entries)
            elif mode == "prepared":
                placeholders = [StepEntry(rid, [-1], (0,)) for rid in prompts]
                prepared = runner.prepare(placeholders)
                assert prepared is not None and runner.holds(prepared, entries)
                logits = runner.step(entries, prepared)
            else:
                prepared = runner.prepare([StepEntry(rid, [-1], (0,)) for rid in prompts])
                assert prepared is not None
                logits = runner.step([StepEntry(rid, [-1], (0,)) for rid in prompts], prepared, device_tokens=device_ids)
            device_ids = ops.sample(logits, runner.status)          # int32 on the device, one per row
            rows.append(logits.clone())
            for rid, token in zip(prompts, device_ids.tolist()):
                tokens[rid] = token
        runner.check()
        return runner, torch.stack(rows)

    _, plain = decode("plain")
    for mode in ("prepared", "device"):
        runner, got = decode(mode)
        assert torch.equal(got, plain), mode
    # A prepared step goes stale when the runner moves on without it.
    stale = runner.prepare([StepEntry(rid, [-1], (0,)) for rid in prompts])
    fresh = [StepEntry(rid, [1], (0,)) for rid in prompts]
    runner.step(fresh)
    assert not runner.holds(stale, fresh)
    runner.step(fresh, stale)                                       # ignored: described afresh
    with pytest.raises(InvalidArgumentError, match="still holds"):
        runner.step(fresh, stale, device_tokens=torch.zeros(3, dtype=torch.int32, device=cuda_device))


CHAIN_LENGTHS = {"B": (30, 35, 40), "C": (30, 35, 40), "W": (60, 35, 90), "D": (200, 270, 140), "E": (100, 260, 70),
                 "F": (40, 80, 130)}


@pytest.mark.parametrize("name", ["B", "C", "W", "D", "E", "F"])
def test_decode_chains_whole_partial_and_off(model_folders, cuda_device, monkeypatch, name):
    """Decode steps of a few tokens run as fused chains of a layer's products.  A product the chain
    kernel refuses (its input too long for shared memory: the down projection of the 8B widths in F)
    runs as kernels of its own between two chains; on the other configurations the down projections
    are refused by hand.  Whole chains, partial chains and no chains all agree with the plain
    implementation, and so does the decode attention that does the position encoding and the cache
    write itself (the engine uses it for large batches).  The traces decode the tails of three
    requests together, and mix portions with single tokens."""
    from zephyr_b200.engine.replay import TraceReplayer
    from zephyr_b200.kernels import ops

    folder = model_folders(name, "bfloat16")
    config = TINY[name]["config"]
    requests = {f"r{i}": random_tokens(config["vocab_size"], n, seed=900 + i) for i, n in enumerate(CHAIN_LENGTHS[name])}
    down_shape = (config["hidden_size"], config["intermediate_size"])
    for build in (lambda r: trace_mixed(r, seed=11, tail=20), lambda r: trace_batched_tail(r, tail=24)):
        steps = build(requests)
        for mode in ("whole", "partial", "off", "one kernel"):
            with monkeypatch.context() as patch:
                refused = []
                real = ops.fused_chain_stage_supported

                def picky(tokens, w, normed_input, swiglu):
                    taken = real(tokens, w, normed_input, swiglu)
                    if tuple(w.shape) == down_shape and (mode == "partial" or not taken):
                        refused.append(tokens)
                        return False
                    return taken
                patch.setattr(ops, "fused_chain_stage_supported", picky)
                replayer = TraceReplayer(folder, "bfloat16", peak_tokens(steps), page_size=TINY[name]["page_size"], max_requests=4)
                replayer.runner.poison_freed_pages = True
                chains = replayer.runner.model.chains
                assert chains is not None and chains.supports(3)
                replayer.runner.model.use_chains = mode != "off"
                if mode == "one kernel":        # position encoding inside the decode attention, whatever the batch
                    for block in replayer.runner.model.layers:
                        block.mixer.fuse_decode_rows = 1
                outputs = {s["step"]: replayer.step(s) for s in steps}
                # F's down projection (K = 12288) does not fit beside the weight ring: refused for real.
                assert bool(refused) == (mode == "partial" or name == "F"), (mode, refused)
            rows = collect(steps, {k: v for k, v in outputs.items() if v is not None})
            first, worst, where = first_mismatch(rows, requests, folder, "bfloat16", f"{name} chains {mode}")
            assert first is None, f"{name} {mode}: {first}; worst {worst:.3e} at {where}"


@pytest.mark.parametrize("name", ["D", "E"])
def test_two_halves_of_a_decode_step_side_by_side(model_folders, cuda_device, name):
    """A decode step of many requests runs as two halves on two streams, each on half the SMs, with
    workspaces of their own (the model does that from 12 requests up; here from 2).  The tails of four
    requests decoded together, first as one batch, then in two lanes: both agree with the plain
    implementation, and the lanes were really used."""
    from zephyr_b200.kernels import ops

    folder = model_folders(name, "bfloat16")
    vocab = TINY[name]["config"]["vocab_size"]
    requests = {f"r{i}": random_tokens(vocab, n, seed=1300 + i) for i, n in enumerate((90, 140, 70, 200))}
    steps = trace_batched_tail(requests, tail=40)
    seen = []
    real = ops.lane

    def two_lanes(replayer):
        replayer.runner.model.lanes_min_rows = 2

        class counted(real):
            def __enter__(self):
                seen.append(self.index)
                return super().__enter__()
        ops.lane = counted

    try:
        for prepare in (None, two_lanes):
            rows = collect(steps, run_in_process(folder, "bfloat16", steps, TINY[name]["page_size"], prepare=prepare))
            first, worst, where = first_mismatch(rows, requests, folder, "bfloat16", f"{name} lanes {prepare is not None}")
            assert first is None, f"{name} lanes={prepare is not None}: {first}; worst {worst:.3e} at {where}"
    finally:
        ops.lane = real
    assert 0 in seen and 1 in seen


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["D", "E"])
def test_decoding_across_the_bounds_of_the_decode_graphs(model_folders, cuda_device, name, dtype):
    """Decode graphs are keyed by a power-of-two bound on the longest context (256, 512, 1024).  Two
    requests decode from below 256 to beyond it, a third joins, and all three go on past 512: every
    change of the bound captures a new graph with another split plan while the requests are live.
    Steps are described ahead (``prepare``) and get their tokens on the device (``device_tokens``)
    across the changes, as the engine runs them.  Every logit is compared with the plain model."""
    import torch

    from zephyr_b200.engine import StepEntry
    from zephyr_b200.engine.replay import TraceReplayer

    folder = model_folders(name, dtype)
    vocab = TINY[name]["config"]["vocab_size"]
    requests = {"a": random_tokens(vocab, 290, seed=1), "b": random_tokens(vocab, 300, seed=2),
                "c": random_tokens(vocab, 540, seed=3)}
    runner = TraceReplayer(folder, dtype, 1280, page_size=TINY[name]["page_size"], max_requests=4).runner
    runner.poison_freed_pages = True
    fed, rows = {}, {}

    def prefill(rid, count):
        assert runner.add_request(rid)
        logits = runner.step([StepEntry(rid, requests[rid][:count], (count - 1,))])
        rows[(rid, count - 1)] = logits[0].cpu().numpy()
        fed[rid] = count

    def decode(live, steps):
        bounds = set()
        for turn in range(steps):
            entries = [StepEntry(rid, [requests[rid][fed[rid]]], (0,)) for rid in live]
            key = runner._graph_key(entries)
            bounds.add(key[1])
            placeholders = [StepEntry(rid, [-1], (0,)) for rid in live]
            prepared = runner.prepare(placeholders)
            if prepared is not None and turn % 2 == 0:
                tokens = torch.tensor([requests[rid][fed[rid]] for rid in live], dtype=torch.int32, device=cuda_device)
                logits = runner.step(placeholders, prepared, device_tokens=tokens)
            else:
                logits = runner.step(entries, prepared)      # prepared may be None: a graph not captured yet
            got = logits.cpu().numpy()
            for index, rid in enumerate(live):
                rows[(rid, fed[rid])] = got[index].copy()
                fed[rid] += 1
            runner.check()
            runner.manager.check_invariants()
        return bounds

    prefill("a", 246)
    prefill("b", 250)
    assert decode(["a", "b"], 20) == {256, 512}                 # b passes 256 after six steps
    prefill("c", 500)
    assert decode(["a", "b", "c"], 24) == {512, 1024}           # c passes 512 after twelve
    decode_graphs = [k for k in runner._graphs if isinstance(k[0], int)]
    assert sorted(decode_graphs) == [(2, 256), (2, 512), (3, 512), (3, 1024)]
    first, worst, where = first_mismatch(rows, requests, folder, dtype, f"{name} graph bounds")
    assert first is None, f"{name} {dtype}: {first}; worst {worst:.3e} at {where}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_shape_graphs_are_evicted_and_captured_again(model_folders, cuda_device, dtype):
    """A step shape other than decode-only is captured when it comes a second time, and at most 16 such
    graphs are kept.  Eighteen shapes come twice each, so the first ones are evicted; then the first
    shape comes again, twice, and is captured again.  Every step agrees with the plain model."""
    from zephyr_b200.engine import StepEntry
    from zephyr_b200.engine.replay import TraceReplayer

    name = "D"
    folder = model_folders(name, dtype)
    tokens = random_tokens(TINY[name]["config"]["vocab_size"], 2 * sum(range(2, 20)) + 8, seed=9)
    requests = {"s": tokens}
    runner = TraceReplayer(folder, dtype, 512, page_size=TINY[name]["page_size"], max_requests=2).runner
    assert runner.add_request("s")
    rows, fed = {}, 0
    sizes = [n for n in range(2, 20) for _ in (0, 1)] + [2, 2, 2]
    captured_first = []
    for n in sizes:
        logits = runner.step([StepEntry("s", tokens[fed:fed + n], (0, n - 1))]).cpu().numpy()
        rows[("s", fed)], rows[("s", fed + n - 1)] = logits[0].copy(), logits[1].copy()
        fed += n
        shaped = [k for k in runner._graphs if not isinstance(k[0], int)]
        assert len(shaped) <= runner.MAX_SHAPE_GRAPHS
        captured_first.append(any(k[0] == ((2, (0, 1)),) for k in shaped))
    runner.check()
    assert captured_first[1] and not captured_first[35]         # captured at its second coming, evicted later
    assert not captured_first[36] and captured_first[37] and captured_first[38]     # counted again, captured again
    first, worst, where = first_mismatch(rows, {"s": tokens[:fed]}, folder, dtype, f"{name} eviction")
    assert first is None, f"{dtype}: {first}; worst {worst:.3e} at {where}"


def test_the_full_0_6b_shape_in_float32(cuda_device, tmp_path):
    """The check run of the benchmarked model: all 28 layers of the Qwen3-0.6B shape with its whole
    vocabulary in true 32-bit arithmetic, a prompt of 24 tokens in two portions and two decoded
    tokens, three rows of logits against the plain implementation."""
    import torch

    from plain_qwen3 import load_model_folder, plain_forward
    from zephyr_b200.config import Qwen3Config
    from zephyr_b200.weights import write_random_model

    config = Qwen3Config(vocab_size=151936, hidden_size=1024, intermediate_size=3072, num_hidden_layers=28,
                         num_attention_heads=16, num_key_value_heads=8, head_dim=128, max_position_embeddings=4096,
                         rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=True)
    folder = write_random_model(config, 7, tmp_path / "qwen3_0_6b_float32", dtype=torch.float32)
    tokens = random_tokens(config.vocab_size, 26, seed=6)
    steps = [{"step": 0, "entries": [{"id": "p", "tokens": tokens[:15], "want": [14]}], "end": []},
             {"step": 1, "entries": [{"id": "p", "tokens": tokens[15:24], "want": [8]}], "end": []},
             {"step": 2, "entries": [{"id": "p", "tokens": tokens[24:25], "want": []}], "end": []},
             {"step": 3, "entries": [{"id": "p", "tokens": tokens[25:26], "want": [0]}], "end": ["p"]}]
    rows = collect(steps, run_in_process(folder, "float32", steps, 16))
    assert sorted(rows) == [("p", 14), ("p", 23), ("p", 25)]
    plain_config, weights = load_model_folder(folder)
    expected = plain_forward(plain_config, weights, tokens).numpy()
    for (_, position), got in rows.items():
        error = float(np.abs(got.astype(np.float64) - expected[position]).max())
        bound = 1e-4 * max(1.0, float(np.abs(expected[position]).max()))
        print(f"[logits] 0.6B float32 position {position}: error {error:.3e}, bound {bound:.1e}")
        assert error <= bound, (position, error)
