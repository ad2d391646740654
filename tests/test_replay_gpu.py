"""The engine against the plain implementation under every way of cutting the work, in 32-bit and
in bfloat16, on three tiny configurations: each request alone and whole; most of it in one step and
the last 32 tokens one by one; portions of changing size down to two tokens; and mixed, up to four
live requests with so few pages that they are used again (pages given back are filled with NaN, so a
kernel that reads a page it should not shows up as a non-finite logit)."""

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from replay_util import (collect, first_mismatch, peak_tokens, random_tokens, run_in_process, trace_mixed,
                         trace_portions, trace_tail, trace_whole)
from tiny_configs import TINY

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [70, 128, 45, 33, 100, 5, 17, 64], "B": [1, 9, 33, 70, 150, 256, 41, 96],
           "C": [60, 130, 250, 40, 90, 33, 17, 200]}
TRACES = {"whole": trace_whole, "tail": trace_tail, "portions": trace_portions, "mixed": trace_mixed}


def make_requests(name: str) -> dict[str, list[int]]:
    vocab = TINY[name]["config"]["vocab_size"]
    return {f"r{i}": random_tokens(vocab, n, seed=1000 * ord(name) + i) for i, n in enumerate(LENGTHS[name])}


@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_replay_matches_plain(model_folders, cuda_device, name, dtype, mode):
    folder = model_folders(name, dtype)
    requests = make_requests(name)
    steps = TRACES[mode](requests)
    outputs = run_in_process(folder, dtype, steps, TINY[name]["page_size"])
    rows = collect(steps, outputs)
    assert len(rows) >= sum(1 for _ in requests)
    first, worst, where = first_mismatch(rows, requests, folder, dtype)
    assert first is None, (f"{name} {dtype} {mode}: first wrong logits at request {first[0]} position {first[1]}: "
                           f"error {first[2]:.3e} > {first[3]:.1e}; worst {worst:.3e} at {where}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cuttings_agree_with_each_other(model_folders, cuda_device, dtype):
    """The same (request, position) gives the same logits however the tokens were cut, beyond rounding."""
    name = "B"
    folder = model_folders(name, dtype)
    requests = make_requests(name)
    results = {}
    for mode, build in TRACES.items():
        steps = build(requests)
        results[mode] = collect(steps, run_in_process(folder, dtype, steps, TINY[name]["page_size"]))
    tol = 2e-4 if dtype == "float32" else 0.04
    for key, row in results["whole"].items():
        for mode in ("portions", "mixed"):
            assert np.abs(results[mode][key] - row).max() <= tol, (mode, key)
    for key, row in results["tail"].items():
        assert np.abs(results["whole"][key] - row).max() <= tol, ("tail", key)


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
    for name, dtype in (("B", "float32"), ("B", "bfloat16"), ("C", "bfloat16")):
        folder = model_folders(name, dtype)
        tokens = random_tokens(TINY[name]["config"]["vocab_size"], 230, seed=77)
        requests = {"long": tokens}
        steps = trace_tail(requests, tail=200)
        rows = collect(steps, run_in_process(folder, dtype, steps, TINY[name]["page_size"]))
        first, worst, where = first_mismatch(rows, requests, folder, dtype)
        assert first is None, f"{name} {dtype}: {first}; worst {worst:.3e} at {where}"


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


def test_decode_chains_whole_partial_and_off(model_folders, cuda_device, monkeypatch):
    """Decode steps of a few tokens run as fused chains of a layer's products.  A product the chain
    kernel refuses (its input too long for shared memory, on a large model) runs as kernels of its
    own between two chains: here the down projections are refused by hand.  Whole chains, partial
    chains and no chains all agree with the plain implementation, and so does the decode attention
    that does the position encoding and the cache write itself (the engine uses it for large batches)."""
    from zephyr_b200.engine.replay import TraceReplayer
    from zephyr_b200.kernels import ops

    for name in ("B", "C"):
        folder = model_folders(name, "bfloat16")
        config = TINY[name]["config"]
        requests = {f"r{i}": random_tokens(config["vocab_size"], 30 + 5 * i, seed=900 + i) for i in range(3)}
        steps = trace_mixed(requests, seed=11, tail=20)
        for mode in ("whole", "partial", "off", "one kernel"):
            with monkeypatch.context() as patch:
                refused = []
                if mode == "partial":
                    real = ops.fused_chain_stage_supported

                    def picky(tokens, w, normed_input, swiglu):
                        if tuple(w.shape) == (config["hidden_size"], config["intermediate_size"]):      # a down projection
                            refused.append(tokens)
                            return False
                        return real(tokens, w, normed_input, swiglu)
                    patch.setattr(ops, "fused_chain_stage_supported", picky)
                replayer = TraceReplayer(folder, "bfloat16", peak_tokens(steps), page_size=TINY[name]["page_size"], max_requests=4)
                chains = replayer.runner.model.chains
                assert chains is not None and chains.supports(3)
                replayer.runner.model.use_chains = mode != "off"
                if mode == "one kernel":        # position encoding inside the decode attention, whatever the batch
                    for block in replayer.runner.model.layers:
                        block.mixer.fuse_decode_rows = 1
                outputs = {s["step"]: replayer.step(s) for s in steps}
                assert (mode == "partial") == bool(refused)
            rows = collect(steps, {k: v for k, v in outputs.items() if v is not None})
            first, worst, where = first_mismatch(rows, requests, folder, "bfloat16")
            assert first is None, f"{name} {mode}: {first}; worst {worst:.3e} at {where}"
