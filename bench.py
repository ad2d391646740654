"""Decode and prefill throughput of the engine on one B200, with the fraction of the roofline.

    python bench.py [--steps K] [--warmup W] [--gpus 1] [--impl ours|reference]
                    [--shape 0.6b|8b|32b] [--batch 8] [--context 4096] [--layers L]

One JSON line on standard output.  A "step" is one decode step of ``--batch`` sequences whose
contexts end at ``--context`` tokens.  ``value`` is decoded tokens a second timed on the device;
``e2e`` is the same through the Python entry point (``Engine.add_request`` / ``Engine.step``), with
the step's inputs copied from pinned host memory and the sampled tokens read back every step.
Weights are seeded random values of the named shape; token ids are seeded uniform random numbers.
Every decode step reads all weights and the whole cache of the live requests, several GB, far more
than the 126 MB L2, so no L2 flush is needed between timed steps (``config.l2`` says so).
"""

from __future__ import annotations

import argparse
import json
import os
import random
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SHAPES = {      # the layer sizes of the Qwen3 family members the benchmark names
    "0.6b": dict(num_hidden_layers=28, hidden_size=1024, num_attention_heads=16, num_key_value_heads=8, head_dim=128,
                 intermediate_size=3072, vocab_size=151936, tie_word_embeddings=True),
    "8b": dict(num_hidden_layers=36, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
               intermediate_size=12288, vocab_size=151936, tie_word_embeddings=False),
    "32b": dict(num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, num_key_value_heads=8, head_dim=128,
                intermediate_size=25600, vocab_size=151936, tie_word_embeddings=False),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def metric_name(args) -> str:
    """One string for both arms: the driver divides their values only if the strings are equal."""
    return f"decode tok/s @ batch {args.batch}, context {args.context} (Qwen3-{args.shape.upper()} shape)"


def kernel_fractions(config, batch: int, context: int, peak: dict) -> tuple[dict, dict]:
    """The step's dominant kernels alone, timed with CUDA events over rotating operands larger than L2
    (``zephyr_b200.kernels.timing``): achieved bytes/s over the copy rate for the decode kernels,
    FLOP/s over the library's burst rate for the prompt kernels.  A layer's share of the decode step
    is its products (one fused chain) and its attention; the head comes once."""
    from types import SimpleNamespace

    from zephyr_b200.kernels import timing

    base = dict(warmup=3, iters=20, heads=config.num_attention_heads, kv_heads=config.num_key_value_heads,
                head_dim=config.head_dim, page_size=PAGE_SIZE, window=0, split=0, hidden=config.hidden_size,
                ffn=config.intermediate_size)
    chain = timing.fused_chain(SimpleNamespace(rows=batch, **base))
    attention = timing.decode_attention(SimpleNamespace(batch=batch, context=context, **base))
    head = timing.gemm_small(SimpleNamespace(rows=batch, n=config.vocab_size, k=config.hidden_size, swiglu=False,
                                             float_out=True, **base))
    hbm, tflops = peak["hbm_gbs"], peak["bf16_tflops"]
    decode = {"layer_products": {"us": chain["us"], "frac": round(chain["gbs"] / hbm, 3)},
              "decode_attention": {"us": attention["us"], "frac": round(attention["gbs"] / hbm, 3)},
              "lm_head": {"us": head["us"], "frac": round(head["gbs"] / hbm, 3)}}
    prompt_attention = timing.prefill_attention(SimpleNamespace(tokens=PREFILL_TOKENS, **base))
    prompt_products = timing.products(SimpleNamespace(tokens=PREFILL_TOKENS, **base))
    prefill = {"attention": {"us": prompt_attention["us"], "frac": round(prompt_attention["tflops"] / tflops, 3)},
               "layer_products": {"us": prompt_products["us"], "frac": round(prompt_products["tflops"] / tflops, 3)}}
    return decode, prefill
PREFILL_TOKENS = 2048
PAGE_SIZE = 16


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            data = json.loads(path.read_text())
            if "hbm_gbs" in data and "bf16_tflops" in data:
                return data, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons every 200 ms while a timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.process = None

    def start(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.process = None

    def stop(self) -> dict:
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.process.terminate()
        try:
            out, _ = self.process.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
            out, _ = self.process.communicate()
        clocks, maxima, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                clocks.append(float(parts[0]))
                maxima.append(float(parts[1]))
            except ValueError:
                continue
            for name, value in zip(names, parts[3:7]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None,
                "sm_max_mhz": max(maxima) if maxima else None, "reasons": sorted(reasons), "samples": len(clocks)}


def build_engine(shape: str, layers: int | None, batch: int, context: int, dtype: str = "bfloat16",
                 prefill_together: int = 1):
    import torch

    from zephyr_b200 import Engine, Qwen3Config
    from zephyr_b200.engine import KvCacheOptions, PagedSchedulerConfig
    from zephyr_b200.parts import expected_weights
    from zephyr_b200.weights import RandomWeights

    sizes = dict(SHAPES[shape])
    full_layers = sizes["num_hidden_layers"]
    if layers:
        sizes["num_hidden_layers"] = layers
    config = Qwen3Config(max_position_embeddings=max(context, 4096), rms_norm_eps=1e-6, rope_theta=1000000.0, **sizes)
    spec = config.to_model_spec()
    store = RandomWeights(expected_weights(spec), seed=0, dtype=getattr(torch, dtype), device="cuda")
    # The pool is sized by the engine from the memory that is left after the weights and a profiled
    # step; it never holds more than ``batch`` sequences of the model's length need.
    engine = Engine(None, dtype=dtype, model_config=config, weights=store, max_seq_len=context,
                    kv_cache=KvCacheOptions(block_size=PAGE_SIZE),
                    # The token budget lets `prefill_together` whole prompts share one step, so that the
                    # sequences of the end-to-end run start decoding together and the batch stays whole.
                    scheduler=PagedSchedulerConfig(max_num_seqs=batch,
                                                   max_num_batched_tokens=max(PREFILL_TOKENS, batch,
                                                                              prefill_together * context),
                                                   max_prefill_chunk_tokens=max(PREFILL_TOKENS, context)))
    needed = batch * -(-context // PAGE_SIZE)
    if engine.runner.manager.groups[0].pool.num_usable < needed:
        raise SystemExit(f"bench.py: the cache pool got {engine.runner.manager.groups[0].pool.num_usable} pages, "
                         f"{needed} are needed for batch {batch} at context {context}")
    return engine, config, full_layers


def model_flops_per_token(config) -> float:
    """Matrix-product FLOPs per token of the layers (the head runs on the wanted rows only)."""
    h, i = config.hidden_size, config.intermediate_size
    qkv = (config.num_attention_heads + 2 * config.num_key_value_heads) * config.head_dim
    per_layer = 2 * (qkv * h + config.num_attention_heads * config.head_dim * h + 2 * i * h + i * h)
    return per_layer * config.num_hidden_layers


def prefill_flops(config, tokens: int) -> float:
    attention = config.num_hidden_layers * config.num_attention_heads * 2.0 * tokens * tokens * config.head_dim
    return model_flops_per_token(config) * tokens + attention + 2.0 * config.vocab_size * config.hidden_size


def device_decode(engine, batch: int, context: int, warmup: int, steps: int, sampler_clock: ClockSampler | None):
    """Device-timed decode: ``steps`` steps of ``batch`` sequences whose contexts end at ``context``."""
    import torch

    from zephyr_b200.engine import StepEntry
    from zephyr_b200.kernels import ops
    from zephyr_b200.sampling import SamplingParams

    runner, vocab = engine.runner, engine.vocab_size
    rng = random.Random(1234)
    start = context - (warmup + steps)
    ids = [("bench", i) for i in range(batch)]
    for rid in ids:
        assert runner.add_request(rid)
        done = 0
        while done < start:
            count = min(PREFILL_TOKENS, start - done)
            runner.step([StepEntry(rid, [rng.randrange(vocab) for _ in range(count)], ())])
            done += count
    runner.check()
    greedy = [SamplingParams(temperature=0.0)] * batch

    def one_step():
        logits = runner.step([StepEntry(rid, [rng.randrange(vocab)], (0,)) for rid in ids])
        return engine.sampler.sample_async(logits, greedy, [None] * batch)

    if sampler_clock:
        sampler_clock.start()        # nvidia-smi takes a moment to start: the warm-up gives it that
    for _ in range(warmup):
        one_step()
    torch.cuda.synchronize()
    launches_before = ops.LAUNCHES
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(steps):
        one_step()
    end.record()
    torch.cuda.synchronize()
    clocks = sampler_clock.stop() if sampler_clock else None
    launches = ops.LAUNCHES - launches_before
    runner.check()
    ms = begin.elapsed_time(end) / steps
    for rid in ids:
        runner.free_request(rid)
    return ms, launches, clocks


def e2e_decode(engine, batch: int, context: int, warmup: int, steps: int):
    """The same through the entry point: every step copies its inputs from pinned host memory and
    reads the sampled tokens back."""
    import torch

    from zephyr_b200 import GenerationParams

    rng = random.Random(4321)
    start = context - (warmup + steps) - 1
    params = GenerationParams(max_tokens=warmup + steps + 1, temperature=0.0, ignore_eos=True)
    requests = [engine.add_request([rng.randrange(engine.vocab_size) for _ in range(start)], params)
                for _ in range(batch)]
    while any(engine.sequences[(r, 0)].state.value != "decode" for r in requests):
        engine.step()
    assert len({len(engine.sequences[(r, 0)].token_ids) for r in requests}) == 1, "the batch must decode in step"
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    # Bytes per step: the packed int32 step description up (taken from the last warm-up step; it
    # grows by a page id per sequence every 16 steps), the sampled ids and two status words down.
    h2d = engine.runner.last_step_h2d_bytes + 8 * 0
    d2h = 4 * batch + 2 * 16
    began = time.perf_counter()
    for _ in range(steps):
        engine.step()
    torch.cuda.synchronize()
    seconds = time.perf_counter() - began
    for r in requests:
        engine.cancel(r)
        engine.take_output(r)
    return batch * steps / seconds, h2d, d2h


def device_prefill(engine, tokens: int, warmup: int, reps: int):
    import torch

    from zephyr_b200.engine import StepEntry

    runner, vocab = engine.runner, engine.vocab_size
    rng = random.Random(99)
    times = []
    for rep in range(warmup + reps):
        rid = ("prefill", rep)
        assert runner.add_request(rid)
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        entry = [StepEntry(rid, [rng.randrange(vocab) for _ in range(tokens)], (tokens - 1,))]
        torch.cuda.synchronize()
        begin.record()
        runner.step(entry)
        end.record()
        torch.cuda.synchronize()
        if rep >= warmup:
            times.append(begin.elapsed_time(end))
        runner.free_request(rid)
    runner.check()
    return statistics.median(times)


def run_ours(args) -> dict:
    import torch

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device")
    peak, peak_source = peaks()
    engine, config, full_layers = build_engine(args.shape, args.layers, max(args.batch, 64) if args.points else args.batch,
                                               args.context, prefill_together=args.batch)
    runner = engine.runner
    clock = ClockSampler()
    ms, launches, clocks = device_decode(engine, args.batch, args.context, args.warmup, args.steps, clock)
    value = args.batch * 1000.0 / ms
    weight_bytes = engine.model.weight_bytes_read_per_step()
    cache_bytes = args.batch * (args.context - args.steps / 2.0) * runner.cache_bytes_per_token()
    achieved = (weight_bytes + cache_bytes) / (ms * 1e-3) / 1e9
    e2e_value, h2d, d2h = e2e_decode(engine, args.batch, args.context, args.warmup, args.steps)
    prefill_ms = device_prefill(engine, PREFILL_TOKENS, 3, 5)
    flops = prefill_flops(config, PREFILL_TOKENS)
    points = {}
    if args.points:
        for batch in (1, 64):
            p_ms, _, _ = device_decode(engine, batch, args.context, 3, max(8, args.steps // 2), None)
            points[f"decode_b{batch}"] = round(batch * 1000.0 / p_ms, 1)
    decode_kernels, prefill_kernels = kernel_fractions(config, args.batch, args.context, peak)
    result = {
        "metric": metric_name(args),
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (seeded random weights and token ids)", "impl": "ours",
        "config": {
            "model": f"Qwen3-{args.shape.upper()} shape", "global_batch": args.batch, "seq_len": args.context,
            "parallelism": "single GPU", "layers": config.num_hidden_layers, "layers_full": full_layers,
            "hidden_size": config.hidden_size, "heads": config.num_attention_heads,
            "kv_heads": config.num_key_value_heads, "head_dim": config.head_dim,
            "intermediate_size": config.intermediate_size, "vocab_size": config.vocab_size,
            "tied_head": config.tie_word_embeddings, "kv_page_size": PAGE_SIZE, "prefill_tokens": PREFILL_TOKENS,
            "l2": "inputs (weights + cache, GBs per step) larger than L2; no flush",
            "peaks": f"{peak_source}: copy rate for decode, burst bf16 product rate for prefill",
            "cache_pages": runner.manager.groups[0].pool.num_usable,
        },
        "e2e": {"value": round(e2e_value, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "clocks": clocks,
        "prefill": {"value": round(PREFILL_TOKENS * 1000.0 / prefill_ms, 1), "tokens": PREFILL_TOKENS,
                    "ms": round(prefill_ms, 3),
                    "frac": round(flops / (prefill_ms * 1e-3) / (peak["bf16_tflops"] * 1e12), 4),
                    "kernels": prefill_kernels},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peak["hbm_gbs"], 4), "kernels": decode_kernels},
        "points": points,
    }
    return result


def run_reference(args) -> dict:
    """The unmodified reference, installed under baseline/_ref, through its own public Python API
    (``zephyr._C.Engine``: ``submit`` / ``wait_for_outputs``) on the same shape: seeded random weights
    written to a model folder, seeded random prompts (fresh ids for every run, so that its prefix
    cache cannot help).  Decode throughput is counted over the token increments it publishes, from
    the moment every sequence has produced its first token to the end of the run."""
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "zephyr").is_dir():
        return {"impl": "reference", "unavailable": "baseline/_ref holds no installed reference (zephyr) package"}
    import tempfile

    import torch

    if not torch.cuda.is_available():
        return {"impl": "reference", "unavailable": "no CUDA device"}
    sys.path.insert(0, str(ref))
    try:
        from zephyr import _C
    except Exception as error:      # the reference's own import chain (tokenizer front end, native module)
        return {"impl": "reference", "unavailable": f"cannot import the installed reference: {type(error).__name__}: {error}"[:300]}

    from zephyr_b200 import Qwen3Config, write_random_model

    sizes = dict(SHAPES[args.shape])
    full_layers = sizes["num_hidden_layers"]
    if args.layers:
        sizes["num_hidden_layers"] = args.layers
    config = Qwen3Config(max_position_embeddings=max(args.context, 4096), rms_norm_eps=1e-6, rope_theta=1000000.0, **sizes)
    rng = random.Random(77)
    steps, batch = args.steps, args.batch
    start = args.context - steps - 1
    with tempfile.TemporaryDirectory() as folder:
        write_random_model(config, 0, folder, dtype=torch.bfloat16)
        try:
            options = _C.EngineOptions(folder, devices=[0], dtype="bfloat16", max_seq_len=args.context,
                                       scheduler=_C.PagedSchedulerConfig(max_num_seqs=batch,
                                                                         max_num_batched_tokens=PREFILL_TOKENS,
                                                                         max_prefill_chunk_tokens=PREFILL_TOKENS),
                                       eos_token_ids=[])
        except Exception as error:
            return {"impl": "reference", "unavailable": f"the reference engine did not start: {type(error).__name__}: {error}"[:300]}

        native = _C.Engine(options, kv_cache=_C.KvCacheOptions(block_size=PAGE_SIZE))

        def run(new_tokens: int, count: int, length: int):
            """Submit ``count`` requests and follow the token increments as they come out.  Returns
            (seconds in all, seconds from the moment every sequence has its first token to the end,
            tokens produced in that second stretch)."""
            requests = [_C.GenerationRequest([rng.randrange(config.vocab_size) for _ in range(length)],
                                             sampling=_C.SamplingParams(temperature=0.0), max_new_tokens=new_tokens,
                                             ignore_eos=True) for _ in range(count)]
            torch.cuda.synchronize()
            began = time.perf_counter()
            produced = {native.submit(request): 0 for request in requests}
            finished, all_started, tokens_at_start = 0, None, 0
            while finished < count:
                for output in native.wait_for_outputs():
                    produced[output.request_id] += sum(len(choice.tokens) for choice in output.result)
                    if output.status is not None:
                        if output.status != _C.RequestStatus.COMPLETED:
                            raise RuntimeError(f"request ended with {output.status}: {output.error_message}")
                        finished += 1
                if all_started is None and all(n >= 1 for n in produced.values()):
                    all_started, tokens_at_start = time.perf_counter(), sum(produced.values())
            ended = time.perf_counter()
            assert all(n == new_tokens for n in produced.values())
            return ended - began, ended - (all_started or ended), sum(produced.values()) - tokens_at_start

        clock = ClockSampler()
        try:
            run(2, batch, start)
            clock.start()
            _, decode_seconds, decode_tokens = run(steps + 1, batch, start)
            clocks = clock.stop()
            prefill_runs = [run(1, 1, PREFILL_TOKENS)[0] for _ in range(3)]
        except Exception as error:
            clock.stop()
            return {"impl": "reference", "unavailable": f"the reference failed while generating: {type(error).__name__}: {error}"[:300]}
        finally:
            native.close()
    value = decode_tokens / max(decode_seconds, 1e-9)
    steps_timed = max(decode_tokens / batch, 1e-9)
    prefill_ms = statistics.median(prefill_runs[1:]) * 1e3
    return {
        "metric": metric_name(args), "value": round(value, 1),
        "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": args.warmup,
        "ms_per_step": round(decode_seconds / steps_timed * 1e3, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded random weights and token ids)",
        "impl": "reference",
        "config": {"model": f"Qwen3-{args.shape.upper()} shape", "global_batch": batch, "seq_len": args.context,
                   "parallelism": "single GPU", "layers": config.num_hidden_layers, "layers_full": full_layers,
                   "kv_page_size": PAGE_SIZE, "prefill_tokens": PREFILL_TOKENS,
                   "timing": "wall clock over _C.Engine token increments, from every sequence's first token to the end"},
        "e2e": {"value": round(value, 1), "unit": "tok/s", "h2d_bytes_per_step": None, "d2h_bytes_per_step": None},
        "clocks": clocks,
        "prefill": {"value": round(PREFILL_TOKENS * 1e3 / prefill_ms, 1), "tokens": PREFILL_TOKENS, "ms": round(prefill_ms, 3)},
    }


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--shape", choices=sorted(SHAPES), default="0.6b")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=4096)
    parser.add_argument("--layers", type=int, default=None, help="fewer layers than the shape has (both are reported)")
    parser.add_argument("--no-points", dest="points", action="store_false", help="skip decode at batch 1 and 64")
    parser.add_argument("--own-products", action="store_true",
                        help="with --only: no product on the vendor library (all on this package's tcgen05 kernel)")
    parser.add_argument("--only", choices=("prefill", "decode"), default=None,
                        help="time only the 2048-token prefill, or only the decode step, and print a short line "
                             "(the program a profiler is pointed at)")
    args = parser.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not measured")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.only is not None and args.impl == "ours":
        if args.own_products:
            from zephyr_b200.kernels import ops
            ops.USE_LIBRARY_PRODUCTS = False
        engine, config, _ = build_engine(args.shape, args.layers, args.batch, args.context, prefill_together=1)
        if args.only == "prefill":
            ms = device_prefill(engine, PREFILL_TOKENS, 3, args.steps)
            print(json.dumps({"only": "prefill", "tokens": PREFILL_TOKENS, "layers": config.num_hidden_layers, "ms": round(ms, 4)}))
        else:
            ms, launches, _ = device_decode(engine, args.batch, args.context, args.warmup, args.steps, None)
            print(json.dumps({"only": "decode", "batch": args.batch, "layers": config.num_hidden_layers, "ms_per_step": round(ms, 4),
                              "gpu_launches": launches}))
        return 0
    result = run_reference(args) if args.impl == "reference" else run_ours(args)
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
