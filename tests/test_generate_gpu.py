"""Generation through the Python entry point: greedy and temperature sampling against the plain
implementation, the benchmark description's two tiny workloads, preemption under a small pool, the
finish rules, and the command line."""

import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from plain_qwen3 import load_model_folder, plain_forward, plain_sample
from replay_util import random_tokens
from tiny_configs import TINY

pytestmark = pytest.mark.gpu


def make_engine(folder, name, dtype, **kwargs):
    from zephyr_b200 import Engine
    from zephyr_b200.engine import KvCacheOptions, PagedSchedulerConfig

    scheduler = PagedSchedulerConfig(**{k: kwargs.pop(k) for k in list(kwargs)
                                        if k in ("max_num_seqs", "max_num_batched_tokens", "max_prefill_chunk_tokens")})
    return Engine(folder, dtype=dtype, scheduler=scheduler,
                  kv_cache=KvCacheOptions(block_size=TINY[name]["page_size"], num_blocks=kwargs.pop("num_blocks", 64)),
                  **kwargs)


def plain_greedy_with_margins(config, weights, prompt, count):
    tokens, margins = list(prompt), []
    for _ in range(count):
        logits = plain_forward(config, weights, tokens)[-1]
        top = torch.topk(logits, 2).values
        margins.append(float(top[0] - top[1]))
        tokens.append(int(logits.argmax()))
    return tokens[len(prompt):], margins


def assert_greedy_agrees(got, expected, margins, tolerance):
    """Equal tokens, except that a first difference is forgiven where the plain logits' two best lie
    closer than the engine's error bound (after which the sequences may part)."""
    for index, (g, e) in enumerate(zip(got, expected)):
        if g != e:
            assert margins[index] <= tolerance, f"token {index}: {g} != {e} with margin {margins[index]:.3e}"
            return
    assert len(got) == len(expected)


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("C", "float32"), ("B", "bfloat16"),
                                        ("C", "bfloat16"), ("W", "bfloat16"), ("D", "float32"), ("D", "bfloat16"),
                                        ("E", "bfloat16")])
def test_greedy_generation_matches_plain(model_folders, cuda_device, name, dtype):
    folder = model_folders(name, dtype)
    config, weights = load_model_folder(folder)
    engine = make_engine(folder, name, dtype, max_num_seqs=4, max_num_batched_tokens=16, max_prefill_chunk_tokens=7)
    prompts = [random_tokens(config["vocab_size"], n, seed=n) for n in (5, 11, 17, 40)]
    outputs = engine.generate(prompts, max_tokens=8, temperature=0.0, ignore_eos=True)
    for prompt, output in zip(prompts, outputs):
        expected, margins = plain_greedy_with_margins(config, weights, prompt, 8)
        assert output.prompt_token_ids == tuple(prompt) and output.status.value == "completed"
        assert output.choices[0].finish_reason.value == "length" and output.usage.completion_tokens == 8
        # A first difference is forgiven where the plain logits' two best lie closer than twice the bound on
        # the engine's error (8 units in the last place of the row's largest logit in bfloat16).
        last = plain_forward(config, weights, prompt)[-1]
        bound = 1e-4 * max(1.0, float(last.abs().max())) if dtype == "float32" else 8 * 2.0 ** -8 * float(last.abs().max())
        assert_greedy_agrees(list(output.token_ids), expected, margins, 2 * bound)
    assert engine.runner.manager.num_requests == 0
    engine.runner.manager.check_invariants()


def test_workload_a_three_requests_greedy(model_folders, cuda_device):
    """Tiny A, prompts of 5/11/17 tokens, 8 greedy tokens each, page size 4 (float32)."""
    folder = model_folders("A", "float32")
    config, weights = load_model_folder(folder)
    prompts = [random_tokens(256, n, seed=10 + n) for n in (5, 11, 17)]
    engine = make_engine(folder, "A", "float32", max_num_seqs=8, max_num_batched_tokens=512,
                         max_prefill_chunk_tokens=512)
    together = [list(o.token_ids) for o in engine.generate(prompts, max_tokens=8, temperature=0.0, ignore_eos=True)]
    alone = [list(engine.generate(p, max_tokens=8, temperature=0.0, ignore_eos=True).token_ids) for p in prompts]
    assert together == alone
    for prompt, got in zip(prompts, together):
        expected, margins = plain_greedy_with_margins(config, weights, prompt, 8)
        assert_greedy_agrees(got, expected, margins, 2e-4)


def test_workload_b_four_requests_temperature(model_folders, cuda_device):
    """Tiny B, prompts of 1/9/33/70 tokens, prompt portions of 16, 12 tokens at temperature 0.7 from
    seeded generators (float32): the batch gives what each request gives alone, and every token is
    the one that the plain logits of its history and the request's own generator select."""
    from zephyr_b200.sampling import MT19937_64

    folder = model_folders("B", "float32")
    config, weights = load_model_folder(folder)
    prompts = [random_tokens(311, n, seed=20 + n) for n in (1, 9, 33, 70)]
    engine = make_engine(folder, "B", "float32", max_num_seqs=4, max_num_batched_tokens=64,
                         max_prefill_chunk_tokens=16)
    from zephyr_b200 import GenerationParams

    ids = [engine.add_request(p, GenerationParams(max_tokens=12, temperature=0.7, seed=100 + i, ignore_eos=True))
           for i, p in enumerate(prompts)]
    while engine.has_unfinished():
        engine.step()
    together = [list(engine.take_output(i).token_ids) for i in ids]
    alone = [list(engine.generate(p, max_tokens=12, temperature=0.7, seed=100 + i, ignore_eos=True).token_ids)
             for i, p in enumerate(prompts)]
    assert together == alone
    followed = 0
    for i, (prompt, got) in enumerate(zip(prompts, together)):
        generator = MT19937_64(100 + i)             # the request's own generator: one number per token
        history = list(prompt)
        for position, token in enumerate(got):
            index, margin = plain_sample(plain_forward(config, weights, history)[-1], 0.7, generator.next_uniform())
            if margin <= 1e-5:
                break           # the draw falls on an interval's edge: float32 prefix sums may fairly pick a neighbour
            assert token == index, f"request {i} token {position}: {token} != {index} (margin {margin:.2e})"
            history.append(token)
            followed += 1
    assert followed >= 40           # nearly all of the 48 tokens were checked


def test_filters_penalties_and_reports_match_the_plain_sampler(model_folders, cuda_device):
    """Tiny B (float32), four requests with different sampling settings in one batch: every token is
    the one that the plain model's logits, the plain sampler and the request's own generator give,
    and the reported log-probabilities are those of the adjusted, scaled logits."""
    import plain_sampler
    from zephyr_b200 import GenerationParams
    from zephyr_b200.sampling import MT19937_64

    folder = model_folders("B", "float32")
    config, weights = load_model_folder(folder)
    vocab = config["vocab_size"]
    prompts = [random_tokens(vocab, n, seed=50 + n) for n in (6, 13, 21, 4)]
    settings = [dict(temperature=0.9, top_k=12, top_logprobs=3),
                dict(temperature=0.7, top_p=0.85, min_p=0.01, frequency_penalty=0.5, presence_penalty=0.25),
                dict(temperature=0.0, repetition_penalty=1.8, logit_bias={5: 4.0, 9: float("-inf")}, top_logprobs=0),
                dict(temperature=1.1, min_p=0.05, repetition_penalty=1.3, top_logprobs=vocab)]
    engine = make_engine(folder, "B", "float32", max_num_seqs=4, max_num_batched_tokens=32, max_prefill_chunk_tokens=8)
    ids = [engine.add_request(p, GenerationParams(max_tokens=6, seed=7 + i, ignore_eos=True, **s))
           for i, (p, s) in enumerate(zip(prompts, settings))]
    while engine.has_unfinished():
        engine.step()
    outputs = [engine.take_output(i) for i in ids]
    compared = 0
    for i, (prompt, setting, output) in enumerate(zip(prompts, settings, outputs)):
        choice = output.choices[0]
        assert len(choice.token_ids) == 6
        assert (choice.logprobs is None) == ("top_logprobs" not in setting)
        generator = MT19937_64(7 + i)
        tokens = list(prompt)
        for step, got in enumerate(choice.token_ids):
            logits = plain_forward(config, weights, tokens)[-1].to(torch.float32)
            adjusted = plain_sampler.adjust(logits, tokens, len(prompt), setting.get("frequency_penalty", 0.0),
                                            setting.get("presence_penalty", 0.0), setting.get("repetition_penalty", 1.0),
                                            setting.get("logit_bias"))
            temperature = setting["temperature"]
            u = generator.next_uniform() if temperature >= 1e-7 else 0.0
            want, margin = plain_sampler.sample(adjusted, temperature, u, setting.get("top_k", -1),
                                                setting.get("top_p", 1.0), setting.get("min_p", 0.0))
            if temperature < 1e-7:
                top = torch.topk(adjusted, 2).values
                margin = float(top[0] - top[1])
            if margin <= 1e-4:
                break                                   # a near tie: the sequences may fairly part here
            assert got == want, (i, step, got, want, margin)
            compared += 1
            if choice.logprobs is not None:
                count = min(setting["top_logprobs"], vocab)
                chosen, best = plain_sampler.report(adjusted, temperature, got, count)
                report = choice.logprobs[step]
                assert abs(report.logprob - chosen) <= 1e-4 * max(1.0, abs(chosen))
                assert len(report.top_logprobs) == count
                for entry, (token, value) in zip(report.top_logprobs, best):
                    assert abs(entry.logprob - value) <= 1e-4 * max(1.0, abs(value))
                # Equal ranks may swap where two log-probabilities differ by less than the engine's error.
                assert sorted(e.token_id for e in report.top_logprobs) == sorted(t for t, _ in best) or count < vocab
            tokens.append(got)
    assert compared >= 20
    assert 9 not in outputs[2].choices[0].token_ids              # a bias of -inf bans the token


def test_top_k_one_is_greedy_and_seeds_repeat(model_folders, cuda_device):
    folder = model_folders("A", "bfloat16")
    engine = make_engine(folder, "A", "bfloat16", max_num_seqs=2, max_num_batched_tokens=16, max_prefill_chunk_tokens=16)
    prompt = random_tokens(256, 9, seed=3)
    greedy = engine.generate(prompt, max_tokens=10, temperature=0.0, ignore_eos=True).token_ids
    assert engine.generate(prompt, max_tokens=10, temperature=0.8, top_k=1, seed=1, ignore_eos=True).token_ids == greedy
    one = engine.generate(prompt, max_tokens=10, temperature=0.9, top_p=0.9, seed=5, ignore_eos=True).token_ids
    two = engine.generate(prompt, max_tokens=10, temperature=0.9, top_p=0.9, seed=5, ignore_eos=True).token_ids
    other = engine.generate(prompt, max_tokens=10, temperature=0.9, top_p=0.9, seed=6, ignore_eos=True).token_ids
    assert one == two and one != other


def test_small_pool_preempts_and_tokens_do_not_change(model_folders, cuda_device):
    folder = model_folders("A", "float32")
    prompts = [random_tokens(256, n, seed=30 + n) for n in (10, 9, 14)]
    roomy = make_engine(folder, "A", "float32", max_num_seqs=3, max_num_batched_tokens=16, max_prefill_chunk_tokens=16)
    expected = [list(o.token_ids) for o in roomy.generate(prompts, max_tokens=20, temperature=0.0, ignore_eos=True)]
    tight = make_engine(folder, "A", "float32", max_num_seqs=3, max_num_batched_tokens=16, max_prefill_chunk_tokens=16,
                        num_blocks=16)          # 64 tokens for three sequences that grow to 30, 29 and 34
    tight.runner.poison_freed_pages = True
    got = [list(o.token_ids) for o in tight.generate(prompts, max_tokens=20, temperature=0.0, ignore_eos=True)]
    assert tight.stats.preemptions > 0
    assert got == expected
    tight.runner.manager.check_invariants()
    assert tight.runner.manager.num_free_pages() == 16


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_planning_a_step_ahead_changes_nothing(model_folders, cuda_device, dtype):
    """While the device runs a step of decoders the engine plans the next one.  Sequences that end on a
    stop token in the middle, requests that arrive while others decode, a cancelled request and a
    pool so small that it preempts: the tokens are those of an engine that plans nothing ahead, and
    plans made ahead (and steps launched ahead, with their tokens still on the device) were both used
    and dropped."""
    folder = model_folders("B", dtype)
    vocab = TINY["B"]["config"]["vocab_size"]
    prompts = [random_tokens(vocab, n, seed=70 + n) for n in (9, 17, 5, 12, 7)]

    def run(look_ahead: bool, num_blocks: int, launch_ahead: bool = False):
        engine = make_engine(folder, "B", dtype, max_num_seqs=4, max_num_batched_tokens=32, max_prefill_chunk_tokens=32,
                             num_blocks=num_blocks)
        engine.look_ahead = look_ahead
        engine.launch_ahead = launch_ahead
        used = dropped = 0
        take, settle = engine._take_ahead, engine._settle_flight

        def counting_flights():
            nonlocal used, dropped
            had = engine._flight
            flight = settle()
            if had is not None:
                whole = flight is not None and len(flight.plan.sequences) == len(had.plan.sequences)
                used += whole
                dropped += not whole
            return flight
        engine._settle_flight = counting_flights

        def counting():
            nonlocal used, dropped
            had = engine._ahead
            plan, prepared = take()
            if had is not None:
                used += plan is had[0]
                dropped += plan is not had[0]
            return plan, prepared
        engine._take_ahead = counting
        from zephyr_b200 import GenerationParams
        free = list(engine.generate(prompts[0], max_tokens=24, temperature=0.0, ignore_eos=True).token_ids)
        params = [GenerationParams(max_tokens=24, temperature=0.0, ignore_eos=True, stop_token_ids=(free[7],)),
                  GenerationParams(max_tokens=30, temperature=0.9, seed=5, ignore_eos=True),
                  GenerationParams(max_tokens=11, temperature=0.0, ignore_eos=True),
                  GenerationParams(max_tokens=40, temperature=0.0, ignore_eos=True),
                  GenerationParams(max_tokens=9, temperature=0.7, seed=2, top_k=5, ignore_eos=True)]
        ids = [engine.add_request(prompts[i], params[i]) for i in range(3)]
        steps = 0
        while engine.has_unfinished():
            engine.step()
            steps += 1
            if steps == 6:
                ids.append(engine.add_request(prompts[3], params[3]))      # arrives while the others decode
            if steps == 14:
                ids.append(engine.add_request(prompts[4], params[4]))
            if steps == 20:
                engine.cancel(ids[3])
            engine.runner.manager.check_invariants()
        outputs = [engine.take_output(i) for i in ids]
        return [list(o.token_ids) for o in outputs], used, dropped, engine.stats.preemptions

    expected, used, dropped, _ = run(False, 64)
    assert used == 0 and dropped == 0
    got, used, dropped, _ = run(True, 64)
    assert got[:3] == expected[:3] and got[4] == expected[4]
    assert got[3] == expected[3]                     # cancelled at the same step in both
    assert used >= 10 and dropped >= 2, (used, dropped)
    # The same with the next step launched before this step's tokens have reached the host.
    got, used, dropped, _ = run(True, 64, launch_ahead=True)
    # A request that arrives while a step is under way joins one step later, so the one that is
    # cancelled at a fixed step has one token fewer by then; what it has is the same.
    assert got[:3] == expected[:3] and got[4] == expected[4]
    assert 0 < len(got[3]) <= len(expected[3]) and got[3] == expected[3][:len(got[3])]
    assert used >= 10 and dropped >= 2, (used, dropped)
    tight_launched, _, _, preempted_launched = run(True, 10, launch_ahead=True)
    assert preempted_launched > 0 and tight_launched[:3] == expected[:3] and tight_launched[4] == expected[4]
    tight_expected, _, _, preempted_without = run(False, 10)
    tight, used, dropped, preempted = run(True, 10)
    assert preempted > 0 and preempted_without > 0
    assert tight[:3] == tight_expected[:3] == expected[:3] and tight[4] == expected[4]


def test_finish_rules_and_choices(model_folders, cuda_device):
    folder = model_folders("A", "float32")
    engine = make_engine(folder, "A", "float32", max_num_seqs=4, max_num_batched_tokens=32, max_prefill_chunk_tokens=32)
    prompt = random_tokens(256, 6, seed=1)
    free = list(engine.generate(prompt, max_tokens=6, temperature=0.0, ignore_eos=True).token_ids)
    # EOS: the terminating token is part of the output (src/engine/generation.cpp:81-99).
    eos_engine = make_engine(folder, "A", "float32", max_num_seqs=4, max_num_batched_tokens=32,
                             max_prefill_chunk_tokens=32, eos_token_ids=[free[2]])
    stopped = eos_engine.generate(prompt, max_tokens=6, temperature=0.0)
    first = free.index(free[2])
    assert list(stopped.token_ids) == free[:first + 1] and stopped.choices[0].finish_reason.value == "eos"
    assert list(eos_engine.generate(prompt, max_tokens=6, temperature=0.0, ignore_eos=True).token_ids) == free
    stop = engine.generate(prompt, max_tokens=6, temperature=0.0, stop_token_ids=[free[1]], ignore_eos=True)
    assert stop.choices[0].finish_reason.value == "stop_token" and stop.choices[0].stop_reason == free[1]
    assert list(stop.token_ids) == free[:free.index(free[1]) + 1]
    # The model's length: a prompt of 126 in a context of 128 can hold two more tokens' keys.
    long_prompt = random_tokens(256, 126, seed=2)
    out = engine.generate(long_prompt, temperature=0.0, ignore_eos=True)
    assert out.choices[0].finish_reason.value in ("length", "model_length") and len(out.token_ids) == 2
    with pytest.raises(ValueError, match="between 1 and"):
        engine.generate(random_tokens(256, 129, seed=3), max_tokens=1)
    with pytest.raises(ValueError, match="outside the model vocabulary"):
        engine.generate([1, 256], max_tokens=1)
    with pytest.raises(ValueError, match="token ids"):
        engine.generate("some text", max_tokens=1)
    # Two choices: seeds seed and seed + 1 (src/engine/engine.cpp:350-351).
    pair = engine.generate(prompt, max_tokens=5, temperature=1.0, seed=7, n=2, ignore_eos=True)
    one = engine.generate(prompt, max_tokens=5, temperature=1.0, seed=8, ignore_eos=True)
    assert len(pair.choices) == 2 and pair.choices[1].token_ids == one.choices[0].token_ids


def test_command_line_generates(model_folders, cuda_device):
    folder = model_folders("A", "float32")
    root = Path(__file__).resolve().parent.parent
    prompt = random_tokens(256, 7, seed=4)
    done = subprocess.run(
        [sys.executable, "-m", "zephyr_b200", "generate", str(folder), "--prompt-ids", ",".join(map(str, prompt)),
         "--max-tokens", "5", "--temperature", "0", "--dtype", "float32", "--kv-block-size", "4", "--num-kv-blocks", "40",
         "--ignore-eos"], capture_output=True, text=True, cwd=root, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    engine = make_engine(folder, "A", "float32", max_num_seqs=2, max_num_batched_tokens=32, max_prefill_chunk_tokens=32)
    expected = list(engine.generate(prompt, max_tokens=5, temperature=0.0, ignore_eos=True).token_ids)
    assert [int(t) for t in done.stdout.split()] == expected
