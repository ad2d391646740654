"""The scheduler's decisions on the host, with a real CacheManager and no GPU: portions under the
token budget, decoders before prompts, FIFO admission, preemption of the youngest when pages run
out, rejection of what can never fit, and determinism."""

import random

import pytest

from zephyr_b200.cache import CacheManager, PagedCacheSpec
from zephyr_b200.config import ConfigError, InvalidArgumentError
from zephyr_b200.engine.scheduler import (PagedSchedulerConfig, Scheduler, Sequence, SequenceState)

SPEC = PagedCacheSpec(num_kv_heads=2, key_dim=16)


class Harness:
    """Drives the scheduler as the engine does, with a stand-in for the model: the next token of a
    sequence is a function of its history, so a preempted sequence must end up with the same tokens."""

    def __init__(self, num_pages, page_size=4, spec=SPEC, **config):
        self.manager = CacheManager([spec], page_size, num_pages, config.get("max_num_seqs", 8))
        self.sequences: dict[int, Sequence] = {}
        self.scheduler = Scheduler(PagedSchedulerConfig(**config), self.sequences, self.manager)
        self.limits: dict[int, int] = {}
        self.log: list = []

    def add(self, sid, prompt, max_new):
        self.sequences[sid] = Sequence(sid, list(prompt))
        self.limits[sid] = max_new
        self.scheduler.add(sid)

    @staticmethod
    def next_token(history):
        return (sum(history) * 31 + len(history)) % 97

    def step(self):
        plan = self.scheduler.schedule()
        self.log.append([(s.sequence_id, s.start_token, s.num_tokens, s.sample) for s in plan.sequences])
        for item in plan.sequences:
            sequence = self.sequences[item.sequence_id]
            assert item.start_token == sequence.num_computed_tokens
            assert item.start_token + item.num_tokens <= len(sequence.token_ids)
            assert self.manager.length(item.sequence_id) >= item.start_token + item.num_tokens
            self.manager.commit(item.sequence_id, item.start_token + item.num_tokens)
        self.scheduler.commit(plan)
        for item in plan.sequences:
            if item.sample:
                sequence = self.sequences[item.sequence_id]
                sequence.token_ids.append(self.next_token(sequence.token_ids[:-0 or None]))
                if len(sequence.token_ids) - sequence.prompt_length >= self.limits[item.sequence_id]:
                    self.scheduler.finish(item.sequence_id)
        self.manager.check_invariants()
        return plan

    def run(self, max_steps=2000):
        steps = 0
        while self.scheduler.has_unfinished:
            plan = self.step()
            steps += 1
            assert steps < max_steps, "the scheduler does not terminate"
            assert plan.sequences or plan.preempted or plan.rejected, "a step without progress"
        return steps


def expected_tokens(prompt, max_new):
    history = list(prompt)
    for _ in range(max_new):
        history.append(Harness.next_token(history))
    return history


def test_config_is_validated():
    with pytest.raises(ConfigError):
        PagedSchedulerConfig(max_num_seqs=0).validate()
    defaults = PagedSchedulerConfig()
    assert (defaults.max_num_seqs, defaults.max_num_batched_tokens, defaults.max_prefill_chunk_tokens,
            defaults.max_decode_steps_before_prefill) == (8, 512, 512, 8)      # src/include/engine/engine.hpp:36-39


def test_prompts_are_cut_under_the_token_budget():
    h = Harness(num_pages=64, max_num_seqs=4, max_num_batched_tokens=16, max_prefill_chunk_tokens=10)
    h.add(0, range(25), 3)
    h.add(1, range(7), 2)
    plan = h.step()
    assert h.log[-1] == [(0, 0, 10, False), (1, 0, 6, False)]        # chunk limit 10, then what is left of 16
    plan = h.step()
    assert h.log[-1] == [(0, 10, 10, False), (1, 6, 1, True)]        # the last portion of a prompt samples
    plan = h.step()
    assert h.log[-1] == [(1, 7, 1, True), (0, 20, 5, True)]          # decoders first, then prompt portions
    assert all(sum(n for _, _, n, _ in step) <= 16 for step in h.log)
    h.run()
    assert h.sequences[0].token_ids == expected_tokens(range(25), 3)
    assert h.sequences[1].token_ids == expected_tokens(range(7), 2)
    assert h.manager.num_free_pages() == 63 and h.manager.num_requests == 0


def test_admission_is_fifo_and_waits_for_room():
    h = Harness(num_pages=9, max_num_seqs=4, max_num_batched_tokens=32, max_prefill_chunk_tokens=32)   # 8 pages = 32 tokens
    h.add(0, range(20), 4)       # 5 pages, grows to 6
    h.add(1, range(16), 2)       # 4 pages: does not fit beside 0
    h.add(2, range(3), 2)        # would fit, but may not overtake 1
    h.step()
    assert [s[0] for s in h.log[-1]] == [0]
    assert h.scheduler.waiting[0] == 1 and h.sequences[2].state == SequenceState.WAITING
    h.run()
    order = [s[0] for step in h.log for s in step if s[1] == 0]
    assert order == [0, 1, 2]
    for sid, (prompt, new) in {0: (range(20), 4), 1: (range(16), 2), 2: (range(3), 2)}.items():
        assert h.sequences[sid].token_ids == expected_tokens(prompt, new)


def test_a_prompt_that_can_never_fit_is_rejected():
    h = Harness(num_pages=5, max_num_seqs=2, max_num_batched_tokens=8, max_prefill_chunk_tokens=8)     # 16 tokens
    h.add(0, range(17), 1)
    h.add(1, range(4), 1)
    plan = h.step()
    assert plan.rejected == [0] and h.sequences[0].state == SequenceState.REJECTED
    assert "capacity" in h.sequences[0].error_message
    h.run()
    assert h.sequences[1].token_ids == expected_tokens(range(4), 1)


def test_out_of_pages_preempts_the_youngest_and_results_do_not_change():
    h = Harness(num_pages=9, max_num_seqs=3, max_num_batched_tokens=16, max_prefill_chunk_tokens=16)   # 32 tokens
    h.add(0, range(10), 14)      # 3 pages -> 6
    h.add(1, range(9), 14)       # 3 pages -> 6
    h.run()
    assert h.scheduler.num_preemptions > 0
    assert h.sequences[1].num_preemptions > 0 and h.sequences[0].num_preemptions == 0     # the younger one yields
    assert h.sequences[0].token_ids == expected_tokens(range(10), 14)
    assert h.sequences[1].token_ids == expected_tokens(range(9), 14)
    # A preempted sequence recomputes prompt and generated tokens from position 0.
    restarts = [s for step in h.log for s in step if s[0] == 1 and s[1] == 0]
    assert len(restarts) >= 2 and restarts[-1][2] > 9
    assert h.manager.num_free_pages() == 8


def test_a_lone_sequence_that_outgrows_the_pool_ends_rejected():
    h = Harness(num_pages=4, max_num_seqs=2, max_num_batched_tokens=8, max_prefill_chunk_tokens=8)      # 12 tokens
    h.add(0, range(6), 50)
    h.run()
    assert h.sequences[0].state == SequenceState.REJECTED
    assert len(h.sequences[0].token_ids) == 13        # it grew until the pool was full, then could not restart


def test_finish_and_add_rules():
    h = Harness(num_pages=16, max_num_seqs=2, max_num_batched_tokens=8, max_prefill_chunk_tokens=8)
    h.add(0, range(5), 5)
    with pytest.raises(InvalidArgumentError):
        h.scheduler.add(0)
    h.step()
    h.scheduler.finish(0)                 # cancellation mid-flight
    h.scheduler.finish(0)                 # safe to repeat
    assert h.sequences[0].state == SequenceState.FINISHED and not h.scheduler.has_unfinished
    assert h.manager.num_free_pages() == 15
    h.add(1, range(3), 1)
    h.scheduler.finish(1)                 # cancelled while waiting
    assert not h.scheduler.has_unfinished


def test_more_decoders_than_the_token_budget_take_turns():
    """Six decoders under a budget of two tokens a step: the turn moves on, so that every decoder is
    served once in three steps and nobody starves."""
    h = Harness(num_pages=64, max_num_seqs=6, max_num_batched_tokens=16, max_prefill_chunk_tokens=16)
    for sid in range(6):
        h.add(sid, [sid + 1], 9)
    h.step()                                                            # all six prompts in one step
    assert all(h.sequences[sid].state == SequenceState.DECODE for sid in range(6))
    h.scheduler.config = PagedSchedulerConfig(max_num_seqs=6, max_num_batched_tokens=2, max_prefill_chunk_tokens=2)
    served = []
    for _ in range(6):
        h.step()
        assert len(h.log[-1]) == 2 and all(n == 1 for _, _, n, _ in h.log[-1])
        served.append(sorted(s[0] for s in h.log[-1]))
    for start in range(0, 6, 3):
        assert sorted(sum(served[start:start + 3], [])) == list(range(6)), served
    h.run()
    for sid in range(6):
        assert h.sequences[sid].token_ids == expected_tokens([sid + 1], 9)


@pytest.mark.parametrize("num_pages", range(7, 16))
def test_long_prompts_in_a_windowed_group_do_not_starve_each_other(num_pages):
    """A windowed group gives pages back while a prompt is still being computed.  The prompt keeps its
    claim on as many pages as it holds at one time, so that requests admitted meanwhile cannot leave
    every prompt short of pages (a step without progress)."""
    windowed = PagedCacheSpec(num_kv_heads=2, key_dim=16, window=8)
    h = Harness(num_pages=num_pages, spec=windowed, max_num_seqs=4, max_num_batched_tokens=16, max_prefill_chunk_tokens=8)
    jobs = {sid: (list(range(sid, sid + 60)), 3) for sid in range(4)}
    for sid, job in jobs.items():
        h.add(sid, *job)
    h.run()
    for sid, (prompt, new) in jobs.items():
        assert h.sequences[sid].token_ids == expected_tokens(prompt, new), sid
    assert h.manager.num_requests == 0 and h.manager.num_free_pages() == num_pages - 1


@pytest.mark.parametrize("seed", range(5))
def test_random_workloads_finish_with_the_right_tokens(seed):
    rng = random.Random(seed)
    h = Harness(num_pages=rng.randrange(12, 30), page_size=4, max_num_seqs=rng.randrange(2, 6),
                max_num_batched_tokens=rng.randrange(8, 24), max_prefill_chunk_tokens=rng.randrange(2, 16))
    jobs = {}
    for sid in range(10):
        prompt = [rng.randrange(97) for _ in range(rng.randrange(1, 30))]
        jobs[sid] = (prompt, rng.randrange(1, 12))
        h.add(sid, *jobs[sid])
    h.run()
    for sid, (prompt, new) in jobs.items():
        assert h.sequences[sid].token_ids == expected_tokens(prompt, new), sid
    assert h.manager.num_requests == 0 and h.manager.num_free_pages() == h.manager.groups[0].pool.num_usable
    again = Harness(num_pages=h.manager.groups[0].pool.num_pages, page_size=4, **{
        k: getattr(h.scheduler.config, k) for k in ("max_num_seqs", "max_num_batched_tokens", "max_prefill_chunk_tokens")})
    for sid, job in jobs.items():
        again.add(sid, *job)
    again.run()
    assert again.log == h.log            # the same requests in the same order give the same schedule
