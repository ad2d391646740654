"""The cache manager on the host: no page lost, held twice or freed twice, under random orders of
requests; groups with windows give pages back as the window passes; state slots; reservations."""

import random

import pytest

from zephyr_b200.cache import NULL_PAGE, CacheManager, PagedCacheSpec, PagePool, StateCacheSpec, StateSlots
from zephyr_b200.config import InvalidArgumentError, OutOfPagesError

FULL = PagedCacheSpec(num_kv_heads=2, key_dim=16, window=0)
WINDOW = PagedCacheSpec(num_kv_heads=2, key_dim=16, window=10)
STATE = StateCacheSpec(shape=(4,))


def test_pool_basics():
    pool = PagePool(6)
    assert pool.num_free == 5 and pool.num_usable == 5
    pages = pool.allocate(3)
    assert pages == [1, 2, 3] and NULL_PAGE not in pages
    with pytest.raises(OutOfPagesError):
        pool.allocate(3)                                   # all or nothing
    assert pool.num_free == 2
    pool.free([2])
    with pytest.raises(InvalidArgumentError, match="not in use"):
        pool.free([2])                                     # freed twice
    with pytest.raises(InvalidArgumentError):
        pool.free([9])
    pool.free([NULL_PAGE])                                 # the null page is never anyone's
    assert pool.allocate(3) == [4, 5, 2]                   # reuse in the order pages came back
    with pytest.raises(InvalidArgumentError):
        PagePool(1)


def test_state_slots():
    slots = StateSlots(2)
    a, b = slots.acquire(), slots.acquire()
    assert {a, b} == {0, 1}
    with pytest.raises(OutOfPagesError):
        slots.acquire()
    slots.release(a)
    with pytest.raises(InvalidArgumentError):
        slots.release(a)
    assert slots.acquire() == a


def test_groups_are_formed_by_need():
    manager = CacheManager([FULL, WINDOW, FULL, STATE, None, WINDOW], page_size=4, num_pages=9, max_requests=3)
    assert len(manager.groups) == 2
    assert manager.groups[0].cache_ids == [0, 2] and manager.groups[1].cache_ids == [1, 5]
    assert manager.state_cache_ids == [3]
    assert manager.group_of_cache == {0: 0, 2: 0, 1: 1, 5: 1}
    with pytest.raises(InvalidArgumentError, match="power of two"):
        CacheManager([FULL], page_size=6, num_pages=4, max_requests=1)


def test_tables_grow_and_pages_return_in_reverse():
    manager = CacheManager([FULL], page_size=4, num_pages=8, max_requests=2)
    assert manager.add_request("a")
    assert manager.ensure_capacity("a", 5) and manager.block_table("a") == [1, 2]
    assert manager.ensure_capacity("a", 8) and manager.block_table("a") == [1, 2]       # still two pages
    assert manager.ensure_capacity("a", 9) and manager.block_table("a") == [1, 2, 3]
    manager.commit("a", 9)
    with pytest.raises(InvalidArgumentError):
        manager.commit("a", 20)
    assert manager.add_request("b") and not manager.add_request("c")                     # two slots only
    assert not manager.ensure_capacity("b", 17)                                          # 5 pages wanted, 4 free
    assert manager.block_table("b") == [] and manager.num_free_pages() == 4              # nothing was taken
    manager.free_request("a")
    manager.check_invariants()
    assert manager.ensure_capacity("b", 17) and manager.block_table("b") == [4, 5, 6, 7, 3]   # 3, 2, 1 came back in that order
    with pytest.raises(InvalidArgumentError):
        manager.add_request("b")


def test_reservation_protects_an_admitted_prompt():
    manager = CacheManager([FULL], page_size=4, num_pages=11, max_requests=4)           # 10 usable pages
    assert manager.add_request("p", reserve_tokens=24)                                   # 6 pages promised
    assert manager.num_unreserved_pages() == 4
    assert manager.add_request("d")
    assert manager.ensure_capacity("d", 16)                                              # 4 pages, all that is unreserved
    assert not manager.ensure_capacity("d", 17)                                          # may not eat the promise
    assert not manager.add_request("q", reserve_tokens=4)                                # nor may a newcomer
    assert manager.ensure_capacity("p", 24) and manager.num_unreserved_pages() == 0
    manager.check_invariants()
    assert manager.fits_at_all(40, 8) and not manager.fits_at_all(41, 8)


def test_window_groups_give_pages_back_as_the_window_passes():
    manager = CacheManager([FULL, WINDOW], page_size=4, num_pages=40, max_requests=2)
    assert manager.add_request("a")
    computed = 0
    for portion in (7, 2, 5, 1, 1, 1, 9, 3):
        assert manager.ensure_capacity("a", computed + portion)
        # Every key a query of this portion may see lies in a page that is still held.
        first_visible = max(0, computed - WINDOW.window + 1)
        for position in range(first_visible, computed + portion):
            assert manager.block_table("a", 1)[position // 4] != NULL_PAGE
        computed += portion
        manager.commit("a", computed)
        manager.check_invariants()
        table = manager.block_table("a", 1)
        dead = max(0, (computed - WINDOW.window + 1) // 4)
        assert all(page == NULL_PAGE for page in table[:dead]) and all(page != NULL_PAGE for page in table[dead:])
        assert NULL_PAGE not in manager.block_table("a", 0)                              # the full group keeps all
    live = sum(1 for page in manager.block_table("a", 1) if page != NULL_PAGE)
    assert live <= -(-(WINDOW.window + 9) // 4) + 1
    manager.free_request("a")
    manager.check_invariants()
    assert manager.num_free_pages(0) == 39 and manager.num_free_pages(1) == 39


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_of_requests(seed):
    rng = random.Random(seed)
    specs = [FULL, WINDOW, FULL, STATE] if seed % 2 else [FULL]
    manager = CacheManager(specs, page_size=1 << rng.randrange(0, 4), num_pages=rng.randrange(8, 40), max_requests=4)
    live: dict[int, int] = {}
    next_id = 0
    for _ in range(600):
        action = rng.random()
        if action < 0.25 and len(live) < 6:
            admitted = manager.add_request(next_id, reserve_tokens=rng.randrange(0, 20), step_tokens=8)
            assert admitted == (next_id in manager)
            if admitted:
                live[next_id] = 0
            else:
                assert manager.num_requests == 4 or True
            next_id += 1
        elif action < 0.8 and live:
            rid = rng.choice(list(live))
            grow = rng.randrange(1, 9)
            before = [list(manager.block_table(rid, g)) for g in range(len(manager.groups))]
            if manager.ensure_capacity(rid, live[rid] + grow):
                live[rid] += grow
                manager.commit(rid, live[rid])
            else:
                assert before == [list(manager.block_table(rid, g)) for g in range(len(manager.groups))]
        elif live:
            rid = rng.choice(list(live))
            manager.free_request(rid)
            del live[rid]
            with pytest.raises(KeyError):
                manager.free_request(rid)                  # freed twice
        manager.check_invariants()
    for rid in list(live):
        manager.free_request(rid)
    manager.check_invariants()
    assert all(g.pool.num_free == g.pool.num_usable for g in manager.groups)
    assert manager.slots.num_free == 4


def test_keys_and_values_of_different_widths_have_pages_of_their_own():
    """A cache whose keys are wider than its values (a compressed or asymmetric mixer) forms a group
    apart from the equal-width ones, costs key_dim + value_dim per position and head, and its storage
    hands out the two halves of every page as views."""
    import torch

    from zephyr_b200.cache import CacheStorage, bytes_per_page

    equal = PagedCacheSpec(num_kv_heads=2, key_dim=16)
    lopsided = PagedCacheSpec(num_kv_heads=2, key_dim=24, value_dim=8)
    assert equal.value_dim == 16 and equal.head_dim == 16
    with pytest.raises(InvalidArgumentError, match="no single head size"):
        lopsided.head_dim
    manager = CacheManager([equal, lopsided, equal], 4, 6, 2)
    assert [g.cache_ids for g in manager.groups] == [[0, 2], [1]]
    assert bytes_per_page(manager.cache_specs, 4, torch.bfloat16) == 2 * (2 * 4 * 32 * 2) + 2 * 4 * 32 * 2
    storage = CacheStorage(manager, torch.float32, "cpu")
    assert storage[0].shape == (6, 2, 2, 4, 16) and storage[1].shape == (6, 2 * 4 * 32)
    keys, values = storage.keys(1), storage.values(1)
    assert keys.shape == (6, 2, 4, 24) and values.shape == (6, 2, 4, 8)
    keys[3, 1, 2, :] = 1.0
    values[3, 1, 2, :] = 2.0
    page = storage[1][3]
    assert page.sum() == 24 + 16 and page[(1 * 4 + 2) * 24] == 1.0 and page[2 * 4 * 24 + (1 * 4 + 2) * 8] == 2.0
    assert storage.keys(0).shape == (6, 2, 4, 16) and storage.values(2).data_ptr() == storage[2][:, 1].data_ptr()
