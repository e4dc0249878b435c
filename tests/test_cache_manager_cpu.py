"""The cache manager's bookkeeping: no page lost, held twice or freed twice, under random
orders of requests; window release; reservations; state slots (no GPU)."""
import random

import pytest

from dispec_b200.cache import CacheGroupSpec, CacheManager, OutOfPagesError, OutOfSlotsError, PagePool


def test_pool_hands_out_ascending_ids_and_refuses_double_free():
    pool = PagePool(4)
    assert [pool.alloc() for _ in range(4)] == [0, 1, 2, 3]
    with pytest.raises(OutOfPagesError):
        pool.alloc()
    assert pool.release(2) and pool.alloc() == 2
    pool.release(1)
    with pytest.raises(RuntimeError, match="double free"):
        pool.release(1)


def test_pages_grow_only_when_full_and_return_on_free():
    m = CacheManager([CacheGroupSpec.key_value(2, 16)], page_size=4, num_pages=8, max_num_seqs=2)
    m.admit("a")
    m.extend("a", 3)
    assert len(m.block_table("a")) == 1
    m.commit("a", 3)
    m.extend("a", 4)
    assert len(m.block_table("a")) == 1
    m.extend("a", 5)
    assert len(m.block_table("a")) == 2 and m.num_free_pages() == 6
    m.commit("a", 5)
    m.check()
    m.free("a")
    assert m.num_free_pages() == 8 and m.free_slots() == 2
    m.check()
    assert m.free("a") == []  # freeing twice is harmless


def test_a_request_after_another_gets_its_pages_in_ascending_order_again():
    m = CacheManager([CacheGroupSpec.key_value(2, 16)], page_size=4, num_pages=12, max_num_seqs=2)
    m.admit("a")
    m.extend("a", 20)
    assert list(m.block_table("a")) == [0, 1, 2, 3, 4]
    m.admit("b")
    m.extend("b", 8)
    m.commit("a", 20)
    m.free("a")
    m.admit("c")
    m.extend("c", 28)  # a's five pages in a's order, then fresh ones
    assert list(m.block_table("c")) == [0, 1, 2, 3, 4, 7, 8]
    m.check()


def test_portions_of_prompts_get_runs_of_consecutive_pages_while_requests_come_and_go():
    """The attention kernel for portions of prompts fetches a key tile with one request where the
    tile's pages follow one another in the pool.  Requests that take their pages portion by portion,
    beside each other, and end in any order still get such runs: here at least three quarters of
    the aligned groups of four pages, over a random workload on a pool that is used several times over."""
    rng = random.Random(5)
    m = CacheManager([CacheGroupSpec.key_value(2, 16)], page_size=16, num_pages=512, max_num_seqs=8)
    live, groups, in_run, next_id = {}, 0, 0, 0
    for _ in range(400):
        if len(live) < 4 and rng.random() < 0.5:
            live[next_id] = [0, rng.choice([300, 700, 1500, 2048])]
            m.admit(next_id)
            next_id += 1
        for rid in list(live):
            have, want = live[rid]
            if have < want:
                step = min(want - have, rng.choice([64, 256, 512]))
                try:
                    m.extend(rid, have + step)
                except OutOfPagesError:
                    continue
                m.commit(rid, have + step)
                live[rid][0] = have + step
            elif rng.random() < 0.3:
                table = list(m.block_table(rid))
                for i in range(0, len(table) - 3, 4):
                    groups += 1
                    in_run += all(table[i + j] == table[i] + j for j in range(4))
                m.free(rid)
                del live[rid]
        m.check()
    assert groups > 300 and in_run >= 0.75 * groups, (in_run, groups)


def test_extend_takes_nothing_when_it_cannot_take_all():
    groups = [CacheGroupSpec.key_value(1, 8), CacheGroupSpec.key_value(1, 8, window=4)]
    m = CacheManager(groups, page_size=2, num_pages=[10, 2], max_num_seqs=2)
    m.admit("a")
    with pytest.raises(OutOfPagesError):
        m.extend("a", 6)  # group 1 has 2 pages, 3 are needed
    assert m.num_free_pages(0) == 10 and m.num_free_pages(1) == 2
    m.check()


def test_window_group_gives_pages_back_as_the_window_passes_them():
    groups = [CacheGroupSpec.key_value(1, 8), CacheGroupSpec.key_value(1, 8, window=5)]
    m = CacheManager(groups, page_size=4, num_pages=[16, 4], max_num_seqs=2)
    m.admit("a")
    stored = 0
    held = []
    for n in [3, 6, 1, 1, 1, 7, 1, 1, 1, 1, 1, 1]:
        m.extend("a", stored + n)
        stored += n
        m.commit("a", stored)
        m.check()
        table = m.block_table("a", 1)
        first_needed = max(0, stored - 5 + 1)
        for j, page in enumerate(table):
            # every position the next query can see is still backed by a page
            if (j + 1) * 4 > first_needed:
                assert page >= 0
            else:
                assert page == -1
        held.append(sum(p >= 0 for p in table))
        assert all(p >= 0 for p in m.block_table("a", 0))
    assert max(held) <= 3 and stored == 25
    m.free("a")
    m.check()
    assert m.num_free_pages(1) == 4


def test_reservation_guarantees_the_prompt_and_is_returned():
    m = CacheManager([CacheGroupSpec.key_value(1, 8)], page_size=4, num_pages=6, max_num_seqs=4)
    assert m.can_admit(16, 20, 8)
    m.admit("a", 16, 20, 8)  # reserves 4 pages
    assert m.num_available_pages() == 2 and m.num_free_pages() == 6
    assert not m.can_admit(12, 12, 8)
    m.admit("b", 8, 8, 8)
    assert m.num_available_pages() == 0
    m.extend("a", 8)
    m.extend("b", 8)
    m.commit("a", 8)
    m.check()
    m.extend("a", 16)  # still covered by the promise
    with pytest.raises(OutOfPagesError):
        m.extend("b", 9)  # beyond its promise and nothing is unpromised
    m.free("a")
    assert m.num_available_pages() == 4
    m.extend("b", 9)
    m.check()


def test_state_slots_are_unique_and_run_out():
    m = CacheManager([CacheGroupSpec.key_value(1, 8)], page_size=4, num_pages=4, max_num_seqs=2)
    a, b = m.admit("a"), m.admit("b")
    assert {a, b} == {0, 1}
    with pytest.raises(OutOfSlotsError):
        m.admit("c")
    with pytest.raises(ValueError):
        m.admit("a")
    m.free("a")
    assert m.admit("c") == a


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_keep_every_invariant(seed):
    rng = random.Random(seed)
    groups = [CacheGroupSpec.key_value(2, 16, 0, 3), CacheGroupSpec.key_value(2, 16, window=rng.choice([3, 8, 21]), num_slots=2)]
    page = rng.choice([2, 4, 8])
    m = CacheManager(groups, page_size=page, num_pages=[rng.randint(12, 40), rng.randint(8, 20)],
                     max_num_seqs=5)
    live = {}
    next_id = 0
    for _ in range(600):
        action = rng.random()
        if action < 0.25 and m.free_slots():
            prompt = rng.randint(1, 40)
            if rng.random() < 0.5:
                if m.can_admit(prompt, prompt + 10, 8):
                    m.admit(next_id, prompt, prompt + 10, 8)
                    live[next_id] = 0
                    next_id += 1
            else:
                m.admit(next_id)
                live[next_id] = 0
                next_id += 1
        elif action < 0.85 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 5, 8])
            if m.can_extend(rid, live[rid] + n):
                m.extend(rid, live[rid] + n)
                live[rid] += n
                m.commit(rid, live[rid])
            else:
                with pytest.raises(OutOfPagesError):
                    m.extend(rid, live[rid] + n)
        elif live:
            rid = rng.choice(list(live))
            m.free(rid)
            del live[rid]
        m.check()
        assert set(m.live_requests()) == set(live)
    for rid in list(live):
        m.free(rid)
    m.check()
    assert all(pool.num_free == pool.num_pages and pool.reserved == 0 for pool in m.pools)
