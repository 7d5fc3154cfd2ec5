"""The cache manager on the host (no GPU): pools, prefix index, groups with a
window, state slots, block tables, packed step arrays, and invariants under
random orders of requests."""

import random

import numpy as np
import pytest

import plain_llama as plain
from stride_b200.cache import CacheManager, runtime

rt = runtime()


def chain_publish_release(pool, tenant, tokens, pages):
    pool.publish(tenant, tokens, len(tokens), pages)
    pool.release(pages)


def test_hash_chain_matches_the_plain_restatement():
    toks = list(range(40))
    assert rt.tenant_root("acme") == 0x0724D383F4F6DE0F
    assert rt.prefix_chain("acme", toks, 16) == plain.prefix_chain("acme", toks, 16)
    assert rt.prefix_chain("acme", toks[:32], 16) == [0xBF0700EAC0C3E9F1, 0x7B8B4746D9BC7AD4]
    assert rt.prefix_chain("acme", toks, 16)[:1] == rt.prefix_chain("acme", toks[:16] + [99] * 24, 16)[:1]
    assert rt.prefix_chain("acme", toks, 16)[1] != rt.prefix_chain("acme", toks[:16] + [99] * 24, 16)[1]


def test_pool_exhaustion_sharing_and_counts():
    pool = rt.PagePool(4, 16)
    pages = pool.allocate(4)
    assert pages == [0, 1, 2, 3] and pool.num_allocatable == 0
    with pytest.raises(rt.OutOfPages):
        pool.allocate(1)
    pool.check_invariants()
    pool.release(pages)
    assert pool.stats()["free"] == 4 and pool.stats()["live"] == 0
    with pytest.raises(rt.InvariantError, match="freed twice"):
        pool.release([pages[0]])
    # a failed allocation leaves the pool untouched
    held = pool.allocate(3)
    before = pool.stats()
    with pytest.raises(rt.OutOfPages):
        pool.allocate(2)
    assert pool.stats() == before
    pool.release(held)
    pool.check_invariants()


def test_prefix_reuse_counts():
    # 64-token prompt, pages of 16: nothing at first, then all but the last page
    pool = rt.PagePool(64, 16)
    prompt = list(range(64))
    for expected in (0, 48, 48):
        hit = pool.acquire_prefix("t", prompt)
        assert len(hit) * 16 == expected
        fresh = pool.allocate(4 - len(hit))
        chain_publish_release(pool, "t", prompt, hit + fresh)
        pool.check_invariants()
    # a shared 32-token system prompt
    system = list(range(1000, 1032))
    a = pool.allocate(3)
    chain_publish_release(pool, "t", system + [1, 2, 3], a)
    assert len(pool.acquire_prefix("t", system + [7, 8, 9, 10])) * 16 == 32
    # divergence at token 20: only the first page matches
    other = prompt[:20] + [5000 + i for i in range(44)]
    assert len(pool.acquire_prefix("t", other)) * 16 == 16
    # another tenant sees nothing
    assert pool.acquire_prefix("u", prompt) == []
    # a prompt that ends exactly on a page edge leaves its last page to be run
    assert len(pool.acquire_prefix("t", prompt[:48])) * 16 == 32


def test_shared_pages_stay_until_the_last_holder_leaves_and_lru_evicts_leaves_first():
    pool = rt.PagePool(6, 4)
    toks = list(range(16))
    pages = pool.allocate(4)
    chain_publish_release(pool, "t", toks, pages)
    assert pool.stats()["cached"] == 4
    a = pool.acquire_prefix("t", toks + [1])
    b = pool.acquire_prefix("t", toks + [2])
    assert a == b == pages and pool.refcount(pages[0]) == 2
    pool.release(a)
    assert pool.stats()["live"] == 4
    pool.release(b)
    assert pool.stats() == {**pool.stats(), "live": 0, "cached": 4, "free": 2}
    # pressure: the free pages go first, then the chain's leaf, never its root first
    got = pool.allocate(3)
    assert got[:2] == [5, 4] or set(got[:2]) == {4, 5}
    assert got[2] == pages[3], "the least recently used page must be the chain's last page"
    assert len(pool.acquire_prefix("t", toks + [3])) == 3
    pool.check_invariants()


def test_the_invariant_check_can_fail():
    for what, match in ((0, "!= capacity"), (1, "free list twice"), (2, "live counter")):
        pool = rt.PagePool(8, 4)
        held = pool.allocate(2)
        pool.check_invariants()
        pool.corrupt_for_test(what)
        with pytest.raises(rt.InvariantError, match=match):
            pool.check_invariants()
        del held


def test_manager_tables_slots_and_windows():
    cm = CacheManager(4, [(10, 0), (6, 8)], 3, True)
    assert not cm.prefix_caching, "sharing by content is only sound when every group keeps all keys"
    assert cm.open(1, "a") in (0, 1, 2)
    assert cm.ensure(1, 9)
    assert len(cm.table(1, 0)) == 3 and len(cm.table(1, 1)) == 3
    # the window group gives back pages that the window has passed; the full group keeps them
    assert cm.ensure(1, 21)
    given = cm.trim(1, 21)
    # next query at >= 21 reads keys >= 14: pages 0..2 (keys 0..11) are passed
    assert given == 3 and cm.table(1, 1)[:3] == [-1, -1, -1] and all(p >= 0 for p in cm.table(1, 1)[3:])
    assert all(p >= 0 for p in cm.table(1, 0))
    assert cm.stats(1)["live"] == 3 and cm.stats(0)["live"] == 6
    cm.check_invariants()
    # all or nothing across groups: group 1 has 3 pages left, group 0 has 4
    cm.open(2, "b")
    assert not cm.ensure(2, 16)
    assert cm.table(2, 0) == [] and cm.table(2, 1) == []
    assert cm.ensure(2, 12)
    cm.open(3, "c")
    with pytest.raises(rt.OutOfPages):
        cm.open(4, "d")          # no state slot left
    with pytest.raises(ValueError, match="already holds"):
        cm.open(3, "c")
    for r in (1, 2, 3):
        cm.close(r)
    with pytest.raises(ValueError, match="holds no cache"):
        cm.close(1)
    cm.check_invariants()
    assert cm.free_slots == 3 and cm.stats(0)["free"] == 10 and cm.stats(1)["free"] == 6


def test_manager_prefix_sharing_through_tables():
    cm = CacheManager(4, [(12, 0)], 4, True)
    toks = list(range(10))
    cm.open(1, "t")
    assert cm.adopt_prefix(1, toks) == 0 and cm.ensure(1, 10)
    cm.publish(1, toks, 9)                # only 9 tokens have keys: two full pages
    cm.close(1)
    assert cm.stats()["cached"] == 2
    cm.open(2, "t")
    cm.open(3, "t")
    assert cm.adopt_prefix(2, toks) == 8 and cm.adopt_prefix(3, toks + [11, 12]) == 8
    assert cm.table(2, 0) == cm.table(3, 0)
    assert cm.ensure(2, 10) and cm.ensure(3, 12)
    assert cm.table(2, 0)[2] != cm.table(3, 0)[2], "the tail page must be private"
    cm.check_invariants()
    cm.close(2)
    cm.check_invariants()
    cm.close(3)
    assert cm.stats()["live"] == 0


def test_random_orders_of_requests_keep_every_invariant():
    rng = random.Random(1234)
    for trial in range(30):
        page = rng.choice([4, 8, 16])
        windows = rng.choice([[0], [0, 12], [20], [0, 0]])
        cm = CacheManager(page, [(rng.randint(6, 20), w) for w in windows], rng.randint(2, 5), trial % 2 == 0)
        held = {}
        next_id = 1
        for _ in range(300):
            op = rng.random()
            if op < 0.25 and cm.free_slots:
                cm.open(next_id, rng.choice("ab"))
                held[next_id] = 0
                next_id += 1
            elif op < 0.75 and held:
                r = rng.choice(list(held))
                grow = rng.randint(1, 3 * page)
                before = [list(cm.table(r, g)) for g in range(cm.num_groups)]
                if cm.ensure(r, held[r] + grow, rng.choice([0, 1])):
                    held[r] += grow
                    cm.trim(r, held[r])
                    if trial % 2 == 0 and rng.random() < 0.3:
                        cm.publish(r, [rng.randrange(3) for _ in range(held[r])], held[r])
                else:
                    assert before == [list(cm.table(r, g)) for g in range(cm.num_groups)], "a failed ensure changed a table"
            elif held:
                r = rng.choice(list(held))
                cm.close(r)
                del held[r]
            cm.check_invariants()
            # no page is held by two requests unless it was shared through the index
            for g in range(cm.num_groups):
                seen = {}
                for r in held:
                    for p in cm.table(r, g):
                        if p >= 0:
                            seen[p] = seen.get(p, 0) + 1
                assert all(n == 1 for n in seen.values()) or cm.prefix_caching
        for r in list(held):
            cm.close(r)
        cm.check_invariants()
        for g in range(cm.num_groups):
            s = cm.stats(g)
            assert s["live"] == 0 and s["free"] + s["cached"] == s["capacity"]
        assert cm.free_slots == cm.slot_capacity


def test_packed_step_arrays():
    cm = CacheManager(4, [(16, 0)], 4, False)
    cm.open(7)
    cm.open(9)
    assert cm.ensure(7, 10) and cm.ensure(9, 6)
    batch = rt.StepBatch(cm)
    batch.add(7, [11, 12, 13], 7, [0, 2])          # a portion in the middle of request 7
    batch.add(9, [21], 5, [0])                      # a single decoded token of request 9
    batch.add(5, [], 0, [])                         # an empty portion is skipped
    assert (batch.num_tokens, batch.num_seqs, batch.num_rows, batch.max_q_len, batch.max_ctx) == (4, 2, 3, 3, 10)
    assert not batch.decode_only and batch.row_requests() == [7, 7, 9]
    arr, lay = batch.pack(1, 6, 3, 4, 5)
    view = lambda name, n: arr[lay[name]: lay[name] + n].tolist()
    assert view("token_ids", 6) == [11, 12, 13, 21, 0, 0]
    assert view("positions", 6) == [7, 8, 9, 5, 0, 0]
    assert view("seq_of_token", 6) == [0, 0, 0, 1, -1, -1]
    assert view("logit_rows", 4) == [0, 2, 3, 0]
    assert view("q_start", 3) == [0, 3, 0] and view("q_len", 3) == [3, 1, 0] and view("ctx_len", 3) == [10, 6, 0]
    assert view("state_slot", 2) == [cm.state_slot(7), cm.state_slot(9)]
    t7, t9 = cm.table(7, 0), cm.table(9, 0)
    slots = arr[lay["slot_mapping"][0]: lay["slot_mapping"][0] + 6].tolist()
    assert slots == [t7[1] * 4 + 3, t7[2] * 4 + 0, t7[2] * 4 + 1, t9[1] * 4 + 1, -1, -1]
    table = arr[lay["block_table"][0]: lay["block_table"][0] + 15].reshape(3, 5).tolist()
    assert table == [t7 + [-1, -1], t9 + [-1, -1, -1], [-1] * 5]
    # slices of the wanted rows
    arr2, _ = batch.pack(1, 6, 3, 2, 5, None, 1, 2)
    assert arr2[lay["logit_rows"]: lay["logit_rows"] + 2].tolist() == [2, 3]
    with pytest.raises(ValueError, match="does not fit"):
        batch.pack(1, 3, 3, 4, 5)
    with pytest.raises(ValueError, match="twice"):
        batch.add(7, [1], 10, [])
    other = rt.StepBatch(cm)
    with pytest.raises(IndexError, match="only 3 are mapped"):
        other.add(7, [1, 2, 3], 10, [])
    with pytest.raises(IndexError, match="outside the portion"):
        other.add(9, [1], 5, [1])
    with pytest.raises(ValueError, match="holds no cache"):
        other.add(5, [1], 0, [0])
