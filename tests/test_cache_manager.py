"""The host cache manager: pages, block tables, windows, slots (CPU).

No page is ever lost, held twice or freed twice, under random orders of requests; the
check is both the manager's own invariant scan and an independent model kept here."""
import random

import pytest
from hypothesis import given, settings, strategies as st

from mstar_b200.cache import CacheExhausted, CacheManager, GroupConfig, NoFreeSlot


def test_growth_commit_and_block_table():
    cm = CacheManager([GroupConfig(page_size=4, num_pages=6)], num_slots=2)
    assert cm.add_request("a") == 0
    cm.reserve(["a"], [9])
    assert cm.block_table("a") == [0, 1, 2]            # first-in first-out page ids
    assert cm.length("a") == 0                         # length moves at commit only
    b = cm.fill_batch(["a"], [9])
    assert b.positions.tolist() == list(range(9)) and b.kv_len.tolist() == [9]
    assert b.qo_indptr.tolist() == [0, 9] and b.tables[0].tolist() == [[0, 1, 2]]
    cm.commit("a", 9)
    assert cm.length("a") == 9 and cm.free_pages() == 3
    cm.reserve(["a"], [3])                             # fills the third page: no new page
    assert cm.free_pages() == 3
    cm.commit("a", 3)
    cm.reserve(["a"], [1])
    assert cm.block_table("a") == [0, 1, 2, 3]
    with pytest.raises(ValueError):
        cm.commit("a", 9)                              # more than was reserved
    cm.free_request("a")
    assert cm.free_pages() == 6 and cm.free_slots() == 2 and cm.check() == 0
    # freed pages go to the tail of the queue: 4, 5 come before 0..3 are used again
    cm.add_request("b")
    cm.reserve(["b"], [12])
    assert cm.block_table("b") == [4, 5, 0]


def test_batch_reservation_is_all_or_nothing():
    cm = CacheManager([GroupConfig(4, 5)], num_slots=3)
    for r in "abc":
        cm.add_request(r)
    cm.reserve(["a"], [8])
    cm.commit("a", 8)
    with pytest.raises(CacheExhausted) as err:
        cm.reserve(["a", "b", "c"], [1, 8, 5])         # needs 1 + 2 + 2 pages, 3 are free
    assert err.value.short_by == [2]
    assert cm.free_pages() == 3 and cm.block_table("b") == [] and cm.check() == 0
    with pytest.raises(ValueError):
        cm.reserve(["a", "a"], [1, 1])
    cm.reserve(["a", "b"], [1, 8])
    b = cm.fill_batch(["a", "b"], [1, 8])
    assert b.token_req.tolist() == [0] + [1] * 8
    assert b.positions.tolist() == [8] + list(range(8))
    assert b.tables[0].tolist() == [[0, 1, 2], [3, 4, -1]]
    assert b.slots.tolist() == [0, 1]


def test_slots():
    cm = CacheManager([GroupConfig(4, 4)], num_slots=2)
    assert cm.add_request("a") == 0 and cm.add_request("b") == 1
    with pytest.raises(NoFreeSlot):
        cm.add_request("c")
    with pytest.raises(ValueError):
        cm.add_request("a")
    cm.free_request("a")
    assert cm.add_request("c") == 0                    # the freed slot is used again
    with pytest.raises(KeyError):
        cm.free_request("a")                           # not twice


def test_window_group_gives_pages_back_while_the_request_runs():
    cm = CacheManager([GroupConfig(4, 100), GroupConfig(4, 6, window=6)], num_slots=1)
    cm.add_request("a")
    held = []
    for step in range(40):                             # 40 tokens, one at a time
        cm.reserve(["a"], [1])
        cm.commit("a", 1)
        held.append(6 - cm.free_pages(1))
        assert cm.check() == 0
    # a window of 6 keys over pages of 4 never needs more than 3 pages
    assert max(held) <= 3
    assert 100 - cm.free_pages(0) == 10                # the full group keeps everything
    table = cm.block_table("a", 1)
    assert len(table) == 10 and table[:8] == [-1] * 8 and all(p >= 0 for p in table[8:])
    # a long portion needs pages for all its tokens at once, and frees most afterwards
    cm.free_request("a")
    cm.add_request("b")
    with pytest.raises(CacheExhausted):
        cm.reserve(["b"], [30])
    cm.reserve(["b"], [24])
    cm.commit("b", 24)
    assert cm.free_pages(1) == 4 and cm.check() == 0


class Model:
    """Independent bookkeeping of who must hold how many pages."""

    def __init__(self, groups):
        self.groups = groups
        self.len = {}

    def pages_held(self, rid, g):
        ps, window = self.groups[g].page_size, self.groups[g].window
        n = self.len[rid]
        total = -(-n // ps)
        if window is None:
            return total
        first_key = max(n - window + 1, 0)
        return total - min(first_key // ps, total)


@settings(max_examples=60, deadline=None)
@given(seed=st.integers(0, 10 ** 6), window=st.sampled_from([None, 5, 16]),
       page=st.sampled_from([1, 4, 16]))
def test_random_orders_lose_nothing(seed, window, page):
    rng = random.Random(seed)
    groups = [GroupConfig(page, 40), GroupConfig(page, 25, window=window)]
    cm = CacheManager(groups, num_slots=4)
    model = Model(groups)
    next_id = 0
    for _ in range(300):
        action = rng.random()
        live = list(model.len)
        if action < 0.25 and len(live) < 4:
            rid = f"r{next_id}"
            next_id += 1
            cm.add_request(rid)
            model.len[rid] = 0
        elif action < 0.4 and live:
            rid = rng.choice(live)
            cm.free_request(rid)
            del model.len[rid]
        elif live:
            batch = rng.sample(live, rng.randint(1, len(live)))
            counts = [rng.choice([1, 1, 1, 2, 7, 33]) for _ in batch]
            before = [cm.free_pages(g) for g in range(2)]
            try:
                cm.reserve(batch, counts)
            except CacheExhausted:
                assert [cm.free_pages(g) for g in range(2)] == before
                continue
            idx = cm.fill_batch(batch, counts)
            for i, (rid, n) in enumerate(zip(batch, counts)):
                start = model.len[rid]
                rows = idx.positions[idx.qo_indptr[i]:idx.qo_indptr[i + 1]].tolist()
                assert rows == list(range(start, start + n))
                # every key the portion can see has a page
                for g, gc in enumerate(groups):
                    lo = 0 if gc.window is None else max(start - gc.window + 1, 0)
                    for key in range(lo, start + n):
                        assert idx.tables[g][i][key // gc.page_size] >= 0
                cm.commit(rid, n)
                model.len[rid] += n
        assert cm.check() == 0
        for g in range(2):
            held = sum(model.pages_held(r, g) for r in model.len)
            assert groups[g].num_pages - cm.free_pages(g) == held
        # no page id appears in two block tables
        for g in range(2):
            seen = [p for r in model.len for p in cm.block_table(r, g) if p >= 0]
            assert len(seen) == len(set(seen))
    for rid in list(model.len):
        cm.free_request(rid)
    assert cm.free_pages(0) == 40 and cm.free_pages(1) == 25 and cm.free_slots() == 4
    assert cm.check() == 0


def test_position_counter_is_kept_apart_from_the_length():
    """Positions advance with the cached length unless a commit says otherwise (the
    reference keeps position_id_start beside seq_len, mstar/engine/kv_store.py:112-116)."""
    cm = CacheManager([GroupConfig(page_size=4, num_pages=8)], num_slots=2)
    cm.add_request("a")
    cm.reserve(["a"], [5])
    cm.commit("a", 5)                                  # default: both by 5
    assert (cm.length("a"), cm.position("a")) == (5, 5)
    cm.reserve(["a"], [3])
    b = cm.fill_batch(["a"], [3])
    assert b.positions.tolist() == [5, 6, 7] and b.cache_pos.tolist() == [5, 6, 7]
    cm.commit("a", 3, pos_advance=1)                   # three keys, one position
    assert (cm.length("a"), cm.position("a")) == (8, 6)
    cm.reserve(["a"], [2])
    b = cm.fill_batch(["a"], [2])
    assert b.positions.tolist() == [6, 7] and b.cache_pos.tolist() == [8, 9]
    assert b.kv_len.tolist() == [10]
    cm.commit("a", 2)
    cm.set_position("a", 100)
    cm.reserve(["a"], [1])
    b = cm.fill_batch(["a"], [1])
    assert b.positions.tolist() == [100] and b.cache_pos.tolist() == [10]
    with pytest.raises(ValueError):
        cm.set_position("a", -1)
    with pytest.raises(ValueError):
        cm.commit("a", 1, pos_advance=-2)
    cm.free_request("a")
    cm.add_request("b")                                # a new request starts at zero again
    assert cm.position("b") == 0 and cm.check() == 0


def test_storage_gives_each_group_its_own_page_size():
    """Two groups (every key / a window of 6) with pages of 8 and of 2 tokens: tensors,
    block tables and the layer caches handed to mixers follow their group's size."""
    import torch

    from mstar_b200.cache.storage import CacheStorage
    from mstar_b200.parts.base import CacheNeed, KVNeed

    needs = [CacheNeed(kv=KVNeed(2, 16)), CacheNeed(kv=KVNeed(1, 32, window=6)),
             CacheNeed(kv=KVNeed(2, 16))]
    st_ = CacheStorage(needs, torch.float32, torch.device("cpu"), [8, 2], [5, 9], num_slots=2)
    assert st_.page_sizes == [8, 2] and st_.group_of == [0, 1, 0]
    assert [tuple(t.shape) for t in st_.kv] == [(6, 2, 2, 8, 16), (10, 2, 1, 2, 32),
                                                (6, 2, 2, 8, 16)]
    cm = st_.manager
    assert [g.page_size for g in cm.groups] == [8, 2]
    cm.add_request("a")
    cm.reserve(["a"], [11])
    assert len(cm.block_table("a", 0)) == 2 and len(cm.block_table("a", 1)) == 6
    idx = cm.fill_batch(["a"], [11])
    tables = [torch.from_numpy(t) for t in idx.tables]
    assert st_.layer_cache(0, tables).page_size == 8
    assert st_.layer_cache(1, tables).page_size == 2
    assert st_.layer_cache(1, tables).block_table.shape == (1, 6)
    cm.commit("a", 11)                                 # the window has passed keys 0..5
    assert cm.block_table("a", 1)[:3] == [-1, -1, -1] and cm.check() == 0
    with pytest.raises(ValueError):
        CacheStorage(needs, torch.float32, torch.device("cpu"), [8, 2, 4], 5, num_slots=2)
