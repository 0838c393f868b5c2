"""Host-side bookkeeping of the serving scheduler (rustgrad_b200/serving.py) without a device:
the prefix cache follows PrefixCache of src/models/transformer/serving/mod.rs:192-352."""
import numpy as np

from rustgrad_b200 import serving


class FakeSnapshot:
    def __init__(self, length, nbytes=1000):
        self.length, self.bytes = length, nbytes


def logits():
    return np.zeros(10, dtype=np.float32)


def entry_bytes(tokens, nbytes=1000):
    return nbytes + 10 * 4 + len(tokens) * 4


def test_longest_prefix_wins_and_counts_hits_and_misses():
    c = serving._PrefixCache(8, 1 << 20)
    assert c.longest([1, 2, 3]) is None and c.stats()["misses"] == 1
    assert c.insert([1, 2], FakeSnapshot(2), logits()) and c.insert([1, 2, 3, 4], FakeSnapshot(4), logits())
    assert c.insert([9], FakeSnapshot(1), logits())
    key, snap, _ = c.longest([1, 2, 3, 4, 5])
    assert key == (1, 2, 3, 4) and snap.length == 4
    key, snap, _ = c.longest([1, 2, 7])
    assert key == (1, 2)
    assert c.longest([2, 1]) is None
    st = c.stats()
    assert (st["entries"], st["hits"], st["misses"]) == (3, 2, 2)
    assert st["bytes"] == entry_bytes([1, 2]) + entry_bytes([1, 2, 3, 4]) + entry_bytes([9])


def test_eviction_is_least_recently_used_and_spares_referenced_entries():
    c = serving._PrefixCache(2, 1 << 20)
    c.insert([1], FakeSnapshot(1), logits())
    c.insert([2], FakeSnapshot(1), logits())
    c.longest([1, 5])                      # touches and leases [1]
    assert c.insert([3], FakeSnapshot(1), logits())
    assert set(c.entries) == {(1,), (3,)} and c.stats()["evictions"] == 1   # [2] was the oldest unreferenced
    c.longest([3, 5])                      # both entries leased now
    assert not c.insert([4], FakeSnapshot(1), logits())                    # nothing may be evicted
    c.release((1,))
    assert c.insert([4], FakeSnapshot(1), logits()) and set(c.entries) == {(3,), (4,)}
    # re-inserting a key replaces it without eviction
    before = c.stats()["evictions"]
    assert c.insert([4], FakeSnapshot(1, 500), logits()) and c.stats()["evictions"] == before
    assert c.stats()["bytes"] == entry_bytes([3]) + entry_bytes([4], 500)


def test_budgets_and_invalidation():
    assert not serving._PrefixCache(0, 1 << 20).insert([1], FakeSnapshot(1), logits())
    assert not serving._PrefixCache(4, 0).insert([1], FakeSnapshot(1), logits())
    c = serving._PrefixCache(4, 1500)
    assert not c.insert([1], FakeSnapshot(1, 2000), logits())              # larger than the whole budget
    assert c.insert([1], FakeSnapshot(1), logits())
    assert c.insert([2], FakeSnapshot(1), logits()) and set(c.entries) == {(2,)}  # byte budget evicts
    c.invalidate()
    st = c.stats()
    assert (st["entries"], st["bytes"], st["generation"]) == (0, 0, 1)
    c.entries[(7,)] = serving._Entry(0, FakeSnapshot(1), logits(), 10, 0)  # an entry of the old generation
    c.bytes = 10
    assert c.longest([7, 8]) is None
    st = c.stats()
    assert (st["stale_rejections"], st["entries"], st["bytes"]) == (1, 0, 0)
