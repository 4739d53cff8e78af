"""Host-side bookkeeping of the paged key / value cache (no GPU): the page allocator."""
import pytest

from pope_pytorch_b200.kv_cache import PageAllocator


def test_pages_are_mapped_in_logical_order_and_only_when_needed():
    al = PageAllocator(batch=2, num_pages=8, page_size=64, max_pages_per_seq=4)
    new = al.reserve(100)                                   # two pages per sequence
    assert [(b, lp) for b, lp, _ in new] == [(0, 0), (0, 1), (1, 0), (1, 1)]
    assert sorted(pg for _, _, pg in new) == [0, 1, 2, 3]
    al.advance(100)
    assert al.lens == [100, 100] and al.reserve(28) == []   # 128 keys still fit the two pages
    al.advance(28)
    new = al.reserve(1)                                     # key 128 opens the third page
    assert [(b, lp) for b, lp, _ in new] == [(0, 2), (1, 2)]
    al.advance(1)
    assert al.lens == [129, 129] and len(al.free) == 2


def test_ragged_rows_release_and_reuse():
    al = PageAllocator(batch=3, num_pages=6, page_size=64, max_pages_per_seq=6)
    al.reserve(200, rows=[1]); al.advance(200, rows=[1])    # 4 pages to sequence 1
    al.reserve(10, rows=[0]); al.advance(10, rows=[0])
    assert al.lens == [10, 200, 0] and len(al.free) == 1
    held = list(al.table[1])
    al.release(1)
    assert al.lens[1] == 0 and al.table[1] == [] and len(al.free) == 5
    new = al.reserve(64, rows=[2])
    assert new[0][2] == held[0]                             # the pages of the released sequence are handed out again


def test_failures_change_nothing():
    al = PageAllocator(batch=2, num_pages=3, page_size=64, max_pages_per_seq=2)
    with pytest.raises(RuntimeError, match="out of pages"):
        al.reserve(128)                                     # 4 pages wanted, 3 in the pool
    assert al.table == [[], []] and len(al.free) == 3
    al = PageAllocator(batch=2, num_pages=8, page_size=64, max_pages_per_seq=2)
    al.reserve(64); al.advance(64)
    with pytest.raises(RuntimeError, match="max_pages_per_seq"):
        al.reserve(128, rows=[0])                           # would be 3 logical pages
    assert len(al.table[0]) == 1 and len(al.free) == 6
    with pytest.raises(ValueError):
        PageAllocator(1, 1, 100, 1)
