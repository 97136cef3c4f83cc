"""Host page bookkeeping against the reference's own expectations
(sdk/javascript/__test__/kv-page-manager.ts and runtime/src/utils.rs IdPool semantics)."""
import numpy as np
import pytest

from pie_b200.pages import IdPool, KvPageList, PagePool, PoolExhausted, build_csr


def test_id_pool_smallest_first_and_reuse():
    p = IdPool(4)
    assert [p.acquire() for _ in range(4)] == [0, 1, 2, 3]
    with pytest.raises(PoolExhausted):
        p.acquire()
    p.release(2)
    p.release(0)
    assert p.available() == 2
    assert p.acquire() == 0 and p.acquire() == 2
    with pytest.raises(ValueError):
        IdPool(4).release(0)  # never allocated
    with pytest.raises(PoolExhausted):
        IdPool(2).acquire_many(3)


def test_id_pool_tail_compaction():
    p = IdPool(5000)
    ids = p.acquire_many(3000)
    p.release_many(ids[1500:])  # > 1000 free ids and they form the tail
    assert p._next == 1500 and len(p._free) == 0
    assert p.available() == 3500
    assert p.acquire() == 1500
    with pytest.raises(ValueError):
        p.set_capacity(10)


# the cases of sdk/javascript/__test__/kv-page-manager.ts, page size 128
def test_grow_shrink_like_reference_manager():
    pool = PagePool(16)
    m = KvPageList(pool, 128)
    assert (m.page_count, m.last_page_len, m.total_tokens) == (0, 0, 0)
    m.grow(100)
    assert (m.page_count, m.last_page_len) == (1, 100)
    m2 = KvPageList(pool, 128)
    m2.grow(200)
    assert (m2.page_count, m2.last_page_len, m2.total_tokens) == (2, 72, 200)
    second = m2.pages[1]
    m2.shrink(100)
    assert (m2.page_count, m2.total_tokens, m2.last_page_len) == (1, 100, 100)
    assert pool.refs[second] == 0
    m2.shrink(100)
    assert (m2.page_count, m2.total_tokens) == (0, 0)
    with pytest.raises(ValueError, match="underflow"):
        KvPageList(pool, 128).shrink(10)
    m3 = KvPageList(pool, 128)
    m3.grow(256)
    assert (m3.page_count, m3.last_page_len) == (2, 128)  # an exactly full last page reports page_size


def test_fork_shares_only_full_pages():
    pool = PagePool(16)
    m = KvPageList(pool, 128)
    m.grow(200)
    child, dropped = m.fork()
    assert (child.page_count, child.total_tokens, dropped) == (1, 128, 72)
    assert pool.refs[m.pages[0]] == 2 and pool.refs[m.pages[1]] == 1
    only_partial = KvPageList(pool, 128)
    only_partial.grow(50)
    c2, d2 = only_partial.fork()
    assert (c2.page_count, c2.total_tokens, d2) == (0, 0, 50)


def test_fork_cow_and_release():
    pool = PagePool(16)
    m = KvPageList(pool, 16)
    m.grow(40)  # pages: 16, 16, 8
    child, copy = m.fork_cow()
    src, dst, valid = copy
    assert src == m.pages[-1] and dst == child.pages[-1] and valid == 8 and dst != src
    assert child.pages[:-1] == m.pages[:-1] and child.total_tokens == 40
    full = KvPageList(pool, 16)
    full.grow(32)
    c2, copy2 = full.fork_cow()
    assert copy2 is None and c2.pages == full.pages
    freed = child.release()
    assert freed == [dst]  # shared pages stay alive
    assert sorted(m.release()) == sorted([0, 1, 2])
    winner = KvPageList(pool, 16)
    winner.adopt(full)
    assert winner.pages == full.pages and all(pool.refs[p] == 3 for p in full.pages)


def test_remove_page_and_csr():
    pool = PagePool(32)
    a, b = KvPageList(pool, 16), KvPageList(pool, 16)
    a.grow(40)
    b.grow(16)
    a.remove_page_at(0)
    assert a.total_tokens == 24 and a.last_page_len == 8
    idx, ptr, last = build_csr([a, b, KvPageList(pool, 16)])
    assert ptr.tolist() == [0, 2, 3, 3] and last.tolist() == [8, 16, 0]
    assert idx.tolist() == a.pages + b.pages and idx.dtype == np.int32
