"""Host page bookkeeping against the reference's own expectations
(sdk/javascript/__test__/kv-page-manager.ts and runtime/src/utils.rs IdPool semantics)."""
import numpy as np
import pytest
import torch

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


# ---- the native (C++) manager: same id rules as IdPool, plus the reference's ownership / OOM / export rules
def test_native_manager_ids_follow_the_python_pool():
    from pie_b200.pages import NativePageManager
    rng = np.random.default_rng(0)
    nat, py = NativePageManager(3000), PagePool(3000)
    held = []
    for step in range(400):
        if held and rng.random() < 0.45:
            k = int(rng.integers(1, min(len(held), 40) + 1))
            idx = sorted(rng.choice(len(held), size=k, replace=False).tolist(), reverse=True)
            drop = [held.pop(i) for i in idx]
            nat.free(1, drop)
            py.release(drop)
        else:
            k = int(rng.integers(1, 60))
            if py.available() < k:
                continue
            a, victims = nat.alloc(1, k)
            b = py.alloc(k)
            assert a == b and victims == []
            held += a
        assert nat.available() == py.available()
    # tail compaction: > 1000 free ids forming the tail fold back, the next id is the smallest again
    nat.free(1, held)
    py.release(held)
    assert nat.available() == py.available() == 3000
    assert nat.alloc(1, 3)[0] == py.alloc(3) == [0, 1, 2]
    nat.close()


def test_native_manager_oom_terminates_newer_instances_newest_first():
    from pie_b200.pages import NativePageManager
    m = NativePageManager(10)
    old, _ = m.alloc(100, 4)      # instance 100 starts first
    mid, _ = m.alloc(200, 3)
    new, _ = m.alloc(300, 3)
    assert m.available() == 0
    # the oldest asks for 5 more: 300 (newest) goes first, then 200; 100 itself is never a victim
    pages, victims = m.alloc(100, 5)
    assert victims == [300, 200] and m.owned(300) == 0 and m.owned(200) == 0 and m.owned(100) == 9
    assert sorted(pages) == sorted(new + mid)[:5]
    # a newer instance cannot evict an older one (resource.rs:262-275): the request fails, nothing changes
    m.alloc(400, 1)
    with pytest.raises(PoolExhausted):
        m.alloc(400, 5)
    assert m.owned(100) == 9 and m.owned(400) == 1
    # an instance without a start time cannot trigger the policy at all
    with pytest.raises(PoolExhausted):
        m.alloc(500, 3)
    m.close()


def test_native_manager_share_export_import():
    from pie_b200.pages import NativePageManager
    m = NativePageManager(8)
    a, _ = m.alloc(1, 3)
    m.share(2, a[:2])                       # a fork keeps the two full pages in common
    assert [m.refcount(p) for p in a] == [2, 2, 1]
    m.cleanup(1)                            # the parent goes away: shared pages stay, its private page returns
    assert [m.refcount(p) for p in a] == [1, 1, 0] and m.available() == 6
    m.export(2, a[:2], "prefix")
    assert m.owned(2) == 0 and m.import_("prefix") == a[:2]
    with pytest.raises(ValueError):
        m.export(2, a[:1], "prefix")        # not held any more / name exists
    with pytest.raises(KeyError):
        m.import_("nope")
    m.cleanup(2)
    assert m.available() == 6               # exported pages survive their exporter
    m.release_exported("prefix")
    assert m.available() == 8
    with pytest.raises(ValueError):
        m.share(3, [7])                     # not allocated
    with pytest.raises(ValueError):
        m.free(3, [])                       # an instance that holds nothing (InstanceNotAllocated in the reference)
    m.close()


def test_native_export_rejects_a_page_listed_twice():
    """A duplicate in an export list would be released twice and drop a co-holder's reference."""
    from pie_b200.pages import NativePageManager
    m = NativePageManager(8)
    a, _ = m.alloc(1, 2)
    p = a[0]
    m.share(2, [p])
    assert m.refcount(p) == 2
    with pytest.raises(ValueError):
        m.export(1, [p, p], "dup")
    assert m.refcount(p) == 2 and m.owned(1) == 2  # nothing moved
    m.export(1, [p], "once")
    m.release_exported("once")
    assert m.refcount(p) == 1                     # instance 2 still holds it
    got, _ = m.alloc(3, 6)
    assert p not in got                           # and it is not handed out again
    m.close()


def test_drop_masked_kv_pages_follows_the_context_rule():
    """Full pages whose tokens are all masked go back to the pool, newest first; a partial last page stays
    (sdk/rust/inferlet/src/context.rs:298-345)."""
    pool = PagePool(16)
    ctx = KvPageList(pool, 4)
    ctx.grow(4 * 5 + 2)  # five full pages and a partial one
    pages = list(ctx.pages)
    masked = np.zeros(22, dtype=bool)
    masked[4:12] = True    # pages 1 and 2 entirely
    masked[12:15] = True   # page 3 all but one token
    masked[20:22] = True   # the partial page, entirely - not a candidate
    before = pool.available()
    dropped = ctx.drop_masked_kv_pages(masked)
    assert dropped == [2, 1]
    assert ctx.pages == [pages[0], pages[3], pages[4], pages[5]]
    assert ctx.total_tokens == 14 and ctx.last_page_len == 2
    assert pool.available() == before + 2
    # a context of full pages that loses its last page, then everything
    full = KvPageList(pool, 4)
    full.grow(8)
    assert full.drop_masked_kv_pages([False] * 4 + [True] * 4) == [1]
    assert full.total_tokens == 4 and full.last_page_len == 4
    assert full.drop_masked_kv_pages([True] * 4) == [0]
    assert full.total_tokens == 0 and full.last_page_len == 0 and full.pages == []
    with pytest.raises(ValueError):
        ctx.drop_masked_kv_pages([True] * 3)


def test_pool_sizing_follows_the_reference_formula():
    """pie/src/pie_worker/model/llama3.py:177-202: usable bytes over the bytes of a page across all layers, KV
    heads divided over the tensor-parallel ranks."""
    from pie_b200.pages import eval_max_num_kv_pages

    free = 100 * 2 ** 30
    per_page = 2 * 2 * 16 * 8 * 128 * 32  # bf16, K+V, 16 tokens, 8 kv heads, D 128, 32 layers
    assert eval_max_num_kv_pages(free, 0.9, 16, 8, 128, 32, torch.bfloat16) == int(free * 0.9 // per_page)
    assert eval_max_num_kv_pages(free, 0.9, 16, 8, 128, 32, torch.bfloat16, tensor_parallel_size=4) == \
        int(free * 0.9 // (per_page // 4))
    assert eval_max_num_kv_pages(free, 0.5, 16, 8, 128, 32, torch.float32) == int(free * 0.5 // (per_page * 2))
