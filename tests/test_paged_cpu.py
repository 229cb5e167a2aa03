"""The page pool and the prefix tree (host bookkeeping, no device): holders counted, the lowest free page first, the
longest chain of whole pages matched, least-recently-used leaves evicted first and never a page a conversation holds."""

import pytest

from btb_b200.paged import PAGE, PagePool, PoolError, PrefixTree


def test_pool_counts_holders_and_hands_out_the_lowest_free_page():
    pool = PagePool(4)
    a, b = pool.alloc(), pool.alloc()
    assert (a.id, b.id) == (0, 1) and len(pool) == 2
    pool.ref(a)
    assert not pool.unref(a) and pool.unref(a)  # the second holder's release frees it
    assert pool.alloc().id == 0  # the lowest free page again
    with pytest.raises(PoolError):
        pool.unref(pool.pages[3])
    pool.alloc(), pool.alloc()
    with pytest.raises(PoolError):
        pool.alloc()
    assert pool.check() == []


def test_tree_matches_whole_pages_and_evicts_unheld_leaves_oldest_first():
    pool = PagePool(8)
    tree = PrefixTree(pool)
    ids = list(range(3 * PAGE + 10))
    node, pages = tree.root, []
    for i in range(3):
        p = pool.alloc()
        pages.append(p)
        node = tree.insert(node, tuple(ids[i * PAGE : (i + 1) * PAGE]), p)
    assert len(tree) == 3 and all(p.refs == 2 for p in pages)
    assert [n.page.id for n in tree.match(ids)] == [0, 1, 2]
    assert [n.page.id for n in tree.match(ids[: 2 * PAGE + 63])] == [0, 1]  # a partial page matches nothing
    other = ids[:PAGE] + [7] * PAGE
    assert [n.page.id for n in tree.match(other)] == [0]
    # an equal page computed twice: the first one stays the tree's
    dup = pool.alloc()
    assert tree.insert(tree.root, tuple(ids[:PAGE]), dup).page is pages[0] and dup.refs == 1
    # the conversation lets go: the tree alone holds the chain; eviction takes the leaf (the deepest page) first
    for p in pages:
        pool.unref(p)
    assert tree.evict(1) == 1 and len(tree) == 2 and pages[2].refs == 0
    pool.ref(pages[1])  # held by a conversation again: not evictable, and neither is its ancestor (not a leaf)
    assert tree.evict(5) == 0
    pool.unref(pages[1])
    assert tree.evict(5) == 2 and len(tree) == 0
    pool.unref(dup)
    assert pool.check() == [] and len(pool) == 0
