"""Cache manager: no page lost, held twice or freed twice, under random orders (no GPU)."""
import random

import pytest
import torch

from poor_mans_mamba_b200.cache import CacheManager, OutOfPages, PageAccountingError, PagePool
from poor_mans_mamba_b200.parts.base import StateSpec


def specs(window=0, layers=3):
    out = {}
    for l in range(layers):
        s = [("attn.kv", StateSpec.paged("kv", 2, 8)), ("ssm.state", StateSpec.fixed("state", (2, 3), "float32")),
             ("ssm.conv", StateSpec.fixed("conv", (3, 5), "float32"))]
        if window and l == 1:
            s[0] = ("attn.kv", StateSpec.paged("kv", 2, 8, window=window))
        out[l] = s
    return out


def make(window=0, num_pages=6, num_slots=3, page_size=4):
    return CacheManager(specs(window), page_size=page_size, num_pages=num_pages, num_slots=num_slots,
                        dtype=torch.float32, device="cpu")


def test_page_pool_discipline():
    p = PagePool(3)
    a, b = p.alloc("x"), p.alloc("y")
    assert (a, b) == (0, 1) and p.n_free == 1
    p.free(a, "x")
    with pytest.raises(PageAccountingError, match="twice"):
        p.free(a, "x")
    with pytest.raises(PageAccountingError, match="held by"):
        p.free(b, "x")
    assert p.alloc("z") == a  # the page just given back is used again first
    p.alloc("z")
    with pytest.raises(OutOfPages):
        p.alloc("z")
    p.check()


def test_groups_by_layout_and_window():
    c = make(window=6)
    assert len(c.groups) == 2
    full = c.groups[(2, 8, 0)]
    win = c.groups[(2, 8, 6)]
    assert [m.layer for m in full.members] == [0, 2] and [m.layer for m in win.members] == [1]
    assert full.storage.shape == (2, 7, 2, 4, 8)  # one spare page
    caches = c.layer_caches({k: torch.zeros(1, 1, dtype=torch.int32) for k in c.groups})
    assert caches[1].paged("attn.kv").window == 6 and caches[0].paged("attn.kv").window == 0
    assert caches[2].fixed("ssm.state").shape == (4, 2, 3)  # one spare slot


def test_grow_is_all_or_nothing_and_release_gives_back():
    c = make(num_pages=4)
    c.admit("a"), c.admit("b")
    c.grow("a", 9)  # 3 pages
    assert c.block_table("a", (2, 8, 0)) == [0, 1, 2] and c.min_free_pages() == 1
    assert c.pages_needed("b", 5) == {(2, 8, 0): 2} and not c.can_grow("b", 5)
    with pytest.raises(OutOfPages):
        c.grow("b", 5)
    assert c.block_table("b", (2, 8, 0)) == [] and c.min_free_pages() == 1
    c.grow("b", 4)
    c.check()
    c.release("a")
    assert c.min_free_pages() == 3
    c.grow("b", 13)
    assert c.block_table("b", (2, 8, 0)) == [3, 2, 1, 0]  # a's pages, last given back first
    with pytest.raises(KeyError):
        c.release("a")
    c.check()


def test_slots_run_out_and_are_zeroed_on_admit():
    c = make(num_slots=2)
    s = c.admit("a")
    c.admit("b")
    with pytest.raises(OutOfPages, match="slot"):
        c.admit("c")
    with pytest.raises(ValueError):
        c.admit("a")
    for t in c._fixed.values():
        t[s].fill_(7.0)
    c.release("a")
    assert c.admit("c") == s
    assert all(float(t[s].abs().sum()) == 0.0 for t in c._fixed.values())
    other = c.slot("b")
    assert all(float(t[other].abs().sum()) == 0.0 for t in c._fixed.values())
    c.check()


def test_fixed_states_of_one_kind_share_storage_and_stay_contiguous():
    """States of the same shape and dtype lie in one tensor [member, slot, *shape] (a request's slot
    is cleared with one fill per kind); each layer still sees a contiguous [slot, *shape] of its
    own, and clearing one request's slot leaves the other slots of every layer alone."""
    c = make(num_slots=3)
    assert len(c._fixed_stores) == 2  # (2, 3) and (3, 5), three layers each
    assert sorted(tuple(st.shape) for st in c._fixed_stores) == [(3, 4, 2, 3), (3, 4, 3, 5)]
    ptrs = set()
    for (layer, name), t in c._fixed.items():
        assert t.is_contiguous() and t.shape[0] == 4
        ptrs.add(t.data_ptr())
    assert len(ptrs) == 6
    a, b = c.admit("a"), c.admit("b")
    for k, t in enumerate(c._fixed.values()):
        t[a].fill_(1.0 + k)
        t[b].fill_(-1.0 - k)
    c.release("a")
    assert c.admit("again") == a
    for k, t in enumerate(c._fixed.values()):
        assert float(t[a].abs().sum()) == 0.0
        assert bool((t[b] == -1.0 - k).all())


def test_window_gives_pages_back_as_it_passes():
    c = make(window=6, num_pages=8)
    c.admit("a")
    win = c.groups[(2, 8, 6)]
    n = 0
    for step in range(30):
        c.grow("a", n + 1)
        n = c.advance("a", 1)
        held = [p for p in c.block_table("a", win.key) if p >= 0]
        # keys n-5..n are still readable by the next token: at most 3 pages of 4
        assert len(held) <= 3
        first_live = max(0, n - 6 + 1) // 4
        assert all(p == -1 for p in c.block_table("a", win.key)[:first_live])
        c.check()
    assert len([p for p in c.block_table("a", (2, 8, 0)) if p >= 0]) == 8  # the full group keeps all
    c.release("a")
    assert c.free_pages() == {(2, 8, 0): 8, (2, 8, 6): 8}


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_the_books(seed):
    rng = random.Random(seed)
    c = make(window=6 if seed % 2 else 0, num_pages=9, num_slots=4)
    live = {}
    next_id = 0
    for _ in range(400):
        op = rng.random()
        if op < 0.25 and c.free_slots:
            c.admit(next_id)
            live[next_id] = 0
            next_id += 1
        elif op < 0.8 and live:
            r = rng.choice(list(live))
            n = rng.choice([1, 1, 2, 5, 9])
            if c.can_grow(r, live[r] + n):
                c.grow(r, live[r] + n)
                live[r] = c.advance(r, n)
            else:
                with pytest.raises(OutOfPages):
                    c.grow(r, live[r] + n)
        elif live:
            r = rng.choice(list(live))
            c.release(r)
            del live[r]
        c.check()
        for g in c.groups.values():
            assert g.pool.n_free + sum(1 for t in g.tables.values() for p in t if p >= 0) == g.num_pages
    for r in list(live):
        c.release(r)
    c.check()
    assert all(n == 9 for n in c.free_pages().values()) and c.free_slots == 4
