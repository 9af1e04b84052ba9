"""Bookkeeping of pages and slots (no GPU): no page lost, held twice or freed
twice, under random orders of requests; windows give pages back early."""
import numpy as np
import pytest
import torch

from gibbs_b200.cache import CacheManager, IdPool, OutOfPages, OutOfSlots, PoolError
from gibbs_b200.parts.base import PagedKV, SlotState


def test_id_pool():
    p = IdPool(3, "page")
    a, b, c = p.take(), p.take(), p.take()
    assert sorted([a, b, c]) == [0, 1, 2] and p.take() is None and p.take_many(1) is None
    p.give_back(b)
    with pytest.raises(PoolError, match="twice"):
        p.give_back(b)
    with pytest.raises(PoolError, match="outside"):
        p.give_back(7)
    assert p.take() == b                      # given back last, handed out first
    p.check()
    assert p.n_free == 0 and p.n_used == 3


def _manager(n_pages=8, page_size=4, n_slots=3, window=None, max_context=64):
    needs = [([SlotState((2, 5))], None), ([PagedKV(2, 4, window)], None), ([SlotState((3,), torch.float32)], None),
             ([PagedKV(1, 8, window)], None), ([], 1)]
    return CacheManager(needs, n_pages, page_size, n_slots, torch.float32, "cpu", max_context)


def test_layout_groups_and_views():
    m = _manager()
    assert len(m.groups) == 1 and m.groups[0].entries == [(1, 0), (3, 0)]
    assert m.kv_bytes_per_token() == 2 * (2 * 4 + 1 * 8) * 4
    rc = m.open("a")
    m.reserve(rc, 6)
    m.advance(rc, 6)
    bt = torch.full((1, 1, m.max_blocks), -7, dtype=torch.int32).numpy()
    m.fill_block_tables([rc], bt)
    assert list(bt[0, 0, :3]) == rc.block_tables[0] + [-1] and len(rc.block_tables[0]) == 2
    views = m.views([torch.from_numpy(bt[0])], torch.tensor([rc.slot], dtype=torch.int32), [rc.slot])
    assert views[1][0].k_pages.shape == (8, 2, 4, 4) and views[3][0].v_pages.shape == (8, 1, 4, 8)
    assert views[4][0].k_pages is views[1][0].k_pages and not views[4][0].writable and views[1][0].writable
    assert views[0][0].state.shape == (3, 2, 5) and views[2][0].state.shape == (3, 3)
    # slot states of different entries do not overlap
    views[0][0].state[rc.slot].fill_(1.0)
    assert float(views[2][0].state.abs().sum()) == 0.0
    m.close("a")
    m.check()


def test_slot_is_zeroed_when_taken_again():
    m = _manager(n_slots=1)
    rc = m.open("a")
    m._slot_views[(0, 0)][rc.slot].fill_(3.0)
    m.close("a")
    rc = m.open("b")
    assert float(m._slot_views[(0, 0)][rc.slot].abs().sum()) == 0.0
    with pytest.raises(OutOfSlots):
        m.open("c")
    with pytest.raises(PoolError, match="already live"):
        m.open("b")
    m.close("b")
    with pytest.raises(PoolError, match="not live"):
        m.close("b")


def test_out_of_pages_takes_nothing():
    m = _manager(n_pages=3, page_size=4)
    a, b = m.open("a"), m.open("b")
    m.reserve(a, 8)
    assert m.free_pages() == [1] and m.can_reserve(b, 4) and not m.can_reserve(b, 5)
    with pytest.raises(OutOfPages):
        m.reserve(b, 9)
    assert m.free_pages() == [1] and b.block_tables == [[]]
    with pytest.raises(ValueError, match="laid out"):
        m.reserve(a, 65)
    m.check()


def test_window_gives_pages_back_and_they_are_reused():
    m = _manager(n_pages=4, page_size=4, window=6, max_context=400)
    rc = m.open("w")
    seen = set()
    for length in range(1, 200):
        m.reserve(rc, length)
        m.advance(rc, length)
        held = [p for p in rc.block_tables[0] if p >= 0]
        seen.update(held)
        # the window of 6 spans at most 3 pages of 4; a fourth is never needed
        assert len(held) <= 3
        # every key the next query may read is still there
        for pos in range(max(0, length - 6), length):
            assert rc.block_tables[0][pos // 4] >= 0
        m.check()
    assert seen == {0, 1, 2} or len(seen) <= 4
    m.close("w")
    assert m.free_pages() == [4]


@pytest.mark.parametrize("seed", range(5))
def test_random_orders_of_requests(seed):
    rng = np.random.default_rng(seed)
    m = _manager(n_pages=12, page_size=4, n_slots=4, window=None if seed % 2 else 9, max_context=80)
    live, next_id = {}, 0
    for _ in range(400):
        r = rng.random()
        if r < 0.25 and len(live) < 4:
            live[next_id] = m.open(next_id)
            next_id += 1
        elif r < 0.85 and live:
            rid = int(rng.choice(list(live)))
            rc = live[rid]
            grow = int(rng.integers(1, 12))
            if rc.length + grow <= 80 and m.can_reserve(rc, rc.length + grow):
                m.reserve(rc, rc.length + grow)
                m.advance(rc, rc.length + grow)
            elif rc.length + grow <= 80:
                before = (m.free_pages(), [list(t) for t in rc.block_tables])
                with pytest.raises(OutOfPages):
                    m.reserve(rc, rc.length + grow)
                assert before == (m.free_pages(), rc.block_tables)
        elif live:
            rid = int(rng.choice(list(live)))
            m.close(rid)
            del live[rid]
        m.check()
        held = sum(1 for rc in live.values() for p in rc.block_tables[0] if p >= 0)
        assert held + m.free_pages()[0] == 12
    for rid in list(live):
        m.close(rid)
    m.check()
    assert m.free_pages() == [12] and m.slots.n_free == 4


def test_windowed_requests_on_an_exactly_full_pool_reserve_all_or_nothing():
    """Two windowed requests fill the pool to the last page.  Their next step fits only because
    each gives back the page its window has passed; a step's requests are reserved together
    (every give-back before any take), so the order of the entries does not matter and a step
    that does not fit takes nothing."""
    m = _manager(n_pages=4, page_size=4, window=4, max_context=64)
    a, b = m.open("a"), m.open("b")
    m.reserve_all([(a, 8), (b, 8)])
    m.advance(a, 8), m.advance(b, 8)
    assert m.free_pages() == [0]
    # positions 8..11 need a third page each; page 0 of each request (positions 0..3) has left the window
    assert m.can_reserve_all([(a, 12), (b, 12)]) and m.can_reserve_all([(b, 12), (a, 12)])
    before = ([list(t) for t in a.block_tables], [list(t) for t in b.block_tables])
    # a step that does not fit (b would need two more pages) changes nothing
    assert not m.can_reserve_all([(a, 12), (b, 16)])
    with pytest.raises(OutOfPages):
        m.reserve_all([(a, 12), (b, 16)])
    assert ([list(t) for t in a.block_tables], [list(t) for t in b.block_tables]) == before and m.free_pages() == [0]
    m.check()
    m.reserve_all([(b, 12), (a, 12)])
    assert a.block_tables[0][0] == -1 and b.block_tables[0][0] == -1 and m.free_pages() == [0]
    m.check()
    # a step that is not run gives back what it took; pages the window had passed stay given back
    m.unreserve(a)
    assert len(a.block_tables[0]) == 2 and m.free_pages() == [1]
    m.check()
    m.close("a"), m.close("b")
    m.check()
    assert m.free_pages() == [4]


def test_values_may_be_narrower_or_wider_than_keys():
    """A mixer may keep values of another width than its keys: the two page tensors of an entry
    then differ in their last axis and are indexed by the same page ids."""
    needs = [([PagedKV(2, 8, None, v_head_dim=12)], None), ([PagedKV(1, 16)], None)]
    m = CacheManager(needs, 6, 4, 2, torch.float32, "cpu", 32)
    assert len(m.groups) == 1
    rc = m.open("a")
    m.reserve(rc, 9)
    views = m.views([torch.zeros(1, m.max_blocks, dtype=torch.int32)], torch.zeros(1, dtype=torch.int32), [0])
    assert views[0][0].k_pages.shape == (6, 2, 4, 8) and views[0][0].v_pages.shape == (6, 2, 4, 12)
    assert views[1][0].k_pages.shape == views[1][0].v_pages.shape == (6, 1, 4, 16)
    assert m.kv_bytes_per_token() == (2 * (8 + 12) + 1 * (16 + 16)) * 4
    m.close("a")
    m.check()


def test_guards_catch_a_write_outside_a_page_or_a_slot():
    m = CacheManager([([PagedKV(1, 4)], None), ([SlotState((3,))], None)], 4, 2, 2, torch.float32, "cpu", 16,
                     guard=True)
    rc = m.open("a")
    m.reserve(rc, 3)
    kp, vp = m._pages[(0, 0)]
    assert kp.shape == (4, 1, 2, 4) and kp.is_contiguous()
    kp.fill_(1.0), vp.fill_(2.0)                       # everything inside the pages may be written
    m._slot_views[(1, 0)].fill_(3.0)
    m.check()
    flat = kp.view(-1)
    flat.as_strided((1,), (1,), flat.storage_offset() + flat.numel())[0] = 9.0     # one element past the last page
    with pytest.raises(PoolError, match="guard"):
        m.check()
    m2 = CacheManager([([SlotState((3,))], None)], 1, 2, 2, torch.float32, "cpu", 16, guard=True)
    view = m2._slot_views[(0, 0)]
    assert view.shape == (2, 3) and view.stride(0) > 3                            # guard bytes behind every slot
    view.as_strided((1,), (1,), view.storage_offset() + 4)[0] = 1.0               # one float behind slot 0 (its 12 bytes are padded to 16)
    with pytest.raises(PoolError, match="guard"):
        m2.check()
