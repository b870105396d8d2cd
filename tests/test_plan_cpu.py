"""Host-side planner of balanced launches (miniattn_plan_fwd): pure arithmetic, no device.

A plan cuts the K/V tile range of some work items into pieces for separate CTAs.  Whatever the
shape, the pieces of an item must tile its range exactly once, slots must be unique, and the plan
must only be used when its predicted makespan beats the plain launch.
"""
import collections

import pytest

from miniattn.ops import plan_info

SMS = 148


def item_tiles(item, B, Hq, Nq, Nk, causal, q_pos0=0, k_pos0=0, group=None):
    """K/V tiles of work item `item` (pair of 128-row Q tiles): heads walked in groups of `group`
    (all B*Hq at once by default), inside a group latest rows first, heads fastest."""
    n_pairs = ((Nq + 127) // 128 + 1) // 2
    group = group or B * Hq
    pair = n_pairs - 1 - (item % (n_pairs * group)) // group
    q0 = pair * 256
    nt = 2 if q0 + 128 < Nq else 1
    kv_end = Nk
    if causal:
        last_row = min(q0 + nt * 128 - 1, Nq - 1)
        kv_end = max(0, min(Nk, q_pos0 + last_row - k_pos0 + 1))
    return (kv_end + 127) // 128


CASES = [
    # B, Hq, Nq, Nk, D, causal, q_pos0, k_pos0
    (2, 8, 8192, 8192, 128, False, 0, 0),
    (2, 8, 4096, 4096, 128, False, 0, 0),
    (2, 8, 1024, 1024, 128, False, 0, 0),
    (1, 1, 8192, 8192, 128, False, 0, 0),
    (1, 4, 4096, 4096, 128, True, 0, 0),
    (1, 3, 1000, 5000, 64, True, 4000, 0),
    (1, 2, 900, 3000, 128, True, 0, 500),
    (3, 5, 2304, 1111, 64, False, 0, 0),
    (1, 16, 8192, 8192, 128, False, 0, 0),
]


@pytest.mark.parametrize("case", CASES)
def test_pieces_tile_every_item_once(case):
    B, Hq, Nq, Nk, D, causal, qp, kp = case
    info, pieces = plan_info(B, Hq, Nq, Nk, D, causal=causal, q_pos0=qp, k_pos0=kp, sm_count=SMS)
    n_items = (((Nq + 127) // 128 + 1) // 2) * B * Hq
    if not info.split:
        assert info.n_ctas == n_items and info.scratch_bytes == 0 and not pieces
        return
    assert info.n_ctas == info.n_whole + info.n_pieces == info.n_whole + len(pieces)
    by_item = collections.defaultdict(list)
    for item, t0, t1, part, nparts, slot in pieces:
        assert item >= info.n_whole, "an item of the whole prefix must not appear in the table"
        by_item[item].append((part, t0, t1, nparts, slot))
    assert sorted(by_item) == list(range(info.n_whole, n_items)), "every other item is in the table"
    slots = []
    cut = 0
    for item, lst in by_item.items():
        lst.sort()
        w = item_tiles(item, B, Hq, Nq, Nk, causal, qp, kp, info.head_group)
        assert [x[0] for x in lst] == list(range(len(lst)))
        assert all(x[3] == len(lst) for x in lst)
        assert lst[0][1] == 0 and lst[-1][2] == w, (item, lst, w)
        for a, b_ in zip(lst, lst[1:]):
            assert a[2] == b_[1], "pieces must be contiguous"
        if len(lst) > 1:
            cut += 1
            assert all(x[2] - x[1] >= 2 for x in lst), "no piece shorter than two K/V tiles"
            slots += [x[4] for x in lst]
            assert [x[4] for x in lst] == list(range(lst[0][4], lst[0][4] + len(lst))), "consecutive slots"
        else:
            assert lst[0][4] == -1
    assert cut == info.n_cut_items and sorted(slots) == list(range(info.n_slots))
    rows = info.n_slots * 2 * 128
    assert info.scratch_bytes == 16384 + ((rows * 8 + 255) // 256) * 256 + rows * D * 4
    assert info.est_balanced <= 0.97 * info.est_plain
    assert info.n_pieces <= 768


def test_headline_shapes_are_split_and_big_grids_are_not():
    assert plan_info(2, 8, 8192, 8192, sm_count=SMS)[0].split == 1      # 512 items: 3.46 rounds
    assert plan_info(2, 8, 4096, 4096, sm_count=SMS)[0].split == 1      # 256 items: 1.73 rounds
    assert plan_info(2, 8, 2048, 2048, sm_count=SMS)[0].split == 0      # 128 items in one round
    assert plan_info(4, 32, 4096, 4096, causal=True, sm_count=SMS)[0].split == 0   # 2048 items
    assert plan_info(1, 32, 131072, 131072, causal=True, sm_count=SMS)[0].split == 0
    info, _ = plan_info(2, 8, 8192, 8192, sm_count=SMS)
    assert info.n_whole == 444 and info.n_cut_items == 68   # three whole rounds, the rest is cut


def test_plan_is_deterministic_and_depends_on_sm_count():
    a = plan_info(2, 8, 4096, 4096, sm_count=SMS)
    b = plan_info(2, 8, 4096, 4096, sm_count=SMS)
    assert a[1] == b[1] and a[0].n_slots == b[0].n_slots
    c = plan_info(2, 8, 4096, 4096, sm_count=128)   # 256 items on 128 SMs: two full rounds
    assert c[0].split == 0


def test_empty_and_degenerate_shapes():
    assert plan_info(0, 8, 512, 512, sm_count=SMS)[0].split == 0
    assert plan_info(2, 8, 512, 0, sm_count=SMS)[0].split == 0
    info, _ = plan_info(1, 1, 128, 128, sm_count=SMS)      # one item, one K/V tile: nothing to cut
    assert info.split == 0 and info.n_ctas == 1


def test_random_shapes_keep_the_invariants():
    """Seeded sweep over shapes, masks, offsets and SM counts: whatever the planner decides, the
    pieces it hands out must tile every item exactly once."""
    import random
    rng = random.Random(7)
    n_split = 0
    for _ in range(120):
        B, Hq = rng.randint(1, 3), rng.randint(1, 12)
        Nq, Nk = rng.randint(1, 40) * rng.choice([100, 128, 256]), rng.randint(1, 60) * rng.choice([100, 128])
        D = rng.choice([64, 128])
        causal = rng.random() < 0.5
        qp = rng.choice([0, 0, max(0, Nk - Nq), rng.randint(0, 3000)]) if causal else 0
        kp = rng.choice([0, 0, rng.randint(0, 500)]) if causal else 0
        sms = rng.choice([148, 132, 64, 16])
        info, pieces = plan_info(B, Hq, Nq, Nk, D, causal=causal, q_pos0=qp, k_pos0=kp, sm_count=sms)
        n_items = (((Nq + 127) // 128 + 1) // 2) * B * Hq
        if not info.split:
            assert info.n_ctas == n_items
            continue
        n_split += 1
        cover = collections.defaultdict(list)
        for item, t0, t1, part, nparts, slot in pieces:
            assert info.n_whole <= item < n_items and 0 <= t0 <= t1
            cover[item].append((t0, t1, nparts, slot))
        assert len(cover) == n_items - info.n_whole
        for item, lst in cover.items():
            lst.sort()
            w = item_tiles(item, B, Hq, Nq, Nk, causal, qp, kp, info.head_group)
            assert lst[0][0] == 0 and lst[-1][1] == w and all(a[1] == b_[0] for a, b_ in zip(lst, lst[1:]))
            assert all(x[2] == len(lst) for x in lst)
            assert all((x[3] >= 0) == (len(lst) > 1) for x in lst)
        assert info.est_balanced <= 0.97 * info.est_plain
    assert n_split >= 20, "the sweep must exercise the cutting path"


def test_plan_entry_rejects_bad_arguments():
    import ctypes as C
    from miniattn import _lib
    p = _lib.FwdParams()
    p.B, p.Hq, p.Hkv, p.Nq, p.Nk, p.D = 1, 1, 1, 128, 128, 80
    info = _lib.PlanInfo()
    assert _lib.lib.miniattn_plan_fwd(C.byref(p), 148, C.byref(info), None, 0) == _lib.EUNSUPPORTED
    p.D = 128
    assert _lib.lib.miniattn_plan_fwd(C.byref(p), 148, None, None, 0) == _lib.EINVAL
    p.Nq = -1
    assert _lib.lib.miniattn_plan_fwd(C.byref(p), 148, C.byref(info), None, 0) == _lib.EINVAL
