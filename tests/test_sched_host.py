"""The split-KV planner's arithmetic, through dsv4_attn_plan_host (the planner kernel's host twin:
same functions, serial).  No GPU needed.  Checked: every (row, head group) is covered exactly once by
its pieces, piece counts and partial slots are consistent, the shares of the block pairs are balanced,
a fixed split count is honoured, capacities reported by dsv4_attn_sched_bytes are enough."""
import ctypes as C

import numpy as np
import pytest

from dsv4_attn_b200 import _lib

TILE = 64
TILE_COST, FIXED = 32, 48      # the planner's cost units: a tile, and the fixed part of an item
PAIRS_OFF = 16
PAIRS_CAP = 1025


def layout(n_units):
    pad4 = lambda n: (n + 3) // 4 * 4
    ns = PAIRS_OFF + pad4(PAIRS_CAP)
    slot = ns + pad4(n_units)
    prefix = slot + pad4(n_units)
    items = prefix + 2 * ((n_units + 1) // 2 * 2)
    return ns, slot, items


def plan(kind, B, s_q, H, *, topk=0, topk_len=None, kv_len=None, win_len=None, splits=0, sms=148):
    po, pl = C.c_int64(), C.c_int64()
    nbytes = _lib.LIB.dsv4_attn_sched_bytes(B * s_q, H, splits, sms, C.byref(po), C.byref(pl))
    assert nbytes > 0
    buf = np.zeros(nbytes // 4, np.int32)
    keep = [None if x is None else np.ascontiguousarray(x, np.int32).reshape(B, s_q) for x in (topk_len, kv_len, win_len)]
    ptr = lambda x: None if x is None else x.ctypes.data
    p = _lib.PlanParams(kind=kind, B=B, s_q=s_q, H=H, topk=topk, num_splits=splits, num_sms=sms,
                        topk_len=ptr(keep[0]), kv_len=ptr(keep[1]), win_len=ptr(keep[2]),
                        sched=buf.ctypes.data, sched_bytes=nbytes)
    rc = _lib.LIB.dsv4_attn_plan_host(C.byref(p))
    assert rc == 0, _lib.LIB.dsv4_attn_last_error()
    hgs = (H + 127) // 128
    n_units = B * s_q * hgs
    ns, slot, items = layout(n_units)
    n_items, n_slots, over, quota = buf[:4].tolist()
    assert over == 0
    pairs = sms // 2
    out = dict(pair_begin=buf[PAIRS_OFF:PAIRS_OFF + pairs + 1].copy(), nsplits=buf[ns:ns + n_units].copy(),
               slot=buf[slot:slot + n_units].copy(), items=buf[items:items + 8 * n_items].reshape(n_items, 8).copy(),
               n_slots=n_slots, quota=quota, slot_cap=po.value // (128 * 512 * 2), hgs=hgs, pairs=pairs)
    assert out["pair_begin"][-1] == n_items
    assert (buf[PAIRS_OFF + pairs:PAIRS_OFF + PAIRS_CAP] == n_items).all()   # blocks beyond the plan find nothing
    return out


def check_cover(pl, n_tok_rows):
    """n_tok_rows[row] = entries of the row.  Returns per-pair cost."""
    hgs = pl["hgs"]
    seen = {}
    for rec in pl["items"]:
        row, hg, t0, nt, slot, n_tok, _, _ = rec.tolist()
        assert n_tok == n_tok_rows[row]
        seen.setdefault((row, hg), []).append((t0, nt, slot))
    assert len(seen) == len(n_tok_rows) * hgs
    used_slots = set()
    for (row, hg), pieces in seen.items():
        tiles = -(-n_tok_rows[row] // TILE)
        pieces.sort()
        u = row * hgs + hg
        assert pl["nsplits"][u] == len(pieces)
        at = 0
        for j, (t0, nt, slot) in enumerate(pieces):
            assert t0 == at and (nt > 0 or tiles == 0)
            at += nt
            if len(pieces) == 1:
                assert slot == -1
            else:
                assert slot == pl["slot"][u] + j and slot not in used_slots
                used_slots.add(slot)
        assert at == tiles
    assert len(used_slots) == pl["n_slots"] <= pl["slot_cap"]
    cost = np.zeros(pl["pairs"])
    for p in range(pl["pairs"]):
        for rec in pl["items"][pl["pair_begin"][p]:pl["pair_begin"][p + 1]]:
            cost[p] += TILE_COST * rec[3] + FIXED if rec[3] > 0 else 1
    return cost


def test_headline_batch_is_left_whole():
    # 64 equal rows on 74 pairs: cutting would save less than the merge costs
    pl = plan(1, 64, 1, 128, kv_len=np.full(64, 782), win_len=np.full(64, 128))
    check_cover(pl, [910] * 64)
    assert (pl["nsplits"] == 1).all() and pl["n_slots"] == 0
    assert np.diff(pl["pair_begin"]).max() == 1


def test_ragged_batch_is_balanced():
    rng = np.random.default_rng(0)
    ctx = np.clip(np.exp(rng.normal(np.log(8192), 1.0, 1024)), 1024, 131072).astype(np.int64)
    kv, win = ctx // 128, np.minimum(128, ctx)
    pl = plan(1, 1024, 1, 128, kv_len=kv, win_len=win)
    cost = check_cover(pl, (kv + win).tolist())
    # equal shares up to the fixed cost of the (at most two) cut pieces of a pair and a tile of rounding at each cut;
    # the last pair takes what is left
    assert cost.max() <= pl["quota"] + 2 * FIXED + 2 * TILE_COST and cost[:-1].min() >= pl["quota"] - 2 * TILE_COST
    assert (pl["nsplits"] > 1).sum() <= pl["pairs"] - 1


def test_few_long_rows_are_cut_over_all_pairs():
    pl = plan(0, 4, 1, 128, topk=2048)
    cost = check_cover(pl, [2048] * 4)
    assert (pl["nsplits"] > 8).all()
    assert (cost > 0).sum() >= pl["pairs"] - 1


def test_fixed_split_count_is_honoured():
    tk = np.array([[2048, 2047], [100, 0], [64, 65]])
    # few units on many pairs: every piece falls to a pair of its own
    pl = plan(0, 3, 2, 128, topk=2048, topk_len=tk, splits=8)
    check_cover(pl, tk.reshape(-1).tolist())
    assert pl["nsplits"].tolist() == [8, 8, 2, 1, 1, 2]


def test_fixed_pieces_on_one_pair_run_as_one_item():
    # many units on few pairs: consecutive pieces of a unit on the same pair are one item, so a unit has at most
    # as many items as pairs it touches, never more than the split count, and the tiles are still covered once
    B = 64
    pl = plan(0, B, 1, 128, topk=2048, splits=8, sms=16)
    check_cover(pl, [2048] * B)
    ns = pl["nsplits"]
    assert ns.max() <= 2 and ns.min() == 1          # 8 units per pair: a unit is whole or cut once at a pair boundary
    assert len(pl["items"]) <= B + pl["pairs"]      # items: units plus at most one cut per pair


def test_two_head_groups_and_empty_rows():
    kv = np.array([0, 5, 700, 0]); win = np.array([0, 0, 128, 3])
    pl = plan(1, 4, 1, 192, kv_len=kv, win_len=win, sms=8)
    check_cover(pl, (kv + win).tolist())
    assert pl["hgs"] == 2


def test_rejected_requests():
    po, pl_ = C.c_int64(), C.c_int64()
    assert _lib.LIB.dsv4_attn_sched_bytes(0, 128, 0, 148, C.byref(po), C.byref(pl_)) == 0
    assert _lib.LIB.dsv4_attn_sched_bytes(4, 128, 65, 148, C.byref(po), C.byref(pl_)) == 0
    buf = np.zeros(64, np.int32)
    p = _lib.PlanParams(kind=0, B=4, s_q=1, H=128, topk=512, num_splits=0, num_sms=148, sched=buf.ctypes.data, sched_bytes=256)
    assert _lib.LIB.dsv4_attn_plan_host(C.byref(p)) == 1
    assert b"smaller" in _lib.LIB.dsv4_attn_last_error()
    p = _lib.PlanParams(kind=7, B=4, s_q=1, H=128, topk=512, num_splits=0, num_sms=148, sched=buf.ctypes.data, sched_bytes=1 << 20)
    assert _lib.LIB.dsv4_attn_plan_host(C.byref(p)) == 1
