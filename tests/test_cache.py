"""The cache's bookkeeping: no slot or page lost, held twice or freed twice (no device needed)."""
import numpy as np
import pytest
import torch

from gopherllm_b200.cache.pool import CacheFull, IdPool
from gopherllm_b200.cache.sequence_cache import PAGE, SequenceCache
from gopherllm_b200.parts.base import KVRequest, StateRequest


def test_pool_hands_out_each_id_once():
    p = IdPool(5, "slot")
    got = [p.take() for _ in range(5)]
    assert sorted(got) == [0, 1, 2, 3, 4] and got == [0, 1, 2, 3, 4]
    with pytest.raises(CacheFull):
        p.take()
    p.give(3)
    p.give(1)
    with pytest.raises(ValueError):
        p.give(3)                       # freed twice
    with pytest.raises(ValueError):
        p.give(9)
    assert p.take() == 1 and p.take() == 3      # lowest first: reuse is deterministic
    p.check()
    with pytest.raises(CacheFull):
        p.take_many(1)


def make(max_tokens=64 * 10, max_positions=300, slots=4, extra=()):
    reqs = [KVRequest(2, 16), KVRequest(2, 16), KVRequest(1, 32, window=128), None, *extra]
    return SequenceCache(reqs, max_tokens, max_positions, torch.bfloat16, "cpu", max_slots=slots, allocate=False)


def test_groups_by_need():
    c = make(extra=(StateRequest((3, 4)),))
    assert len(c.groups) == 2                          # two entries share a shape; the windowed one is apart
    assert c.groups[0].entries == [0, 1] and c.groups[1].entries == [2]
    assert c.n_pages == 10 and c.max_pages_per_seq == 5
    assert c.bytes_per_position() == (2 * 2 * 2 * 16 + 2 * 1 * 32) * 2


def test_reserve_commit_close_and_reuse():
    c = make()
    a, b = c.open(), c.open()
    c.reserve([(a, 130), (b, 1)])
    assert len(c._pages[a][0]) == 3 and len(c._pages[b][0]) == 1 and len(c._pages[a][1]) == 3
    c.commit(a, 130)
    c.commit(b, 1)
    assert c.tokens_held() == 4 * PAGE
    c.reserve([(a, 192)])                               # still three pages
    assert len(c._pages[a][0]) == 3
    c.reserve([(a, 193)])
    assert len(c._pages[a][0]) == 4
    with pytest.raises(ValueError):
        c.commit(b, 65)                                 # never reserved
    with pytest.raises(CacheFull):
        c.reserve([(b, 301)])                           # beyond the longest sequence
    with pytest.raises(CacheFull):
        c.reserve([(a, 300), (b, 6 * 64)])              # 1 + 5 more pages, 5 free: nothing is taken
    assert len(c._pages[a][0]) == 4 and len(c._pages[b][0]) == 1
    rows = c.page_rows(0, [b, a])
    assert rows.shape == (2, 5) and rows.dtype == np.int32 and list(rows[1][:4]) == c._pages[a][0]
    old = list(c._pages[a][0])
    c.close(a)
    with pytest.raises(ValueError):
        c.close(a)                                      # freed twice
    with pytest.raises(ValueError):
        c.length(a)
    c.check()
    n = c.open()
    assert n == a                                       # the slot is used again
    c.reserve([(n, 64)])
    assert c._pages[n][0][0] == min(old)                # and so is its page
    c.check()


def test_fuzz_no_page_lost_or_shared():
    rng = np.random.default_rng(0)
    c = make(max_tokens=64 * 40, max_positions=64 * 9, slots=7)
    live = {}
    for _ in range(3000):
        op = rng.integers(0, 3)
        if op == 0 and c.slots.free_count:
            live[c.open()] = 0
        elif op == 1 and live:
            s = int(rng.choice(list(live)))
            new = live[s] + int(rng.integers(1, 130))
            try:
                c.reserve([(s, new)])
                c.commit(s, new)
                live[s] = new
            except CacheFull:
                pass
        elif op == 2 and live:
            s = int(rng.choice(list(live)))
            c.close(s)
            del live[s]
        c.check()
        assert sorted(c.live_slots()) == sorted(live)
        for s, n in live.items():
            assert c.length(s) == n and len(c._pages[s][0]) >= -(-n // PAGE)
    for s in list(live):
        c.close(s)
    c.check()
    assert all(g.pool.free_count == g.pool.n for g in c.groups) and c.slots.free_count == 7


def test_state_rows_are_zeroed_when_a_slot_is_taken():
    c = SequenceCache([StateRequest((2, 3)), KVRequest(1, 16)], 128, 128, torch.float32, "cpu", max_slots=2)
    s = c.open()
    v = c.view(0)
    assert v.rows.shape == (2, 2, 3) and c.view(1).k.shape == (2, 1, PAGE, 16)
    v.rows[s] += 5.0
    c.close(s)
    s2 = c.open()
    assert s2 == s and float(v.rows[s2].abs().sum()) == 0.0
    assert c.view(5) is None


def test_pages_before_a_window_go_back_as_the_sequence_grows():
    """Group 1 of ``make`` sees the last 128 positions.  Once a page lies wholly before the window of the
    next token it is free again (and reused by another sequence), while the group that sees every
    position keeps all of its pages; the table handed to the kernels shows 0 in a released place."""
    c = make(max_tokens=64 * 14, max_positions=64 * 9, slots=3)
    a = c.open()
    c.reserve([(a, 500)])
    assert c.groups[1].pool.held_count == 8            # a whole prompt needs all its pages while it runs
    c.commit(a, 500)
    # the next token, at 500, sees 373..500: pages 0..4 (positions 0..319) lie before that
    assert c._first_page[a][1] == 5 and c.groups[1].pool.held_count == 3 and c.groups[0].pool.held_count == 8
    rows = c.page_rows(1, [a])
    assert list(rows[0][:5]) == [0] * 5 and all(int(p) == q for p, q in zip(rows[0][5:8], c._pages[a][1][5:8]))
    assert list(c.page_rows(0, [a])[0][:8]) == c._pages[a][0]
    c.check()
    b = c.open()
    c.reserve([(b, 64 * 5)])                           # takes the pages group 1 got back
    assert set(c._pages[b][1]) == {0, 1, 2, 3, 4}
    c.commit(b, 64 * 5)
    c.check()
    for n in range(501, 577):                          # token by token: a page goes back each time the window passes one
        c.reserve([(a, n)])
        c.commit(a, n)
        assert c._first_page[a][1] == (n - 127) // PAGE
        c.check()
    assert len(c._pages[a][1]) == 9 and c.groups[1].pool.held_count == (9 - 7) + (5 - 3)
    c.close(a)
    c.close(b)
    c.check()
    assert all(g.pool.free_count == g.pool.n for g in c.groups)
