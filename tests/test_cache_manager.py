"""The paged cache manager alone (C++, no GPU): page arithmetic, first-in
first-out reuse, windows, state slots, reference counts, and under random
orders of requests no page is lost, held twice or freed twice."""
import random

import pytest

from lyapunov_engine_b200 import build

host = build.load_host()


def seq(i, n, **kw):
    sp = host.SamplingParams()
    for k, v in kw.items():
        setattr(sp, k, v)
    return host.Sequence(i, list(range(n)), sp)


def test_reference_interface():
    # the reference's own test of its manager (tests/test_block_manager.py:11-36)
    bm = host.BlockSpaceManager(100, 16, True)
    assert bm.get_num_free_blocks() == 100 and bm.get_num_used_blocks() == 0
    s = seq(1, 32)
    assert bm.can_allocate(s)
    bm.allocate(s)
    assert bm.get_num_free_blocks() == 98 and len(s.get_block_table()) == 2
    assert bm.can_append_slot(s)
    bm.free(s)
    assert bm.get_num_free_blocks() == 100 and len(s.get_block_table()) == 0
    bm.free(s)                                  # freeing twice changes nothing
    assert bm.get_num_free_blocks() == 100 and bm.audit() == ""


@pytest.mark.parametrize("bs", [1, 4, 16])
def test_grow_is_one_arithmetic_for_prompts_portions_and_decoded_tokens(bs):
    bm = host.BlockSpaceManager(50, bs)
    s = seq(0, 40)
    have = 0
    for n in [1, 2, 3, bs, bs + 1, 2 * bs, 2 * bs + 1, 40]:
        if n > 40:
            continue
        assert bm.grow(s, n)
        have = max(have, (n + bs - 1) // bs)
        assert len(s.get_block_table()) == have
    assert bm.audit() == ""


def test_grow_is_all_or_nothing_and_max_growth_tells_what_fits():
    bm = host.BlockSpaceManager(4, 4)
    a, b = seq(0, 40), seq(1, 40)
    assert bm.grow(a, 9)                        # 3 pages
    assert not bm.can_grow(b, 9) and not bm.grow(b, 9)
    assert b.get_block_table() == [] and bm.get_num_free_blocks() == 1
    assert bm.max_growth(b, 9) == 4 and bm.max_growth(a, 40) == 16
    assert bm.grow(b, 4) and bm.max_growth(b, 9) == 4 and bm.max_growth(a, 13) == 12
    assert bm.audit() == ""


def test_pages_are_used_again_first_in_first_out():
    bm = host.BlockSpaceManager(6, 2)
    a, b, c = seq(0, 4), seq(1, 4), seq(2, 6)
    bm.grow(a, 4); bm.grow(b, 4)
    assert a.get_block_table() == [0, 1] and b.get_block_table() == [2, 3]
    bm.free(a)
    bm.grow(c, 6)
    assert c.get_block_table() == [4, 5, 0]     # the untouched pages first, then the oldest freed
    assert bm.get_num_reuses() == 1 and bm.get_num_allocations() == 7


def test_window_group_gives_pages_back_while_the_request_lives():
    groups = [host.CacheGroupSpec(block_size=4, window=0, num_blocks=32),
              host.CacheGroupSpec(block_size=4, window=6, num_blocks=32)]
    bm = host.BlockSpaceManager(groups, 2)
    s = seq(0, 64)
    for computed in range(1, 41):
        assert bm.grow(s, computed)
        s.set_num_computed_tokens(computed)
        bm.release_passed(s)
        full, win = s.get_block_tables()
        assert all(p >= 0 for p in full) and len(full) == (computed + 3) // 4
        first_needed = max(0, computed - 6 + 1)
        for i, p in enumerate(win):
            assert (p < 0) == ((i + 1) * 4 <= first_needed), (computed, i, win)
        assert bm.get_num_used_blocks(1) <= 3
        assert bm.audit() == ""
    bm.free(s)
    assert bm.get_num_free_blocks(0) == 32 and bm.get_num_free_blocks(1) == 32 and bm.audit() == ""


def test_state_slots_are_taken_with_the_first_page_and_bound_the_live_requests():
    bm = host.BlockSpaceManager([host.CacheGroupSpec(block_size=4, window=0, num_blocks=100)], 2)
    a, b, c = seq(0, 8), seq(1, 8), seq(2, 8)
    assert bm.grow(a, 1) and bm.grow(b, 8)
    assert {a.get_state_slot(), b.get_state_slot()} == {0, 1}
    assert not bm.can_grow(c, 1) and bm.max_growth(c, 8) == 0 and c.get_state_slot() == -1
    bm.free(a)
    assert a.get_state_slot() == -1 and bm.grow(c, 8) and c.get_state_slot() == 0
    assert bm.audit() == ""


def test_a_model_without_pages_still_has_slots():
    bm = host.BlockSpaceManager([], 3)
    s = seq(0, 1000)
    assert bm.grow(s, 1000) and s.get_state_slot() == 0 and s.get_block_tables() == []
    bm.free(s)
    assert bm.get_num_free_state_slots() == 3 and bm.audit() == ""


def test_fork_shares_full_pages_by_reference_count():
    bm = host.BlockSpaceManager(10, 4)
    parent = seq(0, 11)
    bm.grow(parent, 11)
    parent.set_num_computed_tokens(11)
    child = seq(1, 20)
    bm.fork(parent, child)
    assert child.get_block_table() == parent.get_block_table()[:2] and child.get_num_computed_tokens() == 8
    assert bm.get_ref_count(0, parent.get_block_table()[0]) == 2 and bm.get_ref_count(0, parent.get_block_table()[2]) == 1
    assert bm.grow(child, 20) and bm.audit() == ""
    bm.free(parent)
    assert bm.get_ref_count(0, child.get_block_table()[0]) == 1 and bm.get_num_free_blocks() == 10 - 5
    bm.free(child)
    assert bm.get_num_free_blocks() == 10 and bm.audit() == ""


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_lose_nothing(seed):
    rng = random.Random(seed)
    groups = [host.CacheGroupSpec(block_size=rng.choice([1, 2, 8]), window=0, num_blocks=rng.randint(8, 40)),
              host.CacheGroupSpec(block_size=rng.choice([2, 4]), window=rng.randint(3, 20), num_blocks=rng.randint(8, 40))]
    slots = rng.randint(2, 6)
    bm = host.BlockSpaceManager(groups, slots)
    live, next_id = [], 0
    for _ in range(600):
        action = rng.random()
        if action < 0.25 or not live:
            s = seq(next_id, 300)
            next_id += 1
            n = rng.randint(1, 30)
            ok = bm.grow(s, n)
            assert ok == (s.get_state_slot() >= 0)
            if ok:
                s.set_num_computed_tokens(n)
                bm.release_passed(s)
                live.append(s)
            else:
                assert s.get_block_tables() == [] or all(len(t) == 0 for t in s.get_block_tables())
        elif action < 0.8:
            s = rng.choice(live)
            n = s.get_num_computed_tokens() + rng.randint(1, 12)
            before = [list(t) for t in s.get_block_tables()]
            if bm.grow(s, n):
                s.set_num_computed_tokens(n)
                bm.release_passed(s)
            else:
                assert [list(t) for t in s.get_block_tables()] == before
        else:
            s = live.pop(rng.randrange(len(live)))
            bm.free(s)
            if rng.random() < 0.3:
                bm.free(s)
        assert bm.audit() == "", bm.audit()
        assert len(live) <= slots
    for s in live:
        bm.free(s)
    assert bm.audit() == ""
    assert all(bm.get_num_free_blocks(g) == groups[g].num_blocks for g in range(2))
    assert bm.get_num_free_state_slots() == slots


def test_pack_step_layout():
    import numpy as np
    bm = host.BlockSpaceManager([host.CacheGroupSpec(block_size=4, window=0, num_blocks=20)], 4)
    a = host.Sequence(0, [10, 11, 12, 13, 14, 15, 16], host.SamplingParams())
    b = host.Sequence(1, [20, 21, 22], host.SamplingParams())
    bm.grow(a, 5); a.set_num_computed_tokens(5); bm.grow(a, 7)
    bm.grow(b, 3)
    entries = [host.StepEntry(a, 5, 2, [1]), host.StepEntry(b, 0, 3, [0, 2])]
    buf = np.zeros(512, dtype=np.int32)
    p = host.pack_step(entries, bm, [2, 16], 4, [6], buf.ctypes.data, buf.size)
    assert (p.num_tokens, p.num_requests, p.num_real_requests, p.num_wanted, p.max_q_len, p.max_context) == (7, 4, 2, 3, 3, 7)
    T, B = 7, 4
    assert buf[p.off_token_ids:p.off_token_ids + T].tolist() == [15, 16, 20, 21, 22, 0, 0]
    assert buf[p.off_positions:p.off_positions + T].tolist() == [5, 6, 0, 1, 2, 0, 0]
    assert buf[p.off_request_of_token:p.off_request_of_token + T].tolist() == [0, 0, 1, 1, 1, 2, 3]
    assert buf[p.off_cu_q:p.off_cu_q + B + 1].tolist() == [0, 2, 5, 6, 7]
    assert buf[p.off_ctx_before:p.off_ctx_before + B].tolist() == [5, 0, 0, 0]
    assert buf[p.off_state_slots:p.off_state_slots + B].tolist() == [0, 1, -1, -1]
    assert buf[p.off_wanted_rows:p.off_wanted_rows + 3].tolist() == [1, 2, 4]
    table = buf[p.off_block_tables[0]:p.off_block_tables[0] + B * 6].reshape(B, 6)
    assert table[0].tolist() == a.get_block_table() + [20] * 4 and table[1].tolist() == b.get_block_table() + [20] * 5
    assert table[2].tolist() == [20] * 6                       # padding writes to the page nobody owns
    assert p.num_tiles == [5, 4] and p.num_tiles_multi == [3, 2] and p.num_decode == 2
    # tiles of several tokens by the keys they see, fewest first (the kernels start from the end); then single tokens
    assert buf[p.off_tile_request[0]:p.off_tile_request[0] + 5].tolist() == [1, 1, 0, 2, 3]
    assert buf[p.off_tile_q0[0]:p.off_tile_q0[0] + 5].tolist() == [0, 2, 0, 0, 0]
    assert buf[p.off_tile_request[1]:p.off_tile_request[1] + 4].tolist() == [1, 0, 2, 3]
    assert buf[p.off_decode_requests:p.off_decode_requests + 2].tolist() == [2, 3]
    # a step padded to a fixed shape lists one wanted row per request, dummy requests included: there is room
    assert p.off_block_tables[0] - p.off_wanted_rows >= p.num_requests
    nine = []
    for i in range(9):
        s = host.Sequence(10 + i, [1, 2], host.SamplingParams())
        bm.grow(s, 1); s.set_num_computed_tokens(1); bm.grow(s, 2)
        nine.append(s)
    p9 = host.pack_step([host.StepEntry(s, 1, 1, [0]) for s in nine], bm, [16], 16, [6], buf.ctypes.data, buf.size)
    assert p9.num_requests == 16 and p9.off_block_tables[0] - p9.off_wanted_rows >= 16
    for s in nine:
        bm.free(s)
    # the first entry padded with dummy tokens to a fixed number of rows: they continue its positions, carry
    # token 0 and point at the request's own pages, then at the page nobody owns
    pp = host.pack_step([host.StepEntry(b, 0, 3, [2]), host.StepEntry(a, 5, 1, [0])], bm, [2, 16], 4, [6], buf.ctypes.data,
                        buf.size, pad_first_to=8)
    assert (pp.num_tokens, pp.num_requests, pp.num_wanted, pp.max_q_len, pp.max_context, pp.num_decode) == (11, 4, 2, 8, 8, 3)
    assert buf[pp.off_token_ids:pp.off_token_ids + 11].tolist() == [20, 21, 22, 0, 0, 0, 0, 0, 15, 0, 0]
    assert buf[pp.off_positions:pp.off_positions + 11].tolist() == [0, 1, 2, 3, 4, 5, 6, 7, 5, 0, 0]
    assert buf[pp.off_request_of_token:pp.off_request_of_token + 11].tolist() == [0] * 8 + [1, 2, 3]
    assert buf[pp.off_cu_q:pp.off_cu_q + 5].tolist() == [0, 8, 9, 10, 11]
    assert buf[pp.off_wanted_rows:pp.off_wanted_rows + 2].tolist() == [2, 8]
    table = buf[pp.off_block_tables[0]:pp.off_block_tables[0] + 4 * 6].reshape(4, 6)
    assert table[0].tolist() == b.get_block_table() + [20] * 5     # positions 4..7 of the dummies: nobody's page
    assert pp.num_tiles == [4 + 3, 1 + 3] and pp.num_tiles_multi == [4, 1]
    with pytest.raises(ValueError, match="runs past"):
        host.pack_step([host.StepEntry(b, 0, 4, [])], bm, [], 0, [], 0, 0, pad_first_to=8)
    # single-token requests come after the others in the tile lists
    c = host.Sequence(2, [1, 2, 3], host.SamplingParams())
    bm.grow(c, 2); c.set_num_computed_tokens(2); bm.grow(c, 3)
    p2 = host.pack_step([host.StepEntry(c, 2, 1, [0]), host.StepEntry(b, 0, 3, [])], bm, [2], 0, [], buf.ctypes.data, buf.size)
    assert buf[p2.off_tile_request[0]:p2.off_tile_request[0] + 3].tolist() == [1, 1, 0] and p2.num_tiles_multi == [2]
    assert buf[p2.off_decode_requests:p2.off_decode_requests + 1].tolist() == [0] and p2.num_decode == 1
    with pytest.raises(ValueError, match="starts at"):
        host.pack_step([host.StepEntry(a, 4, 2, [])], bm, [], 0, [], 0, 0)
    with pytest.raises(ValueError, match="wanted place"):
        host.pack_step([host.StepEntry(a, 5, 2, [2])], bm, [], 0, [], 0, 0)
