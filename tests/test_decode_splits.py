"""How the split-key decode attention cuts its keys: the choice is a pure
function of the batch, the context and what the device holds, so it is checked
here against the decode steps that were measured on a B200 (Llama-3.2-1B layer
sizes, 4,096 keys, every split count from 1 to 8 forced in turn): the fastest
measured count for each batch."""
from lyapunov_engine_b200.parts.attention_kernels import DECODE_KEYS_PER_SPLIT, choose_decode_splits

# blocks of the decode kernel that a B200 holds at once, by split count (what the runtime answers for head size 64)
B200_HD64 = [296, 296, 279, 284, 280, 270, 259, 264]


def resident(splits):
    return B200_HD64[splits - 1] if splits <= len(B200_HD64) else 296


def test_the_measured_best_split_counts():
    fastest = {1: 16, 2: 16, 3: 8, 4: 8, 5: 6, 6: 5, 7: 4, 8: 4, 12: 2, 16: 2, 20: 3, 24: 1, 28: 1, 32: 1, 64: 1}
    for batch, splits in fastest.items():
        assert choose_decode_splits(batch * 8, 4096, 64, resident) == splits, batch


def test_a_wave_is_never_overfilled_by_a_cluster():
    """7 requests x 8 groups x 5 splits are 280 blocks, exactly what the device
    holds in clusters of 5: inside a step that cost a second wave (0.92 ms a
    step against 0.79 ms with 4 splits)."""
    for batch in range(1, 9):
        s = choose_decode_splits(batch * 8, 4096, 64, resident)
        if 1 < s <= 8:
            assert batch * 8 * s <= 0.97 * resident(s) + 1, (batch, s)


# the same of the form with 16-key tiles (four blocks a multiprocessor), which runs where even the unsplit
# blocks are more than 296
B200_HD64_SMALL = [592, 592, 561, 568, 560, 558, 546, 568]


def test_more_blocks_than_the_device_holds():
    """Measured at 36 to 128 requests (ms per step with 1, 2, 3 splits where
    taken): 64 requests 2.22 with 1; 80 requests 3.24, 2.93, 2.82; 96 requests
    3.41, 3.05; 112 and 128 requests best unsplit; up to 37 requests (296
    blocks) the usual form holds them all and nothing changes."""
    small = lambda s: B200_HD64_SMALL[s - 1] if s <= 8 else 592
    pick = lambda batch: choose_decode_splits(batch * 8, 4096, 64, resident, small, 148)
    assert [pick(b) for b in (36, 37, 40, 48, 64)] == [1, 1, 1, 1, 1]
    assert pick(80) == 3 and pick(96) == 2 and pick(112) == 1 and pick(128) == 1
    for batch in (5, 8, 16, 20, 24, 32):          # not touched by the other form's figures
        assert pick(batch) == choose_decode_splits(batch * 8, 4096, 64, resident)


def test_long_contexts_and_short_ones():
    assert choose_decode_splits(8 * 8, 32768, 64, resident) == 4     # 3 splits: 2.19 ms a step, 4: 1.91 ms
    assert choose_decode_splits(16 * 8, 32768, 64, resident) == 2    # 1 split: 5.43 ms, 2: 3.35 ms
    assert choose_decode_splits(32 * 8, 32768, 64, resident) == 1
    assert choose_decode_splits(8, 100, 64, resident) == 1           # fewer keys than a split is worth
    for context in (300, 1000, 5000):
        assert choose_decode_splits(8, context, 64, resident) <= -(-context // DECODE_KEYS_PER_SPLIT)
