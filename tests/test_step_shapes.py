"""The shapes of captured steps: how many rows a decode step of n requests is
padded to, and how far a prompt portion beside decoded tokens.  Pure functions
of the engine; the figures in the comments are measured on a B200 at
Llama-3.2-1B layer sizes."""
from lyapunov_engine_b200.engine.step import decode_bucket, padded_portion, prompt_bucket


def test_decode_buckets():
    big = 256
    assert [decode_bucket(n, big) for n in (1, 2, 3, 5, 9, 17, 32)] == [1, 2, 4, 8, 16, 32, 32]
    # between the powers of two from 48 on: 33 to 48 requests run as 48 rows, not 64
    assert [decode_bucket(n, big) for n in (33, 48, 49, 64, 65, 96, 97, 128, 129, 192, 193)] == \
        [48, 48, 64, 64, 96, 96, 128, 128, 192, 192, 256]
    # never more rows than the engine is set up for, and never fewer than the requests
    assert decode_bucket(5, 6) == 6 and decode_bucket(40, 40) == 40 and decode_bucket(50, 50) == 50
    assert decode_bucket(7, 4) == 7
    for limit in (1, 3, 8, 40, 64, 100):
        last = 0
        for n in range(1, limit + 1):
            b = decode_bucket(n, limit)
            assert n <= b <= limit and b >= last      # monotone: a larger batch never gets a smaller step
            last = b


def test_prompt_portions_are_padded_to_round_rows():
    assert [prompt_bucket(n) for n in (1, 64, 65, 130, 512, 513, 1000)] == [64, 64, 128, 192, 512, 640, 1024]
    # alone: the portion's own round number
    assert [padded_portion(n, 0) for n in (130, 257, 1000)] == [192, 320, 1024]
    # beside decoded tokens the step's rows as a whole, where that saves a tile of 128 rows ...
    assert padded_portion(504, 8) == 504        # 512 rows, not 512 + 8 (2.47 -> 2.23 ms)
    assert padded_portion(224, 32) == 224       # 256 rows, not 256 + 32
    assert padded_portion(380, 4) == 380        # 384 rows, not 384 + 4
    # ... and the portion's own round number where it does not (fewer dummy tokens)
    assert padded_portion(512, 8) == 512        # 520 rows either way take 5 tiles; 640 would too
    assert padded_portion(256, 32) == 256
    assert padded_portion(130, 4) == 192
    for count in range(2, 1025, 7):
        for bucket in (0, 1, 4, 8, 32, 48, 64):
            rows = padded_portion(count, bucket)
            assert rows >= count
            assert (rows + bucket + 127) // 128 <= (prompt_bucket(count) + bucket + 127) // 128
