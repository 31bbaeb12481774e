"""The scheduler's decisions (C++, no GPU, no model: the tests feed the
"sampled" tokens, as the reference's own scheduler test does,
tests/test_block_manager.py:39-80)."""
import random

import pytest

from lyapunov_engine_b200 import build

host = build.load_host()


def make(num_blocks=100, block_size=16, max_num_seqs=4, budget=512, max_model_len=4096, eos=(), chunk=0, slots=None):
    bm = host.BlockSpaceManager([host.CacheGroupSpec(block_size=block_size, window=0, num_blocks=num_blocks)],
                                slots if slots is not None else max_num_seqs)
    cfg = host.SchedulerConfig()
    cfg.max_num_seqs, cfg.max_num_batched_tokens, cfg.max_model_len = max_num_seqs, budget, max_model_len
    cfg.eos_token_ids = list(eos)
    cfg.max_prefill_chunk = chunk
    return host.ContinuousScheduler(cfg, bm), bm


def seq(i, prompt, max_tokens=3, ignore_eos=False):
    sp = host.SamplingParams()
    sp.max_tokens, sp.ignore_eos = max_tokens, ignore_eos
    return host.Sequence(i, list(prompt), sp)


def shape(out):
    return [(e.seq.get_seq_id(), e.start, e.count, list(e.want)) for e in out.entries]


def test_lifecycle_of_one_request():
    sched, bm = make()
    assert not sched.has_unfinished_sequences()
    s = seq(1, [10, 20, 30], max_tokens=3)
    sched.add_sequence(s)
    assert sched.get_num_waiting_sequences() == 1
    out = sched.schedule()
    assert out.is_prefill and shape(out) == [(1, 0, 3, [2])] and sched.get_num_running_sequences() == 1
    sched.post_step(out, [100])
    assert s.get_num_computed_tokens() == 3 and not s.is_finished()
    out = sched.schedule()
    assert not out.is_prefill and shape(out) == [(1, 3, 1, [0])]
    sched.post_step(out, [101])
    out = sched.schedule()
    sched.post_step(out, [102])
    assert s.is_finished() and s.finish_reason() == "length" and s.get_output_tokens() == [100, 101, 102]
    assert not sched.has_unfinished_sequences() and bm.get_num_free_blocks() == 100 and bm.audit() == ""


def test_prompts_are_cut_under_the_token_budget_and_decodes_come_first():
    sched, bm = make(budget=8, block_size=4)
    a, b = seq(0, range(5), max_tokens=10), seq(1, range(100, 119), max_tokens=2)
    sched.add_sequence(a); sched.add_sequence(b)
    out = sched.schedule()
    assert shape(out) == [(0, 0, 5, [4]), (1, 0, 3, [])] and out.num_batched_tokens == 8 and out.is_prefill
    assert [s.get_seq_id() for s in out.sampled_seqs] == [0]
    sched.post_step(out, [7])
    out = sched.schedule()                       # a decodes (first), b takes the rest of the budget
    assert shape(out) == [(0, 5, 1, [0]), (1, 3, 7, [])]
    sched.post_step(out, [8])
    out = sched.schedule()
    assert shape(out) == [(0, 6, 1, [0]), (1, 10, 7, [])]
    sched.post_step(out, [9])
    out = sched.schedule()                       # b's last portion holds its last prompt token: sampled
    assert shape(out) == [(0, 7, 1, [0]), (1, 17, 2, [1])] and [s.get_seq_id() for s in out.sampled_seqs] == [0, 1]
    sched.post_step(out, [1, 2])
    assert b.get_output_tokens() == [2] and a.get_output_tokens() == [7, 8, 9, 1]
    assert bm.audit() == ""


def test_max_prefill_chunk_and_max_num_seqs():
    sched, _ = make(budget=100, chunk=6, max_num_seqs=2)
    for i in range(3):
        sched.add_sequence(seq(i, range(10)))
    out = sched.schedule()
    assert shape(out) == [(0, 0, 6, []), (1, 0, 6, [])] and sched.get_num_waiting_sequences() == 1
    sched.post_step(out, [])
    out = sched.schedule()
    assert shape(out) == [(0, 6, 4, [3]), (1, 6, 4, [3])]


def test_end_of_sequence_ids_ignore_eos_and_max_model_len():
    sched, bm = make(eos=[7, 9], max_model_len=8)
    a, b, c = seq(0, [1, 2], 50), seq(1, [1, 2], 50, ignore_eos=True), seq(2, [1, 2, 3, 4, 5], 50, ignore_eos=True)
    too_long = seq(3, range(8), 5)
    for s in (a, b, c, too_long):
        sched.add_sequence(s)
    out = sched.schedule()
    assert [s.get_seq_id() for s in out.finished_seqs] == [3] and too_long.finish_reason() == "error"
    assert "max_model_len" in too_long.get_error()
    sched.post_step(out, [9, 9, 5])
    assert a.is_finished() and a.finish_reason() == "stop" and a.get_output_tokens() == [9]
    assert not b.is_finished()
    while sched.has_unfinished_sequences():
        out = sched.schedule()
        sched.post_step(out, [7] * len(out.sampled_seqs))
    assert b.finish_reason() == "length" and b.get_total_len() == 8 and c.get_total_len() == 8
    assert bm.audit() == "" and bm.get_num_free_blocks() == 100


def test_admission_is_first_come_first_served_without_overtaking():
    sched, bm = make(num_blocks=4, block_size=4, budget=64)
    big, small = seq(0, range(14), 2), seq(1, range(3), 2)
    first = seq(2, range(6), 20)
    sched.add_sequence(first)
    out = sched.schedule(); sched.post_step(out, [1])      # first holds 2 pages
    sched.add_sequence(big); sched.add_sequence(small)
    out = sched.schedule()
    # big gets a shortened portion (what fits in the 2 free pages); small must not overtake it
    assert shape(out) == [(2, 6, 1, [0]), (0, 0, 8, [])]
    assert sched.get_num_waiting_sequences() == 1


def test_out_of_pages_preempts_the_request_admitted_last_and_recomputes_it():
    sched, bm = make(num_blocks=8, block_size=2, budget=64)
    a, b = seq(0, range(1, 9), 4, True), seq(1, range(11, 19), 4, True)
    sched.add_sequence(a); sched.add_sequence(b)
    out = sched.schedule()
    assert shape(out) == [(0, 0, 8, [7]), (1, 0, 8, [7])]
    sched.post_step(out, [11, 21])                          # both now need a third page; none is free
    assert bm.get_num_free_blocks() == 0
    out = sched.schedule()
    assert [s.get_seq_id() for s in out.preempted_seqs] == [1] and shape(out) == [(0, 8, 1, [0])]
    assert b.get_num_computed_tokens() == 0 and b.get_block_table() == [] and b.get_num_preemptions() == 1
    assert sched.get_num_waiting_sequences() == 1 and bm.audit() == ""
    sched.post_step(out, [12])
    # b comes back only when pages are free, and is recomputed over prompt and output alike
    seen_b = []
    while sched.has_unfinished_sequences():
        out = sched.schedule()
        for e in out.entries:
            if e.seq.get_seq_id() == 1:
                seen_b.append((e.start, e.count))
        sched.post_step(out, [30 + len(s.get_output_tokens()) for s in out.sampled_seqs])
        assert bm.audit() == ""
    assert a.finish_reason() == "length" and b.finish_reason() == "length"
    assert seen_b[0][0] == 0 and seen_b[0][1] >= 1 and b.get_output_tokens()[0] == 21
    assert len(a.get_output_tokens()) == 4 and len(b.get_output_tokens()) == 4
    assert sched.get_stats().preemptions >= 1 and bm.get_num_free_blocks() == 8


def test_a_request_that_cannot_fit_alone_fails_instead_of_hanging():
    sched, bm = make(num_blocks=2, block_size=2, budget=64)
    s = seq(0, [1, 2, 3], 10, True)
    sched.add_sequence(s)
    steps = 0
    while sched.has_unfinished_sequences():
        out = sched.schedule()
        sched.post_step(out, [5] * len(out.sampled_seqs))
        steps += 1
        assert steps < 20
    assert s.finish_reason() == "error" and "too small" in s.get_error()
    assert len(s.get_output_tokens()) == 2 and bm.get_num_free_blocks() == 2 and bm.audit() == ""


def test_abort_frees_pages_in_both_queues():
    sched, bm = make(max_num_seqs=1)
    a, b = seq(0, range(20)), seq(1, range(20))
    sched.add_sequence(a); sched.add_sequence(b)
    out = sched.schedule()
    sched.abort_sequence(0); sched.abort_sequence(1)
    assert a.finish_reason() == "abort" and b.finish_reason() == "abort"
    assert not sched.has_unfinished_sequences() and bm.get_num_free_blocks() == 100 and bm.audit() == ""
    sched.post_step(out, [3])                               # the step that was in flight changes nothing
    assert a.get_output_tokens() == []


def next_token(tokens):
    """A stand-in model: the next token is a function of all tokens so far."""
    h = 17
    for t in tokens:
        h = (h * 31 + t + 1) % 1009
    return h % 50 + 10


@pytest.mark.parametrize("seed", range(5))
def test_random_load_with_few_pages_gives_the_same_tokens_as_no_pressure(seed):
    rng = random.Random(seed)
    sched, bm = make(num_blocks=rng.randint(16, 24), block_size=rng.choice([2, 4]), budget=rng.randint(6, 24),
                     max_num_seqs=rng.randint(2, 5), eos=[10], chunk=rng.choice([0, 5]))
    seqs, expected = [], {}
    for i in range(12):
        prompt = [rng.randrange(100) for _ in range(rng.randint(1, 18))]
        s = seq(i, prompt, max_tokens=rng.randint(1, 12))
        seqs.append(s)
        toks, outs = list(prompt), []
        while len(outs) < s.get_sampling_params().max_tokens:
            t = next_token(toks)
            outs.append(t); toks.append(t)
            if t == 10:
                break
        expected[i] = outs
    pending = list(seqs)
    steps = 0
    while sched.has_unfinished_sequences() or pending:
        while pending and rng.random() < 0.4:
            sched.add_sequence(pending.pop(0))
        out = sched.schedule()
        assert out.num_batched_tokens <= sched.get_config().max_num_batched_tokens
        assert len(out.entries) <= sched.get_config().max_num_seqs
        total = 0
        for e in out.entries:
            assert e.start == e.seq.get_num_computed_tokens() and e.count >= 1
            assert e.start + e.count <= e.seq.get_total_len()
            need = (e.start + e.count + bm.get_block_size() - 1) // bm.get_block_size()
            assert len(e.seq.get_block_table()) >= need and e.seq.get_state_slot() >= 0
            total += e.count
        assert total == out.num_batched_tokens
        tokens = [next_token(list(s.get_prompt_tokens()) + list(s.get_output_tokens())) for s in out.sampled_seqs]
        sched.post_step(out, tokens)
        assert bm.audit() == "", bm.audit()
        steps += 1
        assert steps < 3000
    for s in seqs:
        assert s.is_finished() and s.finish_reason() in ("stop", "length"), (s.get_seq_id(), s.finish_reason(), s.get_error())
        assert s.get_output_tokens() == expected[s.get_seq_id()]
    assert bm.get_num_free_blocks() == bm.get_num_blocks() and bm.get_num_free_state_slots() == bm.get_num_state_slots()


def test_a_decode_step_is_scheduled_ahead_of_the_result_before_it():
    """schedule_ahead builds the step after a launched decode step without its
    tokens: one more token each, one step ahead; the results come back in order."""
    sched, bm = make(block_size=4, eos=(99,))
    a, b = seq(0, [1, 2, 3], max_tokens=6), seq(1, [4, 5, 6, 7, 8], max_tokens=6)
    sched.add_sequence(a); sched.add_sequence(b)
    first = sched.schedule()
    assert first.is_prefill and not sched.schedule_ahead(first).entries          # prompts: nothing is known ahead
    sched.post_step(first, [10, 20])
    step1 = sched.schedule()
    assert shape(step1) == [(0, 3, 1, [0]), (1, 5, 1, [0])]
    ahead = sched.schedule_ahead(step1)                                          # before step1's tokens are known
    assert [(e.seq.get_seq_id(), e.start, e.count, list(e.want), e.ahead) for e in ahead.entries] == \
        [(0, 4, 1, [0], 1), (1, 6, 1, [0], 1)]
    assert [s.get_seq_id() for s in ahead.sampled_seqs] == [0, 1] and not ahead.is_prefill
    # the step packs although the host does not know its tokens: they come from the device
    packed = host.pack_step(list(ahead.entries), bm, [16], 0, [], 0, 0)
    assert packed.num_tokens == 2 and packed.max_context == 7
    # pages for the token after next are there
    assert len(a.get_block_table()) * 4 >= 5 and bm.audit() == ""
    sched.post_step(step1, [11, 21])
    again = sched.schedule_ahead(ahead)
    assert [(e.start, e.ahead) for e in again.entries] == [(5, 1), (7, 1)]
    sched.post_step(ahead, [12, 99])                                             # b ends with an end-of-sequence token
    assert b.is_finished() and b.finish_reason() == "stop" and b.get_output_tokens() == [20, 21, 99]
    sched.post_step(again, [13, 55])                                             # its token of the step ahead is dropped
    assert b.get_output_tokens() == [20, 21, 99] and a.get_output_tokens() == [10, 11, 12, 13]
    assert a.get_num_computed_tokens() == 6 and not a.is_finished()
    sched.post_step(sched.schedule(), [14])
    # a reaches max_tokens with the token that is still to come: that cannot be scheduled ahead
    last = sched.schedule()
    assert shape(last) == [(0, 7, 1, [0])] and not sched.schedule_ahead(last).entries
    sched.post_step(last, [15])
    assert a.is_finished() and a.finish_reason() == "length" and bm.get_num_free_blocks() == 100 and bm.audit() == ""


def test_nothing_is_scheduled_ahead_of_an_admission_or_without_pages():
    sched, bm = make(num_blocks=3, block_size=4, max_num_seqs=2)
    a = seq(0, [1, 2, 3], max_tokens=50)
    sched.add_sequence(a)
    sched.post_step(sched.schedule(), [9])
    sched.post_step(sched.schedule(), [9])
    step = sched.schedule()
    waiting = seq(1, [5, 6], max_tokens=2)
    sched.add_sequence(waiting)
    assert not sched.schedule_ahead(step).entries                                # a request waits to be admitted
    sched.abort_sequence(1)
    assert sched.schedule_ahead(step).entries
    sched.post_step(step, [9])
    # run a up to the end of its third and last page: the step after needs a fourth
    while a.get_total_len() < 12:
        sched.post_step(sched.schedule(), [9])
    step = sched.schedule()
    assert shape(step) == [(0, 11, 1, [0])] and not sched.schedule_ahead(step).entries and bm.audit() == ""


def test_padded_lengths_of_prompt_portions():
    """Portions run as graphs of padded shape: multiples of 64 up to 512, of 128 above."""
    from lyapunov_engine_b200.engine.step import prompt_bucket
    assert [prompt_bucket(n) for n in (2, 64, 65, 500, 512, 513, 640, 1000, 1024)] == [64, 64, 128, 512, 512, 640, 640, 1024, 1024]

