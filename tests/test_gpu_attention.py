"""The attention kernels alone against plain attention over gathered pages:
mixed batches (portions beside single tokens), scattered pages, windows, head
sizes in steps of 16, and inputs made so that one far key decides the result."""
import pytest
import torch


pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def build_case(dtype, nh, nkv, hd, page, q_lens, ctx_before, seed, window=None, spike=True):
    """Random K/V for every request in scattered pages, queries for the step's
    tokens; returns device tensors and the plain result."""
    g = torch.Generator().manual_seed(seed)
    B = len(q_lens)
    totals = [c + q for c, q in zip(ctx_before, q_lens)]
    max_blocks = max((t + page - 1) // page for t in totals) + 1
    pages_needed = sum((t + page - 1) // page for t in totals)
    num_pages = pages_needed + 3
    perm = torch.randperm(num_pages - 1, generator=g)[:pages_needed].tolist()   # the last page stays unused
    table = torch.full((B, max_blocks), num_pages - 1, dtype=torch.int32)
    k_cache = torch.randn(num_pages, nkv, page, hd, generator=g).to(dtype)     # stale garbage everywhere
    v_cache = torch.randn(num_pages, nkv, page, hd, generator=g).to(dtype)
    T = sum(q_lens)
    q = torch.randn(T, nh * hd, generator=g)
    ks, vs = [], []
    nxt = 0
    for b in range(B):
        k = torch.randn(nkv, totals[b], hd, generator=g)
        v = torch.randn(nkv, totals[b], hd, generator=g)
        if spike and totals[b] > 3:
            # one far key answers the last query of the request strongly
            far = 1 if window is None else max(0, totals[b] - (window or totals[b]))
            t_last = sum(q_lens[:b + 1]) - 1
            for h in range(nh):
                k[h // (nh // nkv), far] = q[t_last, h * hd:(h + 1) * hd] * 1.5
        k, v = k.to(dtype), v.to(dtype)
        ks.append(k.float()); vs.append(v.float())
        for i in range((totals[b] + page - 1) // page):
            pg = perm[nxt]; nxt += 1
            table[b, i] = pg
            n = min(page, totals[b] - i * page)
            k_cache[pg, :, :n] = k[:, i * page:i * page + n]
            v_cache[pg, :, :n] = v[:, i * page:i * page + n]
    q = q.to(dtype)
    want = torch.zeros(T, nh * hd)
    t0 = 0
    for b in range(B):
        for j in range(q_lens[b]):
            p = ctx_before[b] + j
            lo = max(0, p - window + 1) if window else 0
            qq = q[t0 + j].float().view(nh, 1, hd)
            # plain attention of one query over its visible keys (no mask needed)
            kk = ks[b][:, lo:p + 1].repeat_interleave(nh // nkv, 0)
            vv = vs[b][:, lo:p + 1].repeat_interleave(nh // nkv, 0)
            s = torch.matmul(qq, kk.transpose(-1, -2)) / (hd ** 0.5)
            want[t0 + j] = torch.matmul(torch.softmax(s, -1), vv).reshape(-1)
        t0 += q_lens[b]
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    return dict(q=q.to(DEV), k=k_cache.to(DEV), v=v_cache.to(DEV), table=table.to(DEV), cu=cu.to(DEV),
                ctx=torch.tensor(ctx_before, dtype=torch.int32, device=DEV), want=want, T=T)


def tiles(q_lens, size):
    req, q0 = [], []
    for b, n in enumerate(q_lens):
        for s in range(0, n, size):
            req.append(b); q0.append(s)
    return (torch.tensor(req, dtype=torch.int32, device=DEV), torch.tensor(q0, dtype=torch.int32, device=DEV), len(req))


CASES = [
    # nh, nkv, hd, page, q_lens, ctx_before, window
    (4, 2, 16, 4, [5, 1, 17], [0, 9, 3], None),
    (3, 1, 32, 8, [1, 1, 1, 1], [0, 7, 8, 40], None),
    (6, 3, 64, 16, [33, 2, 1], [100, 0, 515], None),
    (8, 8, 48, 2, [40], [0], None),
    (2, 1, 128, 16, [3, 70], [61, 2], None),
    (4, 2, 80, 4, [9, 1], [30, 77], 12),
    (2, 2, 256, 16, [18, 1], [0, 33], None),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", CASES)
def test_generic_kernel(case, dtype):
    from lyapunov_engine_b200 import ops
    nh, nkv, hd, page, q_lens, ctx_before, window = case
    c = build_case(dtype, nh, nkv, hd, page, q_lens, ctx_before, seed=hd + page, window=window)
    out = torch.zeros(c["T"], nh * hd, dtype=dtype, device=DEV)
    status = ops.new_status(DEV)
    tr, tq, n = tiles(q_lens, 16)
    ops.attention_generic(out, c["q"], c["q"].stride(0), c["k"], c["v"], c["table"], c["cu"], c["ctx"], tr, tq, n,
                          nh, nkv, hd, page, window, 1.0 / hd ** 0.5, status)
    ops.check_status(status)
    tol = dict(atol=2e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(out.float().cpu(), c["want"], **tol)


MMA_CASES = CASES[:6] + [
    (32, 8, 64, 16, [1] * 8, [4095, 17, 0, 63, 64, 1000, 2047, 300], None),     # the 1B model's decode shape
    (24, 8, 128, 16, [200, 1, 1, 64, 1], [0, 900, 5, 64, 129], None),
    (32, 1, 32, 8, [1, 1, 3], [77, 300, 10], None),                            # 32 query heads on one kv head: two row tiles
    (4, 4, 96, 16, [130], [700], 256),
    (2, 1, 112, 4, [1, 1], [511, 40], 100),
    (8, 2, 64, 16, [300, 1, 128, 129], [0, 50, 128, 1000], None),               # tcgen05 prefill: several tiles, edges
    (4, 4, 128, 8, [257, 5], [31, 0], None),
    (4, 1, 64, 32, [200, 130], [500, 3], 160),
    (2, 2, 128, 128, [140], [120], None),
]


@pytest.mark.parametrize("case", MMA_CASES)
def test_tensor_core_kernels(case):
    """Requests with several tokens go to the prefill kernel, single tokens to
    the split-key decode kernel, exactly as in a mixed step."""
    from lyapunov_engine_b200 import ops
    nh, nkv, hd, page, q_lens, ctx_before, window = case
    dtype = torch.bfloat16
    c = build_case(dtype, nh, nkv, hd, page, q_lens, ctx_before, seed=hd + page + len(q_lens), window=window)
    assert ops.attention_mma_available(hd)
    status = ops.new_status(DEV)
    multi = [b for b, n in enumerate(q_lens) if n > 1]
    single = [b for b, n in enumerate(q_lens) if n == 1]
    # 3 and 16 splits are merged inside the decode kernel by a cluster of blocks, 24 through scratch memory
    variants = [(1, ops.attention_prefill_bf16), (3, ops.attention_prefill_bf16), (16, ops.attention_prefill_bf16),
                (24, ops.attention_prefill_bf16)]
    if ops.attention_tc_available(hd, page):
        variants.append((2, ops.attention_prefill_tc_bf16))      # the tcgen05 kernel for the requests with several tokens
    for splits, prefill in variants:
        out = torch.full((c["T"], nh * hd), 7.0, dtype=dtype, device=DEV)
        if multi:
            req, q0 = [], []
            for b in multi:
                for s in range(0, q_lens[b], 128):
                    req.append(b); q0.append(s)
            prefill(out, c["q"], c["q"].stride(0), c["k"], c["v"], c["table"], c["cu"], c["ctx"],
                    torch.tensor(req, dtype=torch.int32, device=DEV), torch.tensor(q0, dtype=torch.int32, device=DEV),
                    len(req), nh, nkv, hd, page, window, 1.0 / hd ** 0.5, status)
        if single:
            floats = ops.attention_decode_scratch_floats(hd, len(single), nh, splits)
            scratch = torch.full((max(floats, 1),), float("nan"), device=DEV)
            requests = None if len(single) == len(q_lens) else torch.tensor(single, dtype=torch.int32, device=DEV)
            ops.attention_decode_bf16(out, scratch, c["q"], c["q"].stride(0), c["k"], c["v"], c["table"], c["cu"],
                                      c["ctx"], requests, len(single), nh, nkv, hd, page, window, 1.0 / hd ** 0.5,
                                      splits, status)
        ops.check_status(status)
        torch.testing.assert_close(out.float().cpu(), c["want"], atol=2e-2, rtol=2e-2)


def test_decode_splits_choice():
    """On this device: no choice puts more blocks into a wave than the device
    holds, one split where the batch fills the device by itself, and never
    fewer keys to a split than a split is worth."""
    from lyapunov_engine_b200 import ops
    from lyapunov_engine_b200.parts.attention_kernels import DECODE_KEYS_PER_SPLIT, decode_splits
    for hd in (64, 128):
        whole = ops.attention_decode_resident_blocks(hd, 1)
        assert whole >= ops.sm_count()
        for s in range(2, 9):
            assert 0 < ops.attention_decode_resident_blocks(hd, s) <= whole
        assert decode_splits(1, 32, 8, 100, hd) == 1
        assert decode_splits(64, 32, 8, 4096, hd) == 1
        for n in (1, 2, 3, 5, 7, 8):
            s = decode_splits(n, 32, 8, 4096, hd)
            assert 1 <= s <= 4096 // DECODE_KEYS_PER_SPLIT
            if s > 1:
                assert n * 8 * s <= ops.attention_decode_resident_blocks(hd, s), (hd, n, s)


@pytest.mark.parametrize("splits", [1, 3, 8, 20])
def test_decode_padding_requests_get_zero_rows(splits):
    """A request at position 0 whose table starts with the page nobody owns
    (the pool's last) is padding of a step of fixed shape: its blocks end at
    once, its row comes out as zeros, and the real requests beside it (one of
    them at position 0 too, on a page of its own) get what they get alone."""
    from lyapunov_engine_b200 import ops
    nh, nkv, hd, page = 12, 3, 64, 16
    c = build_case(torch.bfloat16, nh, nkv, hd, page, [1, 1, 1], [700, 0, 95], seed=41)
    status = ops.new_status(DEV)
    null_page = c["k"].shape[0] - 1
    table = torch.cat([c["table"], torch.full((2, c["table"].shape[1]), null_page, dtype=torch.int32, device=DEV)])
    cu = torch.arange(6, dtype=torch.int32, device=DEV)
    ctx = torch.cat([c["ctx"], torch.zeros(2, dtype=torch.int32, device=DEV)])
    q = torch.cat([c["q"], torch.randn(2, c["q"].shape[1], device=DEV).to(torch.bfloat16)])
    out = torch.full((5, nh * hd), 7.0, dtype=torch.bfloat16, device=DEV)
    scratch = torch.full((max(ops.attention_decode_scratch_floats(hd, 5, nh, splits), 1),), float("nan"), device=DEV)
    ops.attention_decode_bf16(out, scratch, q, q.stride(0), c["k"], c["v"], table, cu, ctx, None, 5, nh, nkv, hd, page,
                              None, 1.0 / hd ** 0.5, splits, status)
    ops.check_status(status)
    torch.testing.assert_close(out[:3].float().cpu(), c["want"], atol=2e-2, rtol=2e-2)
    assert bool((out[3:] == 0).all())


def test_decode_many_unsplit_blocks_take_small_tiles():
    """More blocks than the device holds at once and unsplit keys: at head
    size 64 the launcher takes the form of the kernel with 16-key tiles (twice
    as many blocks fit).  Contexts around tile and page edges, one long."""
    from lyapunov_engine_b200 import ops
    nh, nkv, hd, page = 16, 8, 64, 16
    contexts = [0, 1, 15, 16, 17, 31, 32, 33, 47, 48, 63, 64, 65, 100, 127, 128, 129, 255, 256, 700] * 2
    assert len(contexts) * nkv > ops.attention_decode_resident_blocks(hd, 2)
    c = build_case(torch.bfloat16, nh, nkv, hd, page, [1] * len(contexts), contexts, seed=77)
    status = ops.new_status(DEV)
    out = torch.full((c["T"], nh * hd), 7.0, dtype=torch.bfloat16, device=DEV)
    ops.attention_decode_bf16(out, None, c["q"], c["q"].stride(0), c["k"], c["v"], c["table"], c["cu"], c["ctx"], None,
                              len(contexts), nh, nkv, hd, page, None, 1.0 / hd ** 0.5, 1, status)
    ops.check_status(status)
    torch.testing.assert_close(out.float().cpu(), c["want"], atol=2e-2, rtol=2e-2)
