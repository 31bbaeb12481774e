"""Pages far into a large pool: a cache of more than 2^31 elements per tensor,
so that an element offset kept in 32 bits would wrap.  Every kernel that
reads or writes the paged cache gives, with its pages at the end of such a
pool, the bits it gives with the same pages in a small pool."""
import pytest
import torch

import plain_llama
from test_gpu_attention import build_case

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

NH, NKV, HD, PAGE = 32, 8, 64, 16
ELEMENTS_PER_PAGE = NKV * PAGE * HD


def big_pool(small: torch.Tensor, shift: int) -> torch.Tensor:
    """A pool whose pages [shift, shift + len(small)) hold `small`'s pages;
    the rest is left as the allocator gave it."""
    big = torch.empty((shift + small.shape[0],) + tuple(small.shape[1:]), dtype=small.dtype, device=DEV)
    big[shift:] = small
    return big


def test_attention_reads_pages_beyond_2_to_31_elements():
    from lyapunov_engine_b200 import ops
    q_lens, ctx_before = [130, 1, 1, 2], [40, 500, 15, 0]
    c = build_case(torch.bfloat16, NH, NKV, HD, PAGE, q_lens, ctx_before, seed=5)
    shift = (1 << 31) // ELEMENTS_PER_PAGE + 7
    assert shift * ELEMENTS_PER_PAGE > 1 << 31
    scale = 1.0 / HD ** 0.5
    multi = [b for b, n in enumerate(q_lens) if n > 1]
    single = [b for b, n in enumerate(q_lens) if n == 1]
    req = torch.tensor([b for b in multi for _ in range(0, q_lens[b], 128)], dtype=torch.int32, device=DEV)
    q0 = torch.tensor([s for b in multi for s in range(0, q_lens[b], 128)], dtype=torch.int32, device=DEV)
    req16 = torch.tensor([b for b, n in enumerate(q_lens) for _ in range(0, n, 16)], dtype=torch.int32, device=DEV)
    q16 = torch.tensor([s for b, n in enumerate(q_lens) for s in range(0, n, 16)], dtype=torch.int32, device=DEV)
    requests = torch.tensor(single, dtype=torch.int32, device=DEV)

    def run_all(k, v, table):
        status = ops.new_status(DEV)
        outs = {}
        out = torch.zeros(c["T"], NH * HD, dtype=torch.bfloat16, device=DEV)
        ops.attention_generic(out, c["q"], c["q"].stride(0), k, v, table, c["cu"], c["ctx"], req16, q16, len(req16), NH, NKV,
                              HD, PAGE, None, scale, status)
        outs["generic"] = out
        kernels = [("mma", ops.attention_prefill_bf16, 3)]
        if ops.attention_tc_available(HD, PAGE):
            kernels.append(("tcgen05", ops.attention_prefill_tc_bf16, 1))
        for name, prefill, splits in kernels:
            out = torch.zeros(c["T"], NH * HD, dtype=torch.bfloat16, device=DEV)
            prefill(out, c["q"], c["q"].stride(0), k, v, table, c["cu"], c["ctx"], req, q0, len(req), NH, NKV, HD, PAGE,
                    None, scale, status)
            floats = ops.attention_decode_scratch_floats(HD, len(single), NH, splits)
            scratch = torch.zeros(max(floats, 1), device=DEV)
            ops.attention_decode_bf16(out, scratch, c["q"], c["q"].stride(0), k, v, table, c["cu"], c["ctx"], requests,
                                      len(single), NH, NKV, HD, PAGE, None, scale, splits, status)
            outs[name] = out
        ops.check_status(status)
        return outs

    near = run_all(c["k"], c["v"], c["table"])
    k_far, v_far = big_pool(c["k"], shift), big_pool(c["v"], shift)
    far = run_all(k_far, v_far, (c["table"] + shift).contiguous())
    for name in near:
        torch.testing.assert_close(near[name].float().cpu(), c["want"], atol=2e-2, rtol=2e-2)
        assert torch.equal(far[name], near[name]), name


def test_rotary_kernels_write_pages_beyond_2_to_31_elements():
    from lyapunov_engine_b200 import ops
    g = torch.Generator().manual_seed(11)
    M, K = 12, 256
    N = (NH + 2 * NKV) * HD
    x = (torch.randn(M, K, generator=g) * 0.5).bfloat16().to(DEV)
    w = (torch.randn(N, K, generator=g) * K ** -0.5).bfloat16().to(DEV)
    positions = torch.tensor([3 * i % 40 if i % 2 == 0 else 40 + i for i in range(M)], dtype=torch.int32, device=DEV)
    request = torch.tensor([i % 2 for i in range(M)], dtype=torch.int32, device=DEV)
    pages, blocks = 12, 4
    table = torch.randperm(pages, generator=g)[:2 * blocks].to(torch.int32).view(2, blocks).contiguous().to(DEV)
    inv = plain_llama.plain_inv_freq(HD, 10000.0, None)
    ang = torch.outer(torch.arange(64).float(), inv)
    cos_sin = torch.cat([ang.cos(), ang.sin()], -1).contiguous().to(DEV)
    shift = (1 << 31) // ELEMENTS_PER_PAGE + 3
    status = ops.new_status(DEV)
    qkv = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    ops.gemm_skinny(qkv, x, w)

    def run_both(k, v, tbl):
        """(queries, keys, values) after the rotary kernel and after the product with the rotary epilogue"""
        a = qkv.clone()
        ops.rope_kv_write(a, k[0], v[0], cos_sin, positions, request, tbl, NH, NKV, HD, PAGE, True, status)
        b = torch.zeros_like(qkv)
        ops.gemm_skinny_rotary(b, x, w, k[1], v[1], cos_sin, positions, request, tbl, NH, NKV, HD, PAGE, True, status)
        return a[:, :NH * HD], b[:, :NH * HD]

    near_k = [torch.zeros(pages, NKV, PAGE, HD, dtype=torch.bfloat16, device=DEV) for _ in range(2)]
    near_v = [torch.zeros_like(near_k[0]) for _ in range(2)]
    qa, qb = run_both(near_k, near_v, table)
    assert torch.equal(qa, qb) and torch.equal(near_k[0], near_k[1]) and torch.equal(near_v[0], near_v[1])
    assert near_k[0].abs().sum() > 0
    for which in (0, 1):                            # one large pool at a time
        far_k = [None, None]
        far_v = [None, None]
        far_k[which] = big_pool(torch.zeros_like(near_k[0]), shift)
        far_v[which] = big_pool(torch.zeros_like(near_k[0]), shift)
        far_k[1 - which], far_v[1 - which] = torch.zeros_like(near_k[0]), torch.zeros_like(near_k[0])
        tbl = (table + shift).contiguous()
        a = qkv.clone()
        if which == 0:
            ops.rope_kv_write(a, far_k[0], far_v[0], cos_sin, positions, request, tbl, NH, NKV, HD, PAGE, True, status)
        else:
            a = torch.zeros_like(qkv)
            ops.gemm_skinny_rotary(a, x, w, far_k[1], far_v[1], cos_sin, positions, request, tbl, NH, NKV, HD, PAGE, True,
                                   status)
        ops.check_status(status)
        assert torch.equal(a[:, :NH * HD], qa)
        assert torch.equal(far_k[which][shift:], near_k[0]) and torch.equal(far_v[which][shift:], near_v[0])
        del far_k, far_v
        torch.cuda.empty_cache()
