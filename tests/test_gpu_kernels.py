"""Each kernel alone against its plain reference (float32 torch ops written
here or in plain_llama.py), at sizes other than the engine's."""
import math

import pytest
import torch

import plain_llama

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def ops():
    from lyapunov_engine_b200 import ops as o
    return o


def tol(dtype):
    return dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,hidden", [(1, 64), (7, 100), (33, 2050), (5, 8192), (3, 13)])
def test_rmsnorm_with_residual(dtype, rows, hidden):
    g = torch.Generator().manual_seed(rows * hidden)
    resid = torch.randn(rows, hidden, generator=g) * 3
    delta = torch.randn(rows, hidden, generator=g).to(dtype)
    w = 1 + 0.1 * torch.randn(hidden, generator=g)
    eps = 1e-6
    r = resid.to(DEV)
    out = torch.empty(rows, hidden, dtype=dtype, device=DEV)
    ops().rmsnorm(out, r, delta.to(DEV), w.to(DEV), eps)
    summed = resid + delta.float()
    torch.testing.assert_close(r.cpu(), summed, atol=1e-6, rtol=1e-6)
    torch.testing.assert_close(out.float().cpu(), plain_llama.plain_rmsnorm(summed, w, eps), **tol(dtype))
    # without delta, and on chosen rows only (the residual stream stays as it is)
    idx = torch.tensor([rows - 1, 0], dtype=torch.int32)
    out2 = torch.empty(2, hidden, dtype=dtype, device=DEV)
    before = r.clone()
    ops().rmsnorm(out2, r, delta.to(DEV), w.to(DEV), eps, rows=idx.to(DEV))
    assert torch.equal(r, before)
    want = plain_llama.plain_rmsnorm(summed + delta.float(), w, eps)[idx.long()]
    torch.testing.assert_close(out2.float().cpu(), want, **tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed_and_bad_token(dtype):
    o = ops()
    table = torch.randn(37, 24).to(dtype)
    ids = torch.tensor([0, 36, 5, 5, 17], dtype=torch.int32)
    status = o.new_status(DEV)
    out = torch.empty(5, 24, device=DEV)
    o.embed(out, table.to(DEV), ids.to(DEV), status)
    assert torch.equal(out.cpu(), table.float()[ids.long()])
    o.check_status(status)
    o.embed(out, table.to(DEV), torch.tensor([1, 37, 2, -1, 3], dtype=torch.int32, device=DEV), status)
    with pytest.raises(o.KernelError, match="token id"):
        o.check_status(status)
    assert torch.equal(out[1].cpu(), torch.zeros(24))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,inter", [(1, 8), (9, 330), (4, 1000)])
def test_swiglu(dtype, rows, inter):
    gu = (torch.randn(rows, 2 * inter) * 3).to(dtype)
    out = torch.empty(rows, inter, dtype=dtype, device=DEV)
    ops().swiglu(out, gu.to(DEV))
    want = plain_llama.plain_swiglu(gu[:, :inter].float(), gu[:, inter:].float())
    torch.testing.assert_close(out.float().cpu(), want, **tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,page,rot", [(4, 2, 16, 4, 16), (3, 1, 48, 8, 48), (5, 5, 128, 16, 128), (2, 1, 64, 2, 32)])
def test_rope_and_cache_write(dtype, nh, nkv, hd, page, rot):
    o = ops()
    g = torch.Generator().manual_seed(hd)
    # two requests: tokens at scattered positions
    positions = torch.tensor([0, 1, 2, 3, 4, 11, 12, 13], dtype=torch.int32)
    request = torch.tensor([0, 0, 0, 0, 0, 1, 1, 1], dtype=torch.int32)
    T = positions.numel()
    pages = 12
    table = torch.tensor([[3, 1, 9, 11, 11, 11, 11], [0, 2, 4, 5, 6, 7, 8]], dtype=torch.int32)
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, generator=g).to(dtype)
    inv = plain_llama.plain_inv_freq(rot, 10000.0, None)
    ang = torch.outer(torch.arange(40).float(), inv)
    cos_sin = torch.cat([ang.cos(), ang.sin()], -1).contiguous()
    k_cache = torch.zeros(pages, nkv, page, hd, dtype=dtype, device=DEV)
    v_cache = torch.zeros_like(k_cache)
    status = o.new_status(DEV)
    dq = qkv.to(DEV)
    o.rope_kv_write(dq, k_cache, v_cache, cos_sin.to(DEV), positions.to(DEV), request.to(DEV), table.to(DEV), nh, nkv,
                    hd, page, True, status)
    o.check_status(status)
    x = qkv.float().view(T, nh + 2 * nkv, hd)
    cos, sin = plain_llama.plain_cos_sin(positions, inv)   # [T, rot]

    def rotate(h):   # [T, heads, hd]
        head = plain_llama.plain_rotate_half(h[..., :rot].transpose(0, 1), cos, sin).transpose(0, 1)
        return torch.cat([head, h[..., rot:]], -1)
    q_want, k_want, v_want = rotate(x[:, :nh]), rotate(x[:, nh:nh + nkv]), x[:, nh + nkv:]
    got = dq.float().cpu().view(T, nh + 2 * nkv, hd)
    torch.testing.assert_close(got[:, :nh], q_want, **tol(dtype))
    kc, vc = k_cache.float().cpu(), v_cache.float().cpu()
    for t in range(T):
        p, b = int(positions[t]), int(request[t])
        pg = int(table[b, p // page])
        torch.testing.assert_close(kc[pg, :, p % page], k_want[t], **tol(dtype))
        torch.testing.assert_close(vc[pg, :, p % page], v_want[t], atol=0, rtol=0)
    # nothing else was touched
    written = torch.zeros(pages, page, dtype=torch.bool)
    for t in range(T):
        p, b = int(positions[t]), int(request[t])
        written[int(table[b, p // page]), p % page] = True
    assert kc.abs().sum((1, 3))[~written].sum() == 0
    # a page id outside the pool is refused, not followed
    bad = table.clone()
    bad[0, 0] = pages
    o.rope_kv_write(dq, k_cache, v_cache, cos_sin.to(DEV), positions.to(DEV), request.to(DEV), bad.to(DEV), nh, nkv,
                    hd, page, True, status)
    with pytest.raises(o.KernelError, match="block table"):
        o.check_status(status)


@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (5, 67, 33), (130, 515, 96), (64, 64, 64), (3, 1000, 136), (257, 70, 328)])
def test_gemm_fp32_pipes(M, N, K):
    g = torch.Generator().manual_seed(M + N + K)
    a, w = torch.randn(M, K, generator=g), torch.randn(N, K, generator=g)
    out = torch.empty(M, N, device=DEV)
    ops().gemm_simt(out, a.to(DEV), w.to(DEV))
    want = (a.double() @ w.double().t()).float()
    torch.testing.assert_close(out.cpu(), want, atol=1e-5 * math.sqrt(K), rtol=1e-5)
    # bfloat16 inputs, 32-bit accumulation
    ab, wb = a.bfloat16(), w.bfloat16()
    out32 = torch.empty(M, N, device=DEV)
    ops().gemm_simt(out32, ab.to(DEV), wb.to(DEV))
    torch.testing.assert_close(out32.cpu(), (ab.double() @ wb.double().t()).float(), atol=1e-5 * math.sqrt(K), rtol=1e-5)


def test_gemm_rows_do_not_depend_on_the_batch():
    """A token's projection is bit-for-bit the same alone and among others."""
    g = torch.Generator().manual_seed(0)
    a, w = torch.randn(77, 200, generator=g).to(DEV), torch.randn(150, 200, generator=g).to(DEV)
    whole = torch.empty(77, 150, device=DEV)
    ops().gemm_simt(whole, a, w)
    for lo, hi in [(0, 1), (5, 6), (63, 70), (76, 77)]:
        part = torch.empty(hi - lo, 150, device=DEV)
        ops().gemm_simt(part, a[lo:hi].contiguous(), w)
        assert torch.equal(part, whole[lo:hi])


@pytest.mark.parametrize("M,N,K", [(4, 515, 96), (33, 1000, 136), (64, 128256 // 64, 256)])
def test_linear_bf16(M, N, K):
    g = torch.Generator().manual_seed(N)
    a, w = torch.randn(M, K, generator=g).bfloat16(), torch.randn(N, K, generator=g).bfloat16()
    want = (a.double() @ w.double().t()).float()
    out32 = torch.empty(M, N, device=DEV)
    ops().linear(out32, a.to(DEV), w.to(DEV))
    torch.testing.assert_close(out32.cpu(), want, atol=1e-3, rtol=1e-4)
    out16 = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    ops().linear(out16, a.to(DEV), w.to(DEV))
    torch.testing.assert_close(out16.float().cpu(), want, atol=0.05, rtol=1e-2)


@pytest.mark.parametrize("M", [17, 64, 2048])
def test_linear_bf16_long_sums_keep_32_bits(M):
    """Products with more than 16 rows go to the library.  Over K = 8192 its
    result must be the 64-bit product of the same bfloat16 inputs rounded once:
    partial sums that passed through bfloat16 (the library's default for
    split-K reductions, which the runtime switches off) would lose bits of
    every slice.  The bound is one rounding of the output, not a percentage."""
    import lyapunov_engine_b200.engine.runtime as runtime

    runtime.Runtime(DEV, torch.bfloat16)        # (building a runtime is what sets the library's accumulation mode)
    assert torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction is False
    K, N = 8192, 2048
    g = torch.Generator().manual_seed(M)
    # inputs with a common sign, so that the sums grow with K and a lost low-order bit shows
    a = (torch.rand(M, K, generator=g) + 0.5).bfloat16()
    w = (torch.rand(N, K, generator=g) + 0.5).bfloat16()
    want = a.double() @ w.double().t()
    out32 = torch.empty(M, N, device=DEV)
    ops().linear(out32, a.to(DEV), w.to(DEV))
    # 32-bit accumulation of 8192 terms of one sign.  The tensor cores' adders truncate instead of rounding to
    # nearest, which shows as a common shortfall of 2.5e-5 here; partial sums rounded to bfloat16 would show as
    # 1e-3 and more (2^-9 per slice of K).
    assert float(((out32.cpu().double() - want) / want).abs().max()) < 1e-4
    out16 = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    ops().linear(out16, a.to(DEV), w.to(DEV))
    # one rounding to bfloat16: at most half a unit in the last place of the result (8 significant bits: a unit
    # is 2^(exponent - 7)), plus the sum's own error
    half_unit = torch.exp2(torch.floor(torch.log2(want)) - 8)
    assert bool(((out16.cpu().double() - want).abs() <= half_unit + 1e-4 * want).all())


@pytest.mark.parametrize("vocab,scratch", [(1003, False), (1003, True), (128256, True), (20001, True)])
def test_argmax_first_of_equal_maxima(vocab, scratch):
    logits = torch.randn(6, vocab)
    logits[2, 17] = logits[2, vocab - 103] = 50.0
    logits[4, vocab - 1] = 60.0
    edge = 4095 if vocab > 4096 else 500          # a tie across the boundary of two blocks' chunks
    logits[5, edge + 1] = logits[5, edge] = 55.0
    out = torch.empty(6, dtype=torch.int32, device=DEV)
    buf = torch.empty(ops().argmax_scratch_floats(6, vocab), device=DEV) if scratch else None
    ops().argmax(out, logits.to(DEV), buf)
    assert out.cpu().tolist() == [plain_llama.plain_greedy(r) for r in logits]
    assert out[2].item() == 17 and out[5].item() == edge


@pytest.mark.parametrize("vocab", [50, 1003, 128256])
def test_sampling_filters_match_the_reference_rule(vocab):
    o = ops()
    g = torch.Generator().manual_seed(vocab)
    n = 6
    logits = torch.randn(n, vocab, generator=g) * 2.5
    temperature = torch.tensor([1.0, 0.7, 1.3, 0.0, 0.5, 2.0])
    top_k = torch.tensor([-1, 5, -1, -1, 40, 0], dtype=torch.int32)
    top_p = torch.tensor([1.0, 1.0, 0.8, 1.0, 0.6, 0.95])
    u = torch.tensor([0.3, 0.999, 0.0, 0.5, 0.42, 0.77])
    seeds = torch.zeros(n, 3, dtype=torch.int32)
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    probs = torch.empty(n, vocab, device=DEV)
    o.sample(out, logits.to(DEV), temperature.to(DEV), top_p.to(DEV), top_k.to(DEV), seeds.to(DEV), u.to(DEV), probs)
    probs, out = probs.cpu(), out.cpu()
    for i in range(n):
        if temperature[i] < 1e-4:
            assert out[i].item() == plain_llama.plain_greedy(logits[i])
            continue
        want = plain_llama.plain_filtered_probs(logits[i], float(temperature[i]), int(top_k[i]), float(top_p[i]))
        assert ((probs[i] > 0) == (want > 0)).all(), f"row {i}: kept sets differ"
        torch.testing.assert_close(probs[i].double(), want, atol=1e-6, rtol=1e-4)
        cdf = torch.cumsum(want, 0)
        k = int(out[i])
        assert want[k] > 0
        lo = float(cdf[k] - want[k]); hi = float(cdf[k])
        assert lo - 1e-4 <= float(u[i]) * float(cdf[-1]) <= hi + 1e-4, f"row {i}: token {k} covers [{lo}, {hi}), u = {u[i]}"


def test_sampling_frequencies_and_batch_independence():
    o = ops()
    vocab, n = 11, 4000
    logits = torch.tensor([2.0, 1.0, 0.5, 0.0, -1.0, 3.0, -2.0, 0.2, 0.1, 1.5, -0.5])
    rows = logits.repeat(n, 1).to(DEV)
    seeds = torch.zeros(n, 3, dtype=torch.int32)
    seeds[:, 0] = 1234
    seeds[:, 2] = torch.arange(n)
    args = (torch.full((n,), 0.9).to(DEV), torch.full((n,), 1.0).to(DEV), torch.full((n,), -1, dtype=torch.int32).to(DEV))
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    o.sample(out, rows, *args, seeds.to(DEV))
    freq = torch.bincount(out.cpu().long(), minlength=vocab).double() / n
    want = plain_llama.plain_filtered_probs(logits, 0.9, -1, 1.0)
    assert (freq - want).abs().max() < 4 * math.sqrt(0.25 / n)
    # the same (seed, counter) gives the same token whatever the batch
    one = torch.empty(1, dtype=torch.int32, device=DEV)
    for i in (0, 17, 3999):
        o.sample(one, rows[i:i + 1], *(a[i:i + 1] for a in args), seeds[i:i + 1].to(DEV))
        assert one.item() == out[i].item()


@pytest.mark.parametrize("M", [1, 5, 8, 13, 16, 29, 64])
@pytest.mark.parametrize("nh,nkv,hd,page,K", [(4, 2, 16, 4, 64), (3, 1, 32, 8, 96), (6, 3, 64, 16, 136), (32, 8, 64, 16, 2048)])
@pytest.mark.parametrize("write", [True, False])
def test_qkv_product_with_rotary_epilogue(M, nh, nkv, hd, page, K, write):
    """The qkv product that rotates and writes the cache itself gives the bits
    of the product followed by the rotary kernel, which has its own test
    against the plain formulas."""
    o = ops()
    g = torch.Generator().manual_seed(M * hd + K)
    N = (nh + 2 * nkv) * hd
    x = (torch.randn(M, K, generator=g) * 0.5).bfloat16().to(DEV)
    w = (torch.randn(N, K, generator=g) * K ** -0.5).bfloat16().to(DEV)
    # two requests at scattered positions, the second far into its pages
    positions = torch.tensor([(i // 2 * 7) % 32 if i % 2 == 0 else 32 + i // 2 for i in range(M)], dtype=torch.int32)   # no slot twice
    request = torch.tensor([i % 2 for i in range(M)], dtype=torch.int32)
    pages = 40
    blocks = (64 + page - 1) // page
    perm = torch.randperm(pages - 1, generator=g)[:2 * blocks].to(torch.int32)
    table = perm.view(2, blocks).contiguous()
    inv = plain_llama.plain_inv_freq(hd, 10000.0, None)
    ang = torch.outer(torch.arange(64).float(), inv)
    cos_sin = torch.cat([ang.cos(), ang.sin()], -1).contiguous().to(DEV)
    status = o.new_status(DEV)
    assert o.rotary_product_applies(x, w, hd, hd) == (M <= o.SKINNY_NARROW_ROWS)      # the engine's choice; the kernel takes 64 rows
    qkv1 = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    k1 = torch.zeros(pages, nkv, page, hd, dtype=torch.bfloat16, device=DEV)
    v1 = torch.zeros_like(k1)
    o.gemm_skinny(qkv1, x, w)
    o.rope_kv_write(qkv1, k1, v1, cos_sin, positions.to(DEV), request.to(DEV), table.to(DEV), nh, nkv, hd, page, write, status)
    qkv2 = torch.full((M, N), 7.0, dtype=torch.bfloat16, device=DEV)
    k2, v2 = torch.zeros_like(k1), torch.zeros_like(k1)
    o.gemm_skinny_rotary(qkv2, x, w, k2, v2, cos_sin, positions.to(DEV), request.to(DEV), table.to(DEV), nh, nkv, hd, page, write, status)
    o.check_status(status)
    assert torch.equal(qkv2[:, :nh * hd], qkv1[:, :nh * hd])
    assert torch.equal(k2, k1) and torch.equal(v2, v1)
    assert (k1.abs().sum() > 0) == write
    # a position outside the table is reported, and nothing of that token is written
    bad = positions.clone()
    bad[0] = 64
    o.gemm_skinny_rotary(qkv2, x, w, k2, v2, cos_sin, bad.to(DEV), request.to(DEV), table.to(DEV), nh, nkv, hd, page, write, status)
    with pytest.raises(o.KernelError):
        o.check_status(status)
    status.zero_()


@pytest.mark.parametrize("M", [1, 8, 9, 16, 33, 64])
@pytest.mark.parametrize("N,K", [(515, 96), (64, 2048), (1000, 136), (48, 328), (2048, 1024)])
def test_skinny_product(M, N, K):
    """The weight-streaming product for few rows: plain, split over K, gated."""
    o = ops()
    g = torch.Generator().manual_seed(M * N + K)
    a = (torch.randn(M, K, generator=g) * 0.5).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.5).bfloat16()
    want = (a.double() @ w.double().t()).float()
    for dtype, tol in ((torch.float32, dict(atol=2e-3, rtol=1e-4)), (torch.bfloat16, dict(atol=0.1, rtol=1e-2))):
        out = torch.full((M, N), 9.0, dtype=dtype, device=DEV)
        o.gemm_skinny(out, a.to(DEV), w.to(DEV))
        torch.testing.assert_close(out.float().cpu(), want, **tol)
    for splits in (2, 5):
        part = torch.full((splits, M, N), 9.0, device=DEV)
        o.gemm_skinny(part, a.to(DEV), w.to(DEV), splits=splits)
        torch.testing.assert_close(part.sum(0).cpu(), want, atol=2e-3, rtol=1e-4)
    if N % 2 == 0:
        act = torch.full((M, N // 2), 9.0, dtype=torch.bfloat16, device=DEV)
        o.gemm_skinny(act, a.to(DEV), w.to(DEV), gated=True)
        torch.testing.assert_close(act.float().cpu(), plain_llama.plain_swiglu(want[:, :N // 2], want[:, N // 2:]),
                                   atol=0.1, rtol=1e-2)


def test_norm_adds_partial_sums_in_order():
    o = ops()
    g = torch.Generator().manual_seed(5)
    resid = torch.randn(7, 264, generator=g)
    parts = torch.randn(3, 7, 264, generator=g)
    w = 1 + 0.1 * torch.randn(264, generator=g)
    r = resid.to(DEV)
    out = torch.empty(7, 264, dtype=torch.bfloat16, device=DEV)
    o.rmsnorm(out, r, parts.to(DEV), w.to(DEV), 1e-5)
    summed = ((resid + parts[0]) + parts[1]) + parts[2]
    assert torch.equal(r.cpu(), summed)
    torch.testing.assert_close(out.float().cpu(), plain_llama.plain_rmsnorm(summed, w, 1e-5), atol=2e-2, rtol=2e-2)
    rows = torch.tensor([6, 2], dtype=torch.int32, device=DEV)
    out2 = torch.empty(2, 264, dtype=torch.bfloat16, device=DEV)
    o.rmsnorm(out2, r, parts.to(DEV), w.to(DEV), 1e-5, rows=rows)
    want = plain_llama.plain_rmsnorm(summed + parts.sum(0), w, 1e-5)[[6, 2]]
    torch.testing.assert_close(out2.float().cpu(), want, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 256, 256), (200, 384, 136), (17, 515 - 3, 96), (1000, 1000, 328),
                                   (2048, 3072, 2048), (130, 8, 8), (1100, 2600, 200), (2304, 4096, 136), (129, 9600, 72)])
def test_tensor_core_product(M, N, K):
    """The tcgen05 / TMA product against a float64 product of the same bfloat16 inputs."""
    o = ops()
    g = torch.Generator().manual_seed(M + N + K)
    a = (torch.randn(M, K, generator=g) * 0.5).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.5).bfloat16()
    want = (a.double() @ w.double().t()).float()
    scale = float(want.abs().max())
    for dtype, tol in ((torch.float32, dict(atol=1e-4 * scale + 1e-4, rtol=1e-4)), (torch.bfloat16, dict(atol=1e-2 * scale, rtol=1e-2))):
        out = torch.full((M, N), 9.0, dtype=dtype, device=DEV)
        o.gemm_tc(out, a.to(DEV), w.to(DEV))
        torch.cuda.synchronize()
        o.check_status(o.tc_status(DEV))
        torch.testing.assert_close(out.float().cpu(), want, **tol)
    if N % 2 == 0:
        act = torch.full((M, N // 2), 9.0, dtype=torch.bfloat16, device=DEV)
        o.gemm_tc(act, a.to(DEV), w.to(DEV), gated=True)
        torch.cuda.synchronize()
        o.check_status(o.tc_status(DEV))
        ref = plain_llama.plain_swiglu(want[:, :N // 2], want[:, N // 2:])
        torch.testing.assert_close(act.float().cpu(), ref, atol=1e-2 * float(ref.abs().max()) + 1e-3, rtol=2e-2)


def test_tensor_core_product_on_a_strided_input():
    """Rows of x that are wider than K (a slice of a fused buffer)."""
    o = ops()
    g = torch.Generator().manual_seed(1)
    big = (torch.randn(300, 256, generator=g) * 0.5).bfloat16().to(DEV)
    a = big[:, 64:192]
    w = (torch.randn(72, 128, generator=g) * 0.5).bfloat16().to(DEV)
    out = torch.empty(300, 72, dtype=torch.float32, device=DEV)
    o.gemm_tc(out, a, w)
    torch.cuda.synchronize()
    torch.testing.assert_close(out.cpu(), (a.double().cpu() @ w.double().cpu().t()).float(), atol=1e-3, rtol=1e-4)
