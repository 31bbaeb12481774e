"""Thin Python layer over the kernel libraries (ctypes, raw device pointers).

Every function here launches hand-written sm_100a kernels on the current torch
stream and returns at once.  There is no eager or CPU fallback: tensors must be
CUDA tensors, and when a library cannot be built or loaded the call raises.
The reference pairs every kernel with an eager fallback inside the same
function (python/lyapunov_engine/ops.py:12-216); here the plain twins live in
the tests only.

Matrix products in bfloat16 go to the library (cuBLAS through torch), as the
reference's do (nn.Linear, python/lyapunov_engine/models/llama.py:45-48,112-117,177);
32-bit products use the package's own FP32 kernel, never a tensor-core mode.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_int64, c_void_p

import torch

from . import build

F32, BF16 = 0, 1
STATUS_BITS = {1: "a token id outside the vocabulary", 2: "a block table entry outside the page pool",
               4: "a position outside the rotary table", 8: "a bounded wait inside a kernel ran out"}


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, got {dtype}")


def _ptr(t):
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    """The current stream's handle.  (torch.cuda.current_stream() without a
    device costs tens of microseconds, several times per decode step.)"""
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("lyapunov_engine_b200 kernels run on CUDA tensors only (there is no CPU path)")


_core = None
_attention: dict[int, ctypes.CDLL] = {}

_CORE_SIGNATURES = {
    "le_embed": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p],
    "le_zero_fresh_state": [c_void_p, c_int64, c_int, c_void_p, c_void_p, c_int, c_void_p],
    "le_sm_count": [],
    "le_swiglu": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "le_convert": [c_void_p, c_int, c_void_p, c_int, c_int64, c_void_p],
    "le_rmsnorm": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int64, c_void_p, c_void_p, c_float, c_int,
                   c_int, c_void_p],
    "le_gemm_tc_bf16": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int,
                        c_void_p, c_void_p],
    "le_gemm_skinny_bf16": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int,
                            c_int64, c_int, c_void_p],
    "le_gemm_skinny_rotary_bf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p,
                                   c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                   c_int, c_void_p, c_void_p],
    "le_rope_kv_write": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                         c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "le_gemm_simt": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int64, c_int64, c_int64,
                     c_void_p],
    "le_argmax": [c_void_p, c_void_p, c_int, c_int, c_int64, c_void_p, c_void_p],
    "le_sample": [c_void_p, c_void_p, c_int, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                  c_void_p, c_void_p],
}
_ATTENTION_SIGNATURES = {
    "le_attention_generic": [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_int,
                             c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                             c_float, c_void_p, c_void_p],
}


def _declare(lib, signatures):
    for name, args in signatures.items():
        fn = getattr(lib, name, None)
        if fn is None:
            continue
        fn.argtypes = args
        fn.restype = c_int
    lib.le_last_error_fn = getattr(lib, "le_last_error", None)
    if lib.le_last_error_fn is not None:
        lib.le_last_error_fn.restype = ctypes.c_char_p


def core():
    global _core
    if _core is None:
        lib = build.load_core()
        _declare(lib, _CORE_SIGNATURES)
        _core = lib
    return _core


def attention_lib(head_dim: int):
    lib = _attention.get(head_dim)
    if lib is None:
        lib = build.load_attention(head_dim)
        _declare(lib, _ATTENTION_SIGNATURES)
        _declare(lib, _EXTRA_ATTENTION_SIGNATURES)
        lib.le_attention_mma_available.restype = c_int
        lib.le_attention_mma_available.argtypes = []
        lib.le_attention_tc_available.restype = c_int
        lib.le_attention_tc_available.argtypes = [c_int]
        _attention[head_dim] = lib
    return lib


_EXTRA_ATTENTION_SIGNATURES: dict[str, list] = {
    "le_attention_prefill_bf16": [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                  c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                  c_void_p, c_void_p],
    "le_attention_prefill_tc_bf16": [c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                     c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                     c_int, c_float, c_void_p, c_void_p],
    "le_attention_decode_bf16": [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int,
                                 c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                 c_int, c_void_p, c_void_p],
    "le_attention_decode_bf16_form": [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int,
                                      c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                      c_int, c_int, c_void_p, c_void_p],
}


# Launch counters (own kernels, library products) for the benchmark's report.
counters = {"own_kernels": 0, "library_products": 0}


def _check(code: int, name: str, lib=None, launches: int = 1):
    counters["own_kernels"] += launches
    if code != 0:
        lib = lib or core()
        detail = ""
        fn = getattr(lib, "le_last_error_fn", None) or getattr(core(), "le_last_error_fn", None)
        if fn is not None:
            detail = (fn() or b"").decode(errors="replace")
        raise KernelError(f"{name} failed ({code}): {detail}")


def new_status(device) -> torch.Tensor:
    """The status word kernels set instead of faulting on bad indices."""
    return torch.zeros(4, dtype=torch.int32, device=device)


def check_status(status: torch.Tensor) -> None:
    """Reads the status word (this waits for the device) and raises if a kernel
    met an index it refused to follow."""
    word = int(status[0].item())
    if word:
        status.zero_()
        what = "; ".join(text for bit, text in STATUS_BITS.items() if word & bit)
        raise KernelError(f"a kernel refused bad input: {what}")


# --------------------------------------------------------------------------
def embed(out_resid: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, status: torch.Tensor) -> None:
    """out_resid[t] (float32) = table[ids[t]]."""
    _need_cuda(out_resid, table, ids)
    T, H = out_resid.shape
    assert out_resid.dtype == torch.float32 and ids.dtype == torch.int32 and table.shape[1] == H
    assert out_resid.is_contiguous() and table.is_contiguous()
    _check(core().le_embed(_ptr(out_resid), _ptr(table), dtype_code(table.dtype), _ptr(ids), T, H, table.shape[0],
                           _ptr(status), _stream()), "le_embed")


def zero_fresh_state(state: torch.Tensor, state_slots: torch.Tensor, ctx_before: torch.Tensor, num_requests: int) -> None:
    """Zeroes row ``state_slots[b]`` of ``state`` [rows, ...] for every request b
    of the step that has nothing in the cache yet (``ctx_before[b]`` == 0)."""
    _need_cuda(state, state_slots, ctx_before)
    assert state.is_contiguous() and state_slots.dtype == torch.int32 and ctx_before.dtype == torch.int32
    row_bytes = state[0].numel() * state.element_size()
    _check(core().le_zero_fresh_state(_ptr(state), row_bytes, state.shape[0], _ptr(state_slots), _ptr(ctx_before),
                                      num_requests, _stream()), "le_zero_fresh_state")


_sm_count: dict[int, int] = {}


def sm_count() -> int:
    """Multiprocessors of the current device (148 on a B200)."""
    dev = torch.cuda.current_device()
    n = _sm_count.get(dev)
    if n is None:
        n = int(core().le_sm_count())
        if n <= 0:
            raise KernelError("the device's multiprocessor count could not be read")
        _sm_count[dev] = n
    return n


def swiglu(out: torch.Tensor, gate_up: torch.Tensor) -> None:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]."""
    _need_cuda(out, gate_up)
    T, I = out.shape
    assert gate_up.shape == (T, 2 * I) and out.is_contiguous() and gate_up.is_contiguous()
    assert out.dtype == gate_up.dtype
    _check(core().le_swiglu(_ptr(out), _ptr(gate_up), dtype_code(out.dtype), T, I, _stream()), "le_swiglu")


def convert(out: torch.Tensor, src: torch.Tensor) -> None:
    _need_cuda(out, src)
    assert out.numel() == src.numel() and out.is_contiguous() and src.is_contiguous()
    _check(core().le_convert(_ptr(out), dtype_code(out.dtype), _ptr(src), dtype_code(src.dtype), out.numel(),
                             _stream()), "le_convert")


def rmsnorm(out: torch.Tensor, resid: torch.Tensor, delta, weight: torch.Tensor, eps: float, rows=None) -> None:
    """resid += delta (when given and ``rows`` is None); out = rmsnorm(resid) * weight.
    ``delta`` has the residual stream's shape [T, H] in the activations' type,
    or is float32 [S, T, H]: the partial sums of a split-K product, added in
    order.  With ``rows`` (int32 indices) only those rows are normed, into
    out[0..len(rows)), and ``resid`` is left as it is."""
    _need_cuda(out, resid, delta, weight, rows)
    H = resid.shape[1]
    n = out.shape[0]
    assert resid.dtype == torch.float32 and weight.dtype == torch.float32 and weight.numel() == H
    assert out.shape[1] == H and out.is_contiguous() and resid.is_contiguous()
    parts, stride, dcode = 1, 0, dtype_code(out.dtype)
    if delta is not None:
        assert delta.is_contiguous() and tuple(delta.shape[-2:]) == tuple(resid.shape)
        if delta.dim() == 3:
            assert delta.dtype == torch.float32
            parts, stride = delta.shape[0], delta.stride(0)
        else:
            assert delta.dtype in (out.dtype, torch.float32)
        dcode = dtype_code(delta.dtype)
    if rows is not None:
        assert rows.dtype == torch.int32 and rows.numel() >= n
    else:
        assert n == resid.shape[0]
    _check(core().le_rmsnorm(_ptr(out), dtype_code(out.dtype), _ptr(resid), _ptr(delta), dcode, parts, stride,
                             _ptr(weight), _ptr(rows), float(eps), n, H, _stream()), "le_rmsnorm")


def rope_kv_write(qkv, k_cache, v_cache, cos_sin, positions, request_of_token, block_table, num_heads, num_kv_heads,
                  head_dim, page_size, write_kv, status) -> None:
    """Rotates queries (in place) and keys of the fused qkv rows and writes keys
    and values into the paged cache [pages, kv_heads, page, head_dim]."""
    _need_cuda(qkv, k_cache, cos_sin, positions, block_table)
    T = qkv.shape[0]
    assert qkv.shape[1] == (num_heads + 2 * num_kv_heads) * head_dim and qkv.is_contiguous()
    assert cos_sin.dtype == torch.float32 and cos_sin.is_contiguous()
    assert block_table.dtype == torch.int32 and block_table.is_contiguous()
    max_pos, rot = cos_sin.shape
    if write_kv:
        assert k_cache.dtype == qkv.dtype and k_cache.is_contiguous() and v_cache.is_contiguous()
        assert k_cache.shape[1:] == (num_kv_heads, page_size, head_dim), (k_cache.shape, num_kv_heads, page_size)
    num_pages = k_cache.shape[0] if k_cache is not None else 0
    _check(core().le_rope_kv_write(_ptr(qkv), dtype_code(qkv.dtype), _ptr(k_cache), _ptr(v_cache), _ptr(cos_sin),
                                   _ptr(positions), _ptr(request_of_token), _ptr(block_table), block_table.shape[1],
                                   T, num_heads, num_kv_heads, head_dim, rot, max_pos, page_size, num_pages,
                                   1 if write_kv else 0, _ptr(status), _stream()), "le_rope_kv_write")


def gemm_simt(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor) -> None:
    """out[M, N] = a[M, K] @ w[N, K]^T on the FP32 pipes (inputs float32 or
    bfloat16, 32-bit accumulation in ascending k)."""
    _need_cuda(out, a, w)
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N) and a.dtype == w.dtype
    assert a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    _check(core().le_gemm_simt(_ptr(out), dtype_code(out.dtype), _ptr(a), _ptr(w), dtype_code(a.dtype), M, N, K,
                               a.stride(0), w.stride(0), out.stride(0), _stream()), "le_gemm_simt")


# Up to this many rows a product streams weights through the package's own kernel (mma.sync with the weights as
# the 16-row operand).  Up to 16 rows of x a block takes 16 weight rows, and every product of a decode step runs
# there.  From 17 to 32 rows a block takes 32 or 64 weight rows (so that the slice of x it streams beside them is
# no larger than they are), and the products that are bound by their weights' bytes stay: the gated one (12.5 us
# against 18.6 of the tcgen05 kernel and 13.2 + the activation of the library at the 1B sizes) and the split-K
# ones that feed the residual stream (o 3.9 against 5.7 us of the library, down 9.5 against 13.1); the plain qkv
# product goes to the library there (6.9 against 5.7).  Beyond 32 rows mma.sync is the limit (64 rows: 20.5 us
# gated against 18.5 of the tcgen05 kernel).
SKINNY_ROWS = int(os.environ.get("LYAPUNOV_SKINNY_ROWS", "32"))
SKINNY_NARROW_ROWS = 16   # rows of x up to which a block takes 16 weight rows (and the qkv product its rotary epilogue)
SKINNY_BLOCKS_PER_SM = 512 / 148   # blocks worth having in flight per multiprocessor (512 on a B200: 4 slices of K for 2048 columns, measured best of 1..8)


def skinny_applies(a: torch.Tensor, w: torch.Tensor, rows: int | None = None) -> bool:
    """``rows``: the most rows of x the caller's form is worth it for (SKINNY_ROWS by default)."""
    return (a.dtype == torch.bfloat16 and a.shape[0] <= (SKINNY_ROWS if rows is None else rows) and a.shape[1] % 8 == 0 and a.stride(1) == 1
            and w.stride(1) == 1 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0)


def gemm_skinny(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, splits: int = 1, gated: bool = False) -> None:
    """The package's weight-streaming product for at most 64 rows (bfloat16
    inputs).  ``splits`` > 1: ``out`` is float32 [splits, M, N] partial sums.
    ``gated``: ``w`` is [2 I, K] (gate rows, then up rows), out = silu(gate) * up."""
    _need_cuda(out, a, w)
    M, K = a.shape
    N = w.shape[0]
    if splits > 1:
        assert out.dtype == torch.float32 and out.shape == (splits, M, N) and out.is_contiguous()
        ldo, stride = N, out.stride(0)
    else:
        assert out.shape[-2:] == (M, N // 2 if gated else N) and out.stride(-1) == 1
        ldo, stride = out.stride(-2), 0
    _check(core().le_gemm_skinny_bf16(_ptr(out), dtype_code(out.dtype), _ptr(a), _ptr(w), M, N, K, a.stride(0),
                                      w.stride(0), ldo, splits, stride, 1 if gated else 0, _stream()),
           "le_gemm_skinny_bf16")


FUSE_ROTARY = os.environ.get("LYAPUNOV_FUSE_ROTARY", "1") not in ("0", "")


def rotary_product_applies(a: torch.Tensor, w: torch.Tensor, head_dim: int, rot: int) -> bool:
    """Whether the qkv product, the rotation and the cache write can be one kernel."""
    return skinny_applies(a, w, SKINNY_NARROW_ROWS) and rot == head_dim and head_dim % 16 == 0 and head_dim >= 16


def gemm_skinny_rotary(qkv, a, w, k_cache, v_cache, cos_sin, positions, request_of_token, block_table, num_heads,
                       num_kv_heads, head_dim, page_size, write_kv, status) -> None:
    """The fused qkv projection of at most 64 rows with rotary encoding and
    cache write in its epilogue: rotated queries into ``qkv`` (its key and
    value columns are left alone), rotated keys and the values into the paged
    cache.  Same arithmetic and roundings as linear() then rope_kv_write()."""
    _need_cuda(qkv, a, w, k_cache, cos_sin, positions, block_table)
    M, K = a.shape
    assert M <= 64 and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and cos_sin.shape[1] == head_dim and head_dim % 16 == 0
    assert K % 8 == 0 and a.stride(1) == 1 and w.stride(1) == 1 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
    assert w.shape == ((num_heads + 2 * num_kv_heads) * head_dim, K) and qkv.shape == (M, w.shape[0])
    assert qkv.dtype == torch.bfloat16 and qkv.stride(1) == 1 and cos_sin.dtype == torch.float32 and cos_sin.is_contiguous()
    assert block_table.dtype == torch.int32 and block_table.is_contiguous()
    if write_kv:
        assert k_cache.dtype == torch.bfloat16 and k_cache.is_contiguous() and v_cache.is_contiguous()
        assert k_cache.shape[1:] == (num_kv_heads, page_size, head_dim)
    num_pages = k_cache.shape[0] if k_cache is not None else 0
    _check(core().le_gemm_skinny_rotary_bf16(_ptr(qkv), _ptr(a), _ptr(w), M, K, a.stride(0), w.stride(0), qkv.stride(0),
                                             _ptr(k_cache), _ptr(v_cache), _ptr(cos_sin), _ptr(positions),
                                             _ptr(request_of_token), _ptr(block_table), block_table.shape[1], num_heads,
                                             num_kv_heads, head_dim, cos_sin.shape[0], page_size, num_pages,
                                             1 if write_kv else 0, _ptr(status), _stream()), "le_gemm_skinny_rotary_bf16")


_tc_status = {}


def gemm_tc(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, gated: bool = False, status=None) -> None:
    """The package's tcgen05 / TMA product for many rows (bfloat16 inputs):
    out = a @ w^T (bfloat16 or float32), or with ``gated`` out = silu(a Wg^T) *
    (a Wu^T) for w = [Wg; Wu]."""
    _need_cuda(out, a, w)
    M, K = a.shape
    N = w.shape[0]
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] == K
    assert out.shape == (M, N // 2 if gated else N) and out.stride(1) == 1 and a.stride(1) == 1 and w.stride(1) == 1
    if status is None:
        status = tc_status(a.device)
    _check(core().le_gemm_tc_bf16(_ptr(out), dtype_code(out.dtype), _ptr(a), _ptr(w), M, N, K, a.stride(0), w.stride(0),
                                  out.stride(0), 1 if gated else 0, _ptr(status), _stream()), "le_gemm_tc_bf16")


def tc_status(device) -> torch.Tensor:
    """The status word of the tensor-core product (a bounded wait that ran out sets it)."""
    status = _tc_status.get(torch.device(device))
    if status is None:
        status = _tc_status[torch.device(device)] = new_status(device)
    return status


def tc_applies(a: torch.Tensor, w: torch.Tensor) -> bool:
    return (a.dtype == torch.bfloat16 and a.shape[1] % 8 == 0 and a.stride(1) == 1 and w.stride(1) == 1
            and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


# Plain products with many rows: the package's tcgen05 kernel (one block per SM, 128 x 256 tiles) measures 7-18 %
# behind the library's two-SM kernels on this model's shapes, so they go to the library unless this is set; the
# gated product, where the fused activation more than pays for it, always uses the package's kernel.
TC_PLAIN_PRODUCTS = os.environ.get("LYAPUNOV_TC_PLAIN", "0") not in ("0", "")


def tc_fills_the_gpu(m: int, n: int) -> bool:
    """Whether 128 x 256 tiles of an [m, n] product fill the 148 SMs in whole
    rounds.  The package's kernel has that one tile shape; where it leaves the
    last round mostly empty the library, which picks among many shapes, is
    faster, and a plain product may go to it."""
    tiles = ((m + 127) // 128) * ((n + 255) // 256)
    rounds = (tiles + 147) // 148
    return tiles >= 0.8 * rounds * 148


def split_k_for(n_out: int, k: int, rows: int = 1) -> int:
    """How many slices of K give a product enough blocks to fill the GPU."""
    if rows > SKINNY_NARROW_ROWS:
        # blocks of 64 weight rows, two to a multiprocessor
        blocks = (n_out + 63) // 64
        return max(1, min((2 * sm_count() + blocks - 1) // blocks, k // 256, 16))
    blocks = (n_out + 15) // 16
    in_flight = int(SKINNY_BLOCKS_PER_SM * sm_count() + 0.5)
    return max(1, min((in_flight + blocks - 1) // blocks, k // 512, 16))


def linear_for_residual(a: torch.Tensor, w: torch.Tensor, workspace, key: str, status=None):
    """a @ w^T for a product whose only use is to be added to the residual
    stream: returns either the tensor [M, N] in the activations' type or, for
    few rows, float32 partial sums [S, M, N] that the next norm adds up."""
    M, N = a.shape[0], w.shape[0]
    if skinny_applies(a, w):
        splits = split_k_for(N, a.shape[1], M)
        out = workspace.get(key + "_partials", (splits, M, N), torch.float32)
        if splits == 1:
            gemm_skinny(out[0], a, w)
        else:
            gemm_skinny(out, a, w, splits=splits)
        return out
    out = workspace.get(key, (M, N), a.dtype)
    linear(out, a, w, status)
    return out


def gated_linear(out: torch.Tensor, a: torch.Tensor, w_gate_up: torch.Tensor, workspace, status=None) -> None:
    """out = silu(a @ w_gate^T) * (a @ w_up^T), w_gate_up = [gate rows; up rows].
    bfloat16: one kernel of the package (weight-streaming for few rows, tcgen05
    for many) with the activation in its epilogue."""
    if skinny_applies(a, w_gate_up):
        gemm_skinny(out, a, w_gate_up, gated=True)
        return
    if tc_applies(a, w_gate_up):
        gemm_tc(out, a, w_gate_up, gated=True, status=status)
        return
    gu = workspace.get("gate_up", (a.shape[0], w_gate_up.shape[0]), a.dtype)
    linear(gu, a, w_gate_up, status)
    swiglu(out, gu)


def linear(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, status=None) -> None:
    """out = a @ w^T.  float32: the package's FP32 kernel.  bfloat16 with few
    rows: the package's weight-streaming kernel.  bfloat16 with many rows: the
    package's tcgen05 kernel where its tiles fill the GPU, else the library
    product (cuBLAS); 32-bit accumulation everywhere, and a float32 ``out`` is
    written without an intermediate rounding."""
    if a.dtype == torch.float32:
        gemm_simt(out, a, w)
        return
    _need_cuda(out, a, w)
    if skinny_applies(a, w, SKINNY_NARROW_ROWS):
        gemm_skinny(out, a, w)
        return
    if TC_PLAIN_PRODUCTS and tc_applies(a, w) and tc_fills_the_gpu(a.shape[0], w.shape[0]):
        gemm_tc(out, a, w, status=status)
        return
    if out.dtype == torch.bfloat16:
        counters["library_products"] += 1
        torch.mm(a, w.t(), out=out)
    else:
        gemm_bf16_f32out(out, a, w)


_mm_out_dtype_ok = None


def gemm_bf16_f32out(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor) -> None:
    """bfloat16 inputs, float32 output (the output head's logits)."""
    global _mm_out_dtype_ok
    if _mm_out_dtype_ok is None:
        try:
            torch.mm(a[:1], w[:8].t(), out_dtype=torch.float32)
            _mm_out_dtype_ok = True
        except (TypeError, RuntimeError):
            _mm_out_dtype_ok = False
    K, N = a.shape[1], w.shape[0]
    if _mm_out_dtype_ok and K % 8 == 0 and N % 8 == 0:
        counters["library_products"] += 1
        torch.mm(a, w.t(), out_dtype=torch.float32, out=out)
    else:
        gemm_simt(out, a, w)


def attention_generic(out, q, q_stride, k_cache, v_cache, block_table, cu_q, ctx_before, tile_request, tile_q0,
                      num_tiles, num_heads, num_kv_heads, head_dim, page_size, window, scale, status) -> None:
    _need_cuda(out, q, k_cache, v_cache, block_table)
    lib = attention_lib(head_dim)
    assert out.is_contiguous() and out.shape[1] == num_heads * head_dim
    assert k_cache.shape[1:] == (num_kv_heads, page_size, head_dim)
    _check(lib.le_attention_generic(_ptr(out), out.stride(0), _ptr(q), q_stride, _ptr(k_cache), _ptr(v_cache),
                                    dtype_code(out.dtype), _ptr(block_table), block_table.shape[1], _ptr(cu_q),
                                    _ptr(ctx_before), _ptr(tile_request), _ptr(tile_q0), num_tiles, num_heads,
                                    num_kv_heads, page_size, k_cache.shape[0], int(window or 0), float(scale),
                                    _ptr(status), _stream()), "le_attention_generic", lib)


def attention_mma_available(head_dim: int) -> bool:
    """Whether the tensor-core attention kernels exist for this head size."""
    lib = attention_lib(head_dim)
    return bool(lib.le_attention_mma_available())


def attention_prefill_bf16(out, q, q_stride, k_cache, v_cache, block_table, cu_q, ctx_before, tile_request, tile_q0,
                           num_tiles, num_heads, num_kv_heads, head_dim, page_size, window, scale, status) -> None:
    """Tensor-core attention for requests that bring several tokens; the tiles
    list 128 query tokens each."""
    _need_cuda(out, q, k_cache, v_cache, block_table)
    lib = attention_lib(head_dim)
    assert out.dtype == torch.bfloat16 and out.is_contiguous() and out.shape[1] == num_heads * head_dim
    assert k_cache.dtype == torch.bfloat16 and k_cache.shape[1:] == (num_kv_heads, page_size, head_dim)
    _check(lib.le_attention_prefill_bf16(_ptr(out), out.stride(0), _ptr(q), q_stride, _ptr(k_cache), _ptr(v_cache),
                                         _ptr(block_table), block_table.shape[1], _ptr(cu_q), _ptr(ctx_before),
                                         _ptr(tile_request), _ptr(tile_q0), num_tiles, num_heads, num_kv_heads,
                                         page_size, k_cache.shape[0], int(window or 0), float(scale), _ptr(status),
                                         _stream()), "le_attention_prefill_bf16", lib)


def attention_tc_available(head_dim: int, page_size: int) -> bool:
    """Whether the tcgen05 prefill attention exists for this head and page size."""
    return bool(attention_lib(head_dim).le_attention_tc_available(int(page_size)))


def attention_prefill_tc_bf16(out, q, q_stride, k_cache, v_cache, block_table, cu_q, ctx_before, tile_request, tile_q0,
                              num_tiles, num_heads, num_kv_heads, head_dim, page_size, window, scale, status) -> None:
    """tcgen05 / TMA attention for requests that bring several tokens (head
    sizes 64 and 128, pages of 8..128 keys); the tiles list 128 query tokens
    each.  ``q`` is the [T, width] buffer whose rows start with the query heads."""
    _need_cuda(out, q, k_cache, v_cache, block_table)
    lib = attention_lib(head_dim)
    assert out.dtype == torch.bfloat16 and out.is_contiguous() and out.shape[1] == num_heads * head_dim
    assert k_cache.dtype == torch.bfloat16 and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert k_cache.shape[1:] == (num_kv_heads, page_size, head_dim) and q.dim() == 2 and q.stride(1) == 1
    _check(lib.le_attention_prefill_tc_bf16(_ptr(out), out.stride(0), _ptr(q), q_stride, q.shape[0], q.shape[1],
                                            _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1],
                                            _ptr(cu_q), _ptr(ctx_before), _ptr(tile_request), _ptr(tile_q0), num_tiles,
                                            num_heads, num_kv_heads, page_size, k_cache.shape[0], int(window or 0),
                                            float(scale), _ptr(status), _stream()), "le_attention_prefill_tc_bf16", lib)


def attention_decode_scratch_floats(head_dim: int, num_requests: int, num_heads: int, num_splits: int) -> int:
    return 0 if num_splits <= 1 else num_requests * num_heads * num_splits * (head_dim + 2)


_decode_resident: dict[tuple, int] = {}


def attention_decode_resident_blocks(head_dim: int, num_splits: int, small: bool = False) -> int:
    """Blocks of the split-key decode attention that the current device holds
    at once when the keys are cut ``num_splits`` ways (asked once per size).
    Splits that run as a thread-block cluster come in whole clusters, and fewer
    of those fit than twice the multiprocessor count suggests.  ``small``: of
    the form with 16-key tiles, which the launcher takes where the blocks of the
    usual form (32-key tiles at head sizes up to 64) do not all fit at once."""
    key = (torch.cuda.current_device(), head_dim, num_splits, bool(small))
    n = _decode_resident.get(key)
    if n is None:
        fn = attention_lib(head_dim).le_attention_decode_resident_blocks
        fn.restype, fn.argtypes = c_int, [c_int, c_int]
        n = int(fn(num_splits, 1 if small else 0))
        if n <= 0:
            raise KernelError(f"the device did not say how many decode attention blocks of head size {head_dim} it holds")
        _decode_resident[key] = n
    return n


def attention_decode_bf16(out, scratch, q, q_stride, k_cache, v_cache, block_table, cu_q, ctx_before, requests,
                          num_requests, num_heads, num_kv_heads, head_dim, page_size, window, scale, num_splits,
                          status, small_form=None) -> None:
    """Split-key tensor-core attention for requests that bring one token.
    ``scratch``: float32, attention_decode_scratch_floats(...) elements.
    ``small_form``: None lets the launcher choose between the kernel's usual
    form and the one with 16-key tiles by the number of blocks; a caller that
    knows how many of the requests are real says True or False."""
    _need_cuda(out, q, k_cache, v_cache, block_table, scratch)
    lib = attention_lib(head_dim)
    assert out.dtype == torch.bfloat16 and out.is_contiguous() and out.shape[1] == num_heads * head_dim
    assert k_cache.dtype == torch.bfloat16 and k_cache.shape[1:] == (num_kv_heads, page_size, head_dim)
    if num_splits > 1:
        assert scratch is not None and scratch.dtype == torch.float32
        assert scratch.numel() >= attention_decode_scratch_floats(head_dim, num_requests, num_heads, num_splits)
    form = 0 if small_form is None else (2 if small_form else 1)
    _check(lib.le_attention_decode_bf16_form(_ptr(out), out.stride(0), _ptr(scratch), _ptr(q), q_stride, _ptr(k_cache),
                                             _ptr(v_cache), _ptr(block_table), block_table.shape[1], _ptr(cu_q),
                                             _ptr(ctx_before), _ptr(requests), num_requests, num_heads, num_kv_heads,
                                             page_size, k_cache.shape[0], int(window or 0), float(scale), num_splits,
                                             form, _ptr(status), _stream()), "le_attention_decode_bf16", lib,
           launches=2 if num_splits > 1 else 1)       # the attention kernel and the merge


def argmax_scratch_floats(num_rows: int, vocab: int) -> int:
    return 2 * num_rows * ((vocab + 4095) // 4096)


def argmax(out: torch.Tensor, logits: torch.Tensor, scratch=None) -> None:
    """out[r] = index of the first maximum of logits[r].  ``scratch`` (float32,
    argmax_scratch_floats elements) lets many blocks search one wide row."""
    _need_cuda(out, logits, scratch)
    n, V = logits.shape
    assert logits.dtype == torch.float32 and out.dtype == torch.int32 and logits.stride(1) == 1
    if scratch is not None:
        assert scratch.dtype == torch.float32 and scratch.numel() >= argmax_scratch_floats(n, V)
    two_stages = scratch is not None and (V + 4095) // 4096 >= 4
    _check(core().le_argmax(_ptr(out), _ptr(logits), n, V, logits.stride(0), _ptr(scratch), _stream()), "le_argmax",
           launches=2 if two_stages else 1)


def sample(out, logits, temperature, top_p, top_k, seeds, uniforms=None, probs_out=None) -> None:
    """One token per row of ``logits`` [n, V] float32: greedy where temperature
    < 1e-4, else temperature / top-k / top-p sampling.  ``seeds`` is int32
    [n, 3]: seed low word, seed high word, counter."""
    _need_cuda(out, logits, temperature, top_p, top_k, seeds)
    n, V = logits.shape
    assert logits.dtype == torch.float32 and out.dtype == torch.int32 and logits.stride(1) == 1
    assert temperature.dtype == torch.float32 and top_p.dtype == torch.float32
    assert top_k.dtype == torch.int32 and seeds.dtype == torch.int32
    _check(core().le_sample(_ptr(out), _ptr(logits), n, V, logits.stride(0), _ptr(temperature), _ptr(top_p),
                            _ptr(top_k), _ptr(seeds), _ptr(uniforms), _ptr(probs_out), _stream()), "le_sample")
