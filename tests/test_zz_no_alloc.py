"""The decode attention entry point that brings its own scratch memory
(le_attention_decode_bf16_static), called the way a C caller would: through the
exported symbol, with raw pointers.

It serves callers that cannot allocate device memory when they call: plugins
inside an application that owns all device memory, serving loops that gave
every free byte to their page pool.  Its result must be the one the ordinary
entry point gives with caller-provided scratch; the built-in array is shared by
all calls and keeps the previous call's contents, so two different calls in a
row are checked; and a call that would not fit must be refused, not truncated.

This file is named to be collected last: a run that stops at the first failure
has then already run every other test.
"""
import ctypes
from ctypes import c_float, c_int, c_int64, c_void_p

import pytest
import torch

from test_gpu_attention import DEV, build_case

pytestmark = pytest.mark.gpu

STATIC_ARGS = [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
               c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p]


def symbol(head_dim):
    from lyapunov_engine_b200 import ops
    lib = ops.attention_lib(head_dim)
    fn = lib.le_attention_decode_bf16_static
    fn.argtypes, fn.restype = STATIC_ARGS, c_int
    lib.le_last_error.restype = ctypes.c_char_p
    return lib, fn


def call_static(fn, case, nh, nkv, hd, page, splits, out, status):
    return fn(out.data_ptr(), out.stride(0), case["q"].data_ptr(), case["q"].stride(0), case["k"].data_ptr(),
              case["v"].data_ptr(), case["table"].data_ptr(), case["table"].shape[1], case["cu"].data_ptr(),
              case["ctx"].data_ptr(), None, case["T"], nh, nkv, page, case["k"].shape[0], 0, 1.0 / hd ** 0.5, splits,
              status.data_ptr(), torch.cuda.current_stream().cuda_stream)


def test_static_scratch_entry_point_equals_the_ordinary_one_twice_in_a_row():
    from lyapunov_engine_b200 import ops
    nh, nkv, hd, page = 32, 8, 64, 16
    lib, fn = symbol(hd)
    status = ops.new_status(DEV)
    # two different calls in a row: the second finds the first one's leftovers in the array
    # (more splits than a cluster of blocks merges by itself: those go through the scratch array)
    calls = [([1] * 6, [4095, 17, 0, 63, 64, 1000], 24, 1), ([1] * 3, [300, 2047, 5], 20, 2)]
    for q_lens, ctx_before, splits, seed in calls:
        case = build_case(torch.bfloat16, nh, nkv, hd, page, q_lens, ctx_before, seed=seed)
        floats = ops.attention_decode_scratch_floats(hd, case["T"], nh, splits)
        scratch = torch.empty(floats, device=DEV)
        ordinary = torch.zeros(case["T"], nh * hd, dtype=torch.bfloat16, device=DEV)
        ops.attention_decode_bf16(ordinary, scratch, case["q"], case["q"].stride(0), case["k"], case["v"], case["table"],
                                  case["cu"], case["ctx"], None, case["T"], nh, nkv, hd, page, None, 1.0 / hd ** 0.5,
                                  splits, status)
        static = torch.zeros_like(ordinary)
        rc = call_static(fn, case, nh, nkv, hd, page, splits, static, status)
        assert rc == 0, lib.le_last_error().decode()
        torch.cuda.synchronize()
        ops.check_status(status)
        assert torch.equal(static, ordinary)      # the same kernels on the same inputs: bit for bit
        torch.testing.assert_close(static.float().cpu(), case["want"], atol=2e-2, rtol=2e-2)


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from lyapunov_engine_b200 import ops
    nh, nkv, hd, page = 32, 8, 64, 16
    lib, fn = symbol(hd)
    status = ops.new_status(DEV)
    case = build_case(torch.bfloat16, nh, nkv, hd, page, [1] * 9, [100] * 9, seed=3)
    out = torch.full((case["T"], nh * hd), 5.0, dtype=torch.bfloat16, device=DEV)
    assert ops.attention_decode_scratch_floats(hd, 9, nh, 60) > (1 << 20)
    rc = call_static(fn, case, nh, nkv, hd, page, 60, out, status)
    assert rc == -1
    message = lib.le_last_error().decode()
    assert "floats of scratch" in message and "1048576" in message
    torch.cuda.synchronize()
    assert bool((out == 5.0).all())          # nothing was launched
    assert call_static(fn, case, nh, nkv, hd, page, 1, out, status) == 0   # one split needs no scratch at all
    torch.cuda.synchronize()
    torch.testing.assert_close(out.float().cpu(), case["want"], atol=2e-2, rtol=2e-2)


def test_static_scratch_entry_point_of_a_large_head_library_refuses():
    """Libraries for head sizes above 128 export the symbol and refuse the call."""
    lib, fn = symbol(256)
    assert fn(None, 0, None, 0, None, None, None, 0, None, None, None, 1, 4, 2, 16, 8, 0, 1.0, 2, None, None) == -1
    assert "head sizes up to 128" in lib.le_last_error().decode()
