"""The allocation-free attention entry point, called the way its users call it: through the exported
C symbol `lb_attention_decode_static`, with raw pointers, no scratch argument and no tensor allocator
on the library's side.

Who needs it: a program that may not allocate device memory at the time of the call (a host that
fixed its memory plan at start-up, a latency-critical loop, a caller without torch's allocator).  The
ranges' partial results go into a 4 MiB array inside the library instead of a caller's buffer
(see csrc/include/lb200/attention_decode_static.h).

The test runs two calls in a row with different sizes, so that the second call finds the first call's
leftovers in the shared array, and compares each with the ordinary entry point (`lb_attention_decode`,
scratch allocated by the caller) on the same inputs.  It also checks that a call too large for the
array is refused with its own error code and a message, before anything runs.

This file sorts last on purpose: a run that stops at the first failure has then already run every
other test.
"""
import ctypes
from ctypes import c_char_p, c_float, c_int, c_size_t, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}          # the tolerances of the kernel tests
STATIC_SCRATCH_FLOATS = 1 << 20
ERR_STATIC_SCRATCH = -4


def _case(seed, dtype, Hq, Hkv, hd, page, lengths):
    """One decoded token per request (the last position), keys/values on shuffled pages."""
    g = torch.Generator().manual_seed(seed)
    total_pages = sum(-(-n // page) for n in lengths) + 2
    perm = torch.randperm(total_pages, generator=g).tolist()
    kc = torch.randn(total_pages, page, Hkv, hd, generator=g).to(dtype)
    vc = torch.randn(total_pages, page, Hkv, hd, generator=g).to(dtype)
    bt = torch.full((len(lengths), max(-(-n // page) for n in lengths) + 1), -1, dtype=torch.int32)
    for r, n in enumerate(lengths):
        for p in range(-(-n // page)):
            bt[r, p] = perm.pop()
    q = torch.randn(len(lengths), Hq, hd, generator=g).to(dtype)
    token_req = torch.arange(len(lengths), dtype=torch.int32)
    positions = torch.tensor([n - 1 for n in lengths], dtype=torch.int32)
    return [t.cuda() for t in (q, kc, vc, bt, token_req, positions)]


def _static_entry():
    from logssms_b200.ops import build
    lib = build.load("attention_decode")
    f = lib.lb_attention_decode_static
    f.restype = c_int
    f.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                  c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_void_p, c_char_p, c_size_t]
    return f


def _call_static(f, q, kc, vc, bt, token_req, positions, scale, window, splits):
    out = torch.empty_like(q)
    err = ctypes.create_string_buffer(256)
    code = f(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), out.data_ptr(), bt.data_ptr(), bt.stride(0),
             token_req.data_ptr(), positions.data_ptr(), None, q.shape[0], q.shape[1], kc.shape[2], q.shape[2],
             kc.shape[1], scale, window, splits, 0 if q.dtype == torch.float32 else 1,
             torch.cuda.current_stream().cuda_stream, err, len(err))
    return code, err.value.decode(), out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_static_scratch_entry_matches_the_allocating_one_twice_in_a_row(dtype):
    from logssms_b200.ops import kernels as K
    f = _static_entry()
    calls = [  # seed, Hq, Hkv, hd, page, lengths, splits, window
        (1, 8, 2, 64, 64, [700, 1, 130, 64, 333], 6, 0),
        (2, 6, 3, 48, 16, [90, 257, 17], 3, 100),        # smaller: most of the array still holds call 1's data
    ]
    for seed, Hq, Hkv, hd, page, lengths, splits, window in calls:
        q, kc, vc, bt, token_req, positions = _case(seed, dtype, Hq, Hkv, hd, page, lengths)
        scale = hd ** -0.5
        want = K.attention_decode(q, kc, vc, bt, token_req, positions, scale, window, splits=splits)
        code, msg, got = _call_static(f, q, kc, vc, bt, token_req, positions, scale, window, splits)
        assert code == 0, msg
        torch.cuda.synchronize()
        assert torch.isfinite(got).all()
        err = float((got.double() - want.double()).abs().max() / want.double().abs().max())
        assert err <= TOL[dtype], f"static-scratch attention differs from the allocating entry point: {err:.3g}"


def test_static_scratch_entry_refuses_what_does_not_fit():
    f = _static_entry()
    Hq, Hkv, hd, page = 8, 2, 64, 64
    lengths = [65] * 40
    q, kc, vc, bt, token_req, positions = _case(3, torch.bfloat16, Hq, Hkv, hd, page, lengths)
    splits = STATIC_SCRATCH_FLOATS // (len(lengths) * Hq * (hd + 2)) + 1
    code, msg, _ = _call_static(f, q, kc, vc, bt, token_req, positions, hd ** -0.5, 0, splits)
    assert code == ERR_STATIC_SCRATCH
    assert "scratch" in msg and str(STATIC_SCRATCH_FLOATS) in msg
    code, msg, _ = _call_static(f, q, kc, vc, bt, token_req, positions, hd ** -0.5, 0, splits - 1)
    assert code == 0, msg
    torch.cuda.synchronize()
