"""The allocation-free decode matmul (magb200_matmul_skinny_noalloc) against the regular entry point.

It exists for callers that may not call cudaMalloc -- code running inside another framework's stream-ordered
region, or a serving loop that must leave the allocator alone once warm. Its split-K partial sums live in an
array inside the library instead of an allocated workspace, and that array keeps the previous call's
contents, so the check is made on two calls in a row with different activations: both must equal what
magb200_matmul gives for the same operands, bit for bit. This file sorts last on purpose: a run that stops
at the first failure has then already run every other test."""
import ctypes as C

import numpy as np
import pytest

import magnetron_b200 as mb
from oracle import mag_oracle as O
from tests import cases

pytestmark = pytest.mark.gpu


def test_noalloc_matches_regular_entry_point_twice_in_a_row(gpu):
    L = mb.lib()
    dt = O.BFLOAT16
    M, N, K = 8, 5120, 25600          # long K: the kernel splits K and goes through the scratch array
    rng = np.random.default_rng(31)
    wb = O.f32_to_bits(dt, cases.gen_storage(rng, (N, K), 0.02))
    tw = mb.Tensor.from_bits(gpu, dt, wb)
    stream = L.magb200_get_stream(gpu)

    def free_bytes():
        f, t = C.c_uint64(), C.c_uint64()
        mb.check(L.magb200_mem_info(gpu, C.byref(f), C.byref(t)))
        return f.value

    for call in range(2):
        xb = O.f32_to_bits(dt, cases.gen_storage(rng, (M, K), 1.0 + call))
        tx = mb.Tensor.from_bits(gpu, dt, xb)
        want = tx @ tw.T
        assert mb.last_kernel() == "skinny_splitk"
        want_bits = want.to_bits()
        out = mb.Tensor(gpu, dt, (M, N))
        mb.check(L.magb200_fill(gpu, C.byref(out.view_struct()), 0.0))
        mb.synchronize(gpu)
        before = free_bytes()
        mb.check(L.magb200_matmul_skinny_noalloc(gpu, stream, C.byref(tx.view_struct()), C.byref(tw.T.view_struct()),
                                                 C.byref(out.view_struct())))
        mb.synchronize(gpu)
        # the very first call on a device may load the library's code for this entry point, built-in array included (the
        # driver loads modules on first use); from then on the amount of free device memory must not move
        if call > 0:
            assert free_bytes() == before, "the allocation-free entry point changed the amount of free device memory"
        got = out.to_bits()
        assert np.array_equal(got, want_bits), f"call {call}: {np.count_nonzero(got != want_bits)} elements differ"
        # and the result is right, not merely the same: fp64 truth on sampled columns
        cols = rng.integers(0, N, 64)
        x, w = O.bits_to_f64(dt, xb), O.bits_to_f64(dt, wb[cols])
        m = O.error_metrics(dt, got[:, cols], x @ w.T, np.abs(x) @ np.abs(w).T)
        assert m["e"] <= 2.0 ** -8 + K * 2.0 ** -24, m
        for t in (out, want, tx):
            t.release()
    tw.release()


def test_noalloc_refuses_what_does_not_fit(gpu):
    L = mb.lib()
    dt = O.BFLOAT16
    # 8 x 65536 outputs with K split several ways: more partial sums than the built-in array holds
    x = mb.Tensor(gpu, dt, (8, 16384))
    w = mb.Tensor(gpu, dt, (65536, 16384))
    out = mb.Tensor(gpu, dt, (8, 65536))
    rc = L.magb200_matmul_skinny_noalloc(gpu, L.magb200_get_stream(gpu), C.byref(x.view_struct()), C.byref(w.T.view_struct()),
                                         C.byref(out.view_struct()))
    assert rc == mb.ERR_TOO_LARGE and b"built-in scratch array" in L.magb200_last_error()
    # a prefill-shaped problem is not what this entry point is for
    x2 = mb.Tensor(gpu, dt, (64, 256))
    w2 = mb.Tensor(gpu, dt, (128, 256))
    out2 = mb.Tensor(gpu, dt, (64, 128))
    rc = L.magb200_matmul_skinny_noalloc(gpu, L.magb200_get_stream(gpu), C.byref(x2.view_struct()), C.byref(w2.T.view_struct()),
                                         C.byref(out2.view_struct()))
    assert rc == mb.ERR_INVALID_ARG
    for t in (x, w, out, x2, w2, out2):
        t.release()
