"""GPU tests of the parts of the matmul path that are about scheduling and failure handling rather than arithmetic:
weight operands that are themselves fresh results of the decode kernels,
the bounded device-side waits, the device memory pool, non-finite operands, and more than one device per process."""
import ctypes as C

import numpy as np
import pytest

import magnetron_b200 as mb
from oracle import mag_oracle as O
from tests import cases
from tests.common import unit_roundoff

pytestmark = pytest.mark.gpu


def bits(dt, rng, shape, scale):
    return O.f32_to_bits(dt, cases.gen_storage(rng, shape, scale))


# (M, N, K, weight layout): 256 x 256 tiles on 74 CTA pairs
BALANCED_SHAPES = [
    (2560, 2048, 2048, "wT"),    # 80 tiles: one full wave, 6 tiles shared by 48 pairs (8 runs per tile)
    (2560, 2560, 1024, "wT"),    # 100 tiles: 26 shared by 52 pairs (cap: 2 runs per tile)
    (4096, 4096, 4096, "wT"),    # 256 tiles: 34 shared by 74 pairs, runs cross tile boundaries
    (2048, 2048, 4096, "wT"),    # 64 tiles, less than a wave: all of them shared by 74 pairs
    (2560, 2000, 1416, "wT"),    # ragged N and K
    (2560, 2048, 1024, "kn"),    # contiguous [K,N] weight (N-major B)
    (2560, 2048, 256, "wT"),     # too few K groups to share: falls back to whole tiles
]


@pytest.mark.parametrize("M,N,K,layout", BALANCED_SHAPES)
@pytest.mark.parametrize("dname", ["bf16", "f16"])
def test_shared_last_wave(gpu, M, N, K, layout, dname):
    """The two-SM kernel shares the tiles of a partial last wave among all CTA pairs along K (fp32 partials, fixed order).
    The result must be reproducible bit for bit, meet the accuracy bar against fp64 on sampled rows, and differ from the
    unshared schedule only in a few elements (the fp32 sum is associated differently, which can move the last bit)."""
    dt = cases.DTYPES[dname]
    L = mb.lib()
    rng = np.random.default_rng(41)
    xb = bits(dt, rng, (M, K), 1.0)
    wb = bits(dt, rng, (N, K) if layout == "wT" else (K, N), 0.1)
    tx, tw = mb.Tensor.from_bits(gpu, dt, xb), mb.Tensor.from_bits(gpu, dt, wb)
    y = tw.T if layout == "wT" else tw
    mb.force_kernel("tcgen05_2sm")
    try:
        mb.check(L.magb200_set_balanced_last_wave(2))      # share whenever the shape allows, not only where it pays
        r1 = tx @ y
        assert mb.last_kernel() == "tcgen05_2sm"
        got = r1.to_bits()
        r2 = tx @ y
        again = r2.to_bits()
        mb.check(L.magb200_set_balanced_last_wave(0))
        r0 = tx @ y
        plain = r0.to_bits()
    finally:
        mb.check(L.magb200_set_balanced_last_wave(1))
        mb.force_kernel(None)
    assert np.array_equal(got, again), "two runs of the shared last wave differ"
    differ = got != plain
    assert differ.mean() < 0.05, differ.mean()
    rows = np.unique(np.concatenate([[0, 255, 256, M - 257, M - 1], rng.integers(0, M, 27)]))
    wf = O.bits_to_f64(dt, wb)
    wkn = wf.T if layout == "wT" else wf
    xf = O.bits_to_f64(dt, xb[rows])
    m = O.error_metrics(dt, got[rows], xf @ wkn, np.abs(xf) @ np.abs(wkn))
    assert m["e"] <= unit_roundoff(dt) + K * 2.0 ** -24, m
    for t in (r0, r1, r2, tx, tw):
        t.release()


def test_back_to_back_gemms_overlap_only_when_independent(gpu):
    """Consecutive magb200_matmul calls: products that share nothing but read-only operands are launched so that they may run
    side by side (counted), and give the bits of the fully ordered launches; a product that reads the result of the one
    before it, one that overwrites an operand of the one before it, one that writes the same result again, and a product
    after any other operation are ordered (not counted) -- and right."""
    dt = O.BFLOAT16
    L = mb.lib()
    rng = np.random.default_rng(41)
    M, N, K = 1024, 1024, 1024
    xb = bits(dt, rng, (M, K), 1.0)
    wbs = [bits(dt, rng, (N, K), 0.05) for _ in range(5)]
    tx = mb.Tensor.from_bits(gpu, dt, xb)
    tws = [mb.Tensor.from_bits(gpu, dt, w) for w in wbs]
    outs = [mb.Tensor(gpu, dt, (M, N)) for _ in range(5)]
    xv = tx.view_struct()
    wv = [w.T.view_struct() for w in tws]
    ov = [o.view_struct() for o in outs]

    def run_independent():
        mb.synchronize(gpu)
        before = L.magb200_overlapped_launch_count()
        for i in range(5):
            mb.check(L.magb200_matmul(gpu, C.byref(xv), C.byref(wv[i]), C.byref(ov[i])))
        n = L.magb200_overlapped_launch_count() - before
        mb.synchronize(gpu)
        return n, [o.to_bits() for o in outs]

    try:
        mb.check(L.magb200_set_gemm_overlap(1))
        n_on, got_on = run_independent()
        mb.check(L.magb200_set_gemm_overlap(0))
        n_off, got_off = run_independent()
        assert n_on == 4 and n_off == 0
        for a, b in zip(got_on, got_off):
            assert np.array_equal(a, b)
        mb.check(L.magb200_set_gemm_overlap(1))
        # a chain of dependent products: out0 = x @ w0.T, out1 = out0 @ w1.T, out2 = out1 @ w2.T
        mb.synchronize(gpu)
        before = L.magb200_overlapped_launch_count()
        mb.check(L.magb200_matmul(gpu, C.byref(xv), C.byref(wv[0]), C.byref(ov[0])))
        mb.check(L.magb200_matmul(gpu, C.byref(ov[0]), C.byref(wv[1]), C.byref(ov[1])))
        mb.check(L.magb200_matmul(gpu, C.byref(ov[1]), C.byref(wv[2]), C.byref(ov[2])))
        # overwrites an operand of the product before it (out1), then writes the same result again
        mb.check(L.magb200_matmul(gpu, C.byref(xv), C.byref(wv[3]), C.byref(ov[1])))
        mb.check(L.magb200_matmul(gpu, C.byref(xv), C.byref(wv[4]), C.byref(ov[1])))
        assert L.magb200_overlapped_launch_count() == before
        mb.synchronize(gpu)
        f = lambda b: O.bits_to_f64(dt, b)
        r0 = f(O.f32_to_bits(dt, (f(xb) @ f(wbs[0]).T).astype(np.float32)))
        assert np.array_equal(outs[0].to_bits(), got_on[0])
        r1 = f(outs[0].to_bits()) @ f(wbs[1]).T
        # out2 was computed from the out1 of the chain, before out1 was overwritten
        chain1 = O.f32_to_bits(dt, r1.astype(np.float32))
        r2 = f(chain1) @ f(wbs[2]).T
        got2 = f(outs[2].to_bits())
        assert np.max(np.abs(got2 - r2)) <= 2.0 ** -7 * np.max(np.abs(r2)) + 1e-6
        assert np.array_equal(outs[1].to_bits(), got_on[4])                       # the last writer of out1 was x @ w4.T
        # another operation in between (a fill of an unrelated tensor) closes the run: the product behind it is ordered
        before = L.magb200_overlapped_launch_count()
        other = mb.Tensor(gpu, dt, (64,))
        mb.check(L.magb200_matmul(gpu, C.byref(xv), C.byref(wv[0]), C.byref(ov[0])))
        mb.check(L.magb200_fill(gpu, C.byref(other.view_struct()), C.c_double(1.0)))
        mb.check(L.magb200_matmul(gpu, C.byref(xv), C.byref(wv[2]), C.byref(ov[2])))
        assert L.magb200_overlapped_launch_count() == before
        mb.synchronize(gpu)
        assert np.array_equal(outs[2].to_bits(), got_on[2])
        # a contiguous cast of an uninvolved tensor behind a product joins the run; a cast of that product's result does not
        before = L.magb200_overlapped_launch_count()
        f32 = mb.Tensor(gpu, mb.FLOAT32, (M, K))
        f32b = mb.Tensor(gpu, mb.FLOAT32, (M, N))
        mb.check(L.magb200_matmul(gpu, C.byref(xv), C.byref(wv[0]), C.byref(ov[0])))
        mb.check(L.magb200_cast(gpu, C.byref(xv), C.byref(f32.view_struct())))
        assert L.magb200_overlapped_launch_count() == before + 1
        mb.check(L.magb200_cast(gpu, C.byref(ov[0]), C.byref(f32b.view_struct())))
        assert L.magb200_overlapped_launch_count() == before + 1
        mb.synchronize(gpu)
        assert np.array_equal(f32.to_bits(), O.cast_bits(dt, O.FLOAT32, xb))
        assert np.array_equal(f32b.to_bits(), O.cast_bits(dt, O.FLOAT32, got_on[0]))
        for t in (other, f32, f32b):
            t.release()
    finally:
        mb.check(L.magb200_set_gemm_overlap(1))
    for t in [tx] + tws + outs:
        t.release()


@pytest.mark.parametrize("dname", ["bf16", "f16"])
@pytest.mark.parametrize("batch,M,N,K", [((), 512, 2048, 2048), ((), 128, 128, 1024), ((), 300, 200, 1096), ((2, 3), 130, 136, 4160)])
def test_small_outputs_split_k_over_cta_pairs(gpu, dname, batch, M, N, K):
    """Outputs of at most 74 tiles of 128 x 128 with a long K: two CTAs per tile split K and exchange accumulator halves through
    distributed shared memory. Against fp64 within the own bar, reproducible, and within two roundings of the one-CTA-per-tile
    result; ragged M, N, K and batches included."""
    dt = cases.DTYPES[dname]
    L = mb.lib()
    rng = np.random.default_rng(35)
    xb, wb = bits(dt, rng, batch + (M, K), 1.0), bits(dt, rng, (N, K), 0.05)
    tx, tw = mb.Tensor.from_bits(gpu, dt, xb), mb.Tensor.from_bits(gpu, dt, wb)
    xf, wf = O.bits_to_f64(dt, xb), O.bits_to_f64(dt, wb)
    truth, scale = xf @ wf.T, np.abs(xf) @ np.abs(wf).T
    got = {}
    mb.force_kernel("tcgen05")
    try:
        for on in (1, 0):
            mb.check(L.magb200_set_small_output_split(on))
            r1, r2 = tx @ tw.T, tx @ tw.T
            got[on] = r1.to_bits()
            assert np.array_equal(got[on], r2.to_bits())
            m = O.error_metrics(dt, got[on], truth, scale)
            assert m["e"] <= unit_roundoff(dt) + K * 2.0 ** -24, (on, m)
            r1.release(); r2.release()
    finally:
        mb.force_kernel(None)
        mb.check(L.magb200_set_small_output_split(1))
    a, b = O.bits_to_f64(dt, got[1]), O.bits_to_f64(dt, got[0])
    assert np.all(np.abs(a - b) <= 2 * unit_roundoff(dt) * np.maximum(np.abs(a), np.abs(b)) + 2.0 ** -20 * scale)
    for t in (tx, tw):
        t.release()


@pytest.mark.parametrize("dname", ["bf16", "f16"])
@pytest.mark.parametrize("batch,M,N,K", [((), 1, 40000, 1024), ((), 8, 39992, 1031), ((), 4, 12288, 4096), ((), 5, 136, 777), ((3,), 2, 1000, 300),
                                         ((), 8, 8, 20)])
def test_decode_with_n_major_weights(gpu, dname, batch, M, N, K):
    """y = a contiguous [K, N] weight (the layout of the reference's GEMV fast path, magnetron/cpu/mag_cpu_impl_ops_matmul.inl:2940):
    the mma.sync kernel with transposing fragment loads against fp64 within the own bar, reproducible, and within two roundings
    of the FFMA kernel; K not a multiple of 8 or 16, ragged strips, K split across CTAs, batches."""
    dt = cases.DTYPES[dname]
    L = mb.lib()
    rng = np.random.default_rng(39)
    xb, wb = bits(dt, rng, batch + (M, K), 1.0), bits(dt, rng, (K, N), 0.05)
    tx, tw = mb.Tensor.from_bits(gpu, dt, xb), mb.Tensor.from_bits(gpu, dt, wb)
    xf, wf = O.bits_to_f64(dt, xb), O.bits_to_f64(dt, wb)
    truth, scale = xf @ wf, np.abs(xf) @ np.abs(wf)
    got = {}
    try:
        for on in (1, 0):
            mb.check(L.magb200_set_decode_row_streaming(on))
            r1, r2 = tx @ tw, tx @ tw
            assert mb.last_kernel() in ("skinny", "skinny_splitk")
            got[on] = r1.to_bits()
            assert np.array_equal(got[on], r2.to_bits())
            m = O.error_metrics(dt, got[on], truth, scale)
            assert m["e"] <= unit_roundoff(dt) + K * 2.0 ** -24, (on, m)
            r1.release(); r2.release()
    finally:
        mb.check(L.magb200_set_decode_row_streaming(1))
    a, b = O.bits_to_f64(dt, got[1]), O.bits_to_f64(dt, got[0])
    assert np.all(np.abs(a - b) <= 2 * unit_roundoff(dt) * np.maximum(np.abs(a), np.abs(b)) + 2.0 ** -20 * scale)
    for t in (tx, tw):
        t.release()


@pytest.mark.parametrize("dname", ["bf16", "f16"])
@pytest.mark.parametrize("M,N,K", [(1, 40000, 1024), (8, 39993, 1032), (3, 24000, 4096), (8, 20000, 5120), (2, 50000, 264)])
def test_decode_streaming_kernels_agree(gpu, dname, M, N, K):
    """Weight matrices with plenty of rows: the row-contiguous streaming kernel and the per-lane-ring kernel against fp64 within
    the own bar, each reproducible, and within two roundings of each other; ragged N, K not a multiple of the 256-wide step,
    and a K that needs a split across CTAs."""
    dt = cases.DTYPES[dname]
    L = mb.lib()
    rng = np.random.default_rng(37)
    xb, wb = bits(dt, rng, (M, K), 1.0), bits(dt, rng, (N, K), 0.05)
    tx, tw = mb.Tensor.from_bits(gpu, dt, xb), mb.Tensor.from_bits(gpu, dt, wb)
    xf, wf = O.bits_to_f64(dt, xb), O.bits_to_f64(dt, wb)
    truth, scale = xf @ wf.T, np.abs(xf) @ np.abs(wf).T
    got = {}
    try:
        for on in (1, 0):
            mb.check(L.magb200_set_decode_row_streaming(on))
            r1, r2 = tx @ tw.T, tx @ tw.T
            assert mb.last_kernel() in ("skinny", "skinny_splitk")
            got[on] = r1.to_bits()
            assert np.array_equal(got[on], r2.to_bits())
            m = O.error_metrics(dt, got[on], truth, scale)
            assert m["e"] <= unit_roundoff(dt) + K * 2.0 ** -24, (on, m)
            r1.release(); r2.release()
    finally:
        mb.check(L.magb200_set_decode_row_streaming(1))
    a, b = O.bits_to_f64(dt, got[1]), O.bits_to_f64(dt, got[0])
    assert np.all(np.abs(a - b) <= 2 * unit_roundoff(dt) * np.maximum(np.abs(a), np.abs(b)) + 2.0 ** -20 * scale)
    for t in (tx, tw):
        t.release()


@pytest.mark.parametrize("M", [1, 5, 8])
@pytest.mark.parametrize("N,K", [(1024, 2048), (1024, 3072), (1000, 4104), (48, 8192)])
def test_decode_clusters_split_k_like_one_cta(gpu, M, N, K):
    """Weight matrices with few 16-row tiles run as clusters of 2 or 4 CTAs that split K and meet through distributed shared
    memory: against fp64 within the usual bar, reproducible, and within two roundings of the one-CTA result."""
    dt = O.BFLOAT16
    L = mb.lib()
    rng = np.random.default_rng(33)
    xb, wb = bits(dt, rng, (M, K), 1.0), bits(dt, rng, (N, K), 0.05)
    tx, tw = mb.Tensor.from_bits(gpu, dt, xb), mb.Tensor.from_bits(gpu, dt, wb)
    xf, wf = O.bits_to_f64(dt, xb), O.bits_to_f64(dt, wb)
    truth, scale = xf @ wf.T, np.abs(xf) @ np.abs(wf).T
    got = {}
    try:
        for cl in (1, 2, 4):
            mb.check(L.magb200_set_decode_cluster(cl))
            r1, r2 = tx @ tw.T, tx @ tw.T
            assert mb.last_kernel() in ("skinny", "skinny_splitk")
            got[cl] = r1.to_bits()
            assert np.array_equal(got[cl], r2.to_bits())
            m = O.error_metrics(dt, got[cl], truth, scale)
            assert m["e"] <= unit_roundoff(dt) + K * 2.0 ** -24, (cl, m)
            r1.release(); r2.release()
    finally:
        mb.check(L.magb200_set_decode_cluster(4))
    a, b = O.bits_to_f64(dt, got[1]), O.bits_to_f64(dt, got[4])
    assert np.all(np.abs(a - b) <= 2 * unit_roundoff(dt) * np.maximum(np.abs(a), np.abs(b)) + 2.0 ** -20 * scale)
    for t in (tx, tw):
        t.release()
    assert L.magb200_set_decode_cluster(3) != 0


@pytest.mark.parametrize("M", [1, 3, 8])
@pytest.mark.parametrize("dname", ["bf16", "f16"])
def test_grouped_decode_matches_separate_calls(gpu, M, dname):
    """q/k/v and gate/up of a decode step as one grouped launch each: bit-identical to the separate matmuls when both cut K the
    same way (within two roundings otherwise), also when a weight's row count is not a multiple of the 16-row tile, and a group that cannot be one launch (a prefill-shaped x)
    still gives the separate calls' results."""
    dt = cases.DTYPES[dname]
    L = mb.lib()
    rng = np.random.default_rng(19)
    K = 1024
    xb = bits(dt, rng, (M, K), 1.0)
    tx = mb.Tensor.from_bits(gpu, dt, xb)
    for Ns in ((2048, 1024, 1024), (3072, 3072), (1000, 24, 520, 8)):
        ws = [mb.Tensor.from_bits(gpu, dt, bits(dt, rng, (N, K), 0.05)) for N in Ns]
        want = [(tx @ w.T).to_bits() for w in ws]
        outs = [mb.Tensor(gpu, dt, (M, N)) for N in Ns]
        for o in outs:
            mb.check(L.magb200_fill(gpu, C.byref(o.view_struct()), 0.0))
        yv = [w.T.view_struct() for w in ws]
        rv = [o.view_struct() for o in outs]
        ys = (C.POINTER(mb.View) * len(Ns))(*[C.pointer(v) for v in yv])
        rs = (C.POINTER(mb.View) * len(Ns))(*[C.pointer(v) for v in rv])
        L.magb200_launch_count_reset()
        mb.check(L.magb200_matmul_grouped(gpu, C.byref(tx.view_struct()), len(Ns), ys, rs))
        assert L.magb200_launch_count() == 1, "the group did not run as one launch"
        mb.synchronize(gpu)
        same_slicing = sum((N + 15) // 16 for N in Ns) <= 296      # else the group cuts K into fewer slices than a member alone
        for o, wnt in zip(outs, want):
            if same_slicing:
                assert np.array_equal(o.to_bits(), wnt)
            else:
                a, b = O.bits_to_f64(dt, o.to_bits()), O.bits_to_f64(dt, wnt)
                assert np.all(np.abs(a - b) <= 2 * unit_roundoff(dt) * np.maximum(np.abs(a), np.abs(b)) + 1e-3 * unit_roundoff(dt) * K)
                assert np.mean(a != b) < 0.2
        for t in ws + outs:
            t.release()
    # prefill-shaped: falls back to one matmul per product
    xb2 = bits(dt, rng, (64, 256), 1.0)
    tx2 = mb.Tensor.from_bits(gpu, dt, xb2)
    ws = [mb.Tensor.from_bits(gpu, dt, bits(dt, rng, (N, 256), 0.05)) for N in (128, 64)]
    want = [(tx2 @ w.T).to_bits() for w in ws]
    outs = [mb.Tensor(gpu, dt, (64, N)) for N in (128, 64)]
    yv = [w.T.view_struct() for w in ws]
    rv = [o.view_struct() for o in outs]
    mb.check(L.magb200_matmul_grouped(gpu, C.byref(tx2.view_struct()), 2, (C.POINTER(mb.View) * 2)(*[C.pointer(v) for v in yv]),
                                      (C.POINTER(mb.View) * 2)(*[C.pointer(v) for v in rv])))
    for o, wnt in zip(outs, want):
        assert np.array_equal(o.to_bits(), wnt)
    for t in ws + outs + [tx, tx2]:
        t.release()


PACK_CASES = [
    # name, x storage, x view recipe, w storage, w view recipe (applied before .T)
    ("odd_k", (640, 1001), [], (512, 1001), []),                                        # row pitch 2002 bytes: both operands are packed
    ("inner_stride_2", (640, 2048), [("slice", 1, 0, 1024, 2)], (512, 1024), []),       # x[:, ::2]: only x is packed
    ("misaligned_slice", (640, 1032), [("slice", 1, 3, 1024, 1)], (512, 1024), []),     # x[:, 3:1027]: base 6 bytes off a 16-byte boundary
    ("batched_broadcast_w", (3, 300, 1001), [], (520, 1001), []),                       # batch folds into M = 900
]


@pytest.mark.parametrize("name,xs,xops,ws,wops", PACK_CASES)
@pytest.mark.parametrize("dname", ["bf16", "f16"])
def test_operands_tma_cannot_describe_are_packed_on_the_device(gpu, name, xs, xops, ws, wops, dname):
    """16-bit operands with an odd row pitch, an inner stride of 2 or a misaligned base cannot be read by TMA. Large enough
    problems are repacked on the device and still run on the tensor cores instead of the FFMA kernel."""
    dt = cases.DTYPES[dname]
    rng = np.random.default_rng(29)
    xb, wb = bits(dt, rng, xs, 1.0), bits(dt, rng, ws, 0.1)
    tx, tw = mb.Tensor.from_bits(gpu, dt, xb), mb.Tensor.from_bits(gpu, dt, wb)
    vx, vw = cases.apply_ops(tx, xops), cases.apply_ops(tw, wops)
    r = vx @ vw.T
    assert mb.last_kernel().startswith("tcgen05"), mb.last_kernel()
    xf = cases.apply_ops(cases.NpView(O.bits_to_f64(dt, xb)), xops).a
    wf = cases.apply_ops(cases.NpView(O.bits_to_f64(dt, wb)), wops).a
    truth = xf @ wf.T
    m = O.error_metrics(dt, r.to_bits(), truth, np.abs(xf) @ np.abs(wf).T)
    assert m["e"] <= unit_roundoff(dt) + xf.shape[-1] * 2.0 ** -24, m
    for t in (r, tx, tw):
        t.release()


def test_fresh_result_as_weight_operand_in_a_decode_chain(gpu):
    """k = x @ Wk.T followed at once by s = q @ k.T on the same stream, many times with changing x and no
    synchronisation in between. The decode kernels let their successors start early and fetch weights ahead of their
    wait -- but k is a result that may still be in flight, so it must be read after the wait: every s must be the
    product with the k of ITS round."""
    dt = O.BFLOAT16
    L = mb.lib()
    rng = np.random.default_rng(9)
    T, H, D = 8, 1024, 1024
    wk = bits(dt, rng, (D, H), 0.05)
    tw = mb.Tensor.from_bits(gpu, dt, wk)
    rounds = 24
    xs = [bits(dt, rng, (T, H), 1.0) for _ in range(rounds)]
    qb = bits(dt, rng, (4, D), 1.0)
    tq = mb.Tensor.from_bits(gpu, dt, qb)
    txs = [mb.Tensor.from_bits(gpu, dt, x) for x in xs]
    tk = mb.Tensor(gpu, dt, (T, D))
    outs = [mb.Tensor(gpu, dt, (4, T)) for _ in range(rounds)]
    mb.synchronize(gpu)
    for r in range(rounds):
        mb.check(L.magb200_matmul(gpu, C.byref(txs[r].view_struct()), C.byref(tw.T.view_struct()), C.byref(tk.view_struct())))
        assert mb.last_kernel().startswith("skinny")
        mb.check(L.magb200_matmul(gpu, C.byref(tq.view_struct()), C.byref(tk.T.view_struct()), C.byref(outs[r].view_struct())))
        assert mb.last_kernel().startswith("skinny")
    mb.synchronize(gpu)
    wf, qf = O.bits_to_f64(dt, wk), O.bits_to_f64(dt, qb)
    for r in range(rounds):
        kf = O.bits_to_f64(dt, O.f32_to_bits(dt, (O.bits_to_f64(dt, xs[r]) @ wf.T).astype(np.float32)))
        truth = qf @ kf.T
        got = O.bits_to_f64(dt, outs[r].to_bits())
        # k itself is rounded to bf16 once more on the device than in this restatement only where the fp32 sums differ in
        # the last bit: allow two output roundings
        assert np.max(np.abs(got - truth)) <= 4 * 2.0 ** -8 * np.max(np.abs(truth)), r
    for t in txs + outs + [tw, tq, tk]:
        t.release()


@pytest.mark.parametrize("kernel,M,N", [("tcgen05", 128, 128), ("tcgen05_2sm", 256, 256)])
def test_a_wait_that_runs_out_is_reported_and_the_device_stays_usable(gpu, kernel, M, N):
    """One-tile launch whose producer leaves one stage unarmed (test hook): the MMA thread's bounded wait runs out after
    the (shortened) limit, the kernel drains and returns, synchronize reports MAGB200_ERR_TIMEOUT, and the next ordinary
    matmul on the same device is correct. Nothing traps, faults or spins without a limit."""
    dt = O.BFLOAT16
    L = mb.lib()
    rng = np.random.default_rng(5)
    K = 512
    xb, wb = bits(dt, rng, (M, K), 1.0), bits(dt, rng, (N, K), 0.1)
    tx, tw = mb.Tensor.from_bits(gpu, dt, xb), mb.Tensor.from_bits(gpu, dt, wb)
    out = mb.Tensor(gpu, dt, (M, N))
    old = L.magb200_get_wait_limit_ns()
    mb.check(L.magb200_set_wait_limit_ns(5_000_000))           # 5 ms
    mb.force_kernel(kernel)
    try:
        mb.check(L.magb200_test_leave_stage_unarmed(2))
        mb.check(L.magb200_matmul(gpu, C.byref(tx.view_struct()), C.byref(tw.T.view_struct()), C.byref(out.view_struct())))
        rc = L.magb200_synchronize(gpu)
        assert rc == mb.ERR_TIMEOUT, (rc, L.magb200_last_error())
        assert b"wait ran out" in L.magb200_last_error()
        # the hook was consumed by that launch; the same call now runs normally
        mb.check(L.magb200_matmul(gpu, C.byref(tx.view_struct()), C.byref(tw.T.view_struct()), C.byref(out.view_struct())))
        mb.synchronize(gpu)
    finally:
        mb.force_kernel(None)
        mb.check(L.magb200_set_wait_limit_ns(old))
    xf, wf = O.bits_to_f64(dt, xb), O.bits_to_f64(dt, wb)
    m = O.error_metrics(dt, out.to_bits(), xf @ wf.T, np.abs(xf) @ np.abs(wf).T)
    assert m["e"] <= unit_roundoff(dt) + K * 2.0 ** -24, m
    for t in (tx, tw, out):
        t.release()


def test_pool_reuses_freed_blocks_without_cuda_calls(gpu):
    L = mb.lib()

    def stats():
        v = [C.c_uint64() for _ in range(4)]
        mb.check(L.magb200_pool_stats(gpu, *[C.byref(x) for x in v]))
        return [x.value for x in v]          # live, cached, hits, misses

    a = mb.Tensor(gpu, O.BFLOAT16, (1000, 1000))
    ptr = a.ptr
    live0, _, hits0, misses0 = stats()
    a.release()
    live1, cached1, _, _ = stats()
    assert live1 < live0 and cached1 >= 2_000_000
    b = mb.Tensor(gpu, O.BFLOAT16, (999, 1001))      # same size class
    _, _, hits2, misses2 = stats()
    assert b.ptr == ptr and hits2 == hits0 + 1 and misses2 == misses0
    b.release()
    # results stay right when a block changes hands while its last reader is still queued
    dt = O.BFLOAT16
    rng = np.random.default_rng(2)
    xb, wb = bits(dt, rng, (512, 512), 1.0), bits(dt, rng, (512, 512), 0.1)
    tx, tw = mb.Tensor.from_bits(gpu, dt, xb), mb.Tensor.from_bits(gpu, dt, wb)
    want = (tx @ tw.T).to_bits()
    for _ in range(8):
        r = tx @ tw.T          # block comes from the pool ...
        r2 = r @ tw.T          # ... is read by a second matmul ...
        r.release()            # ... and goes back while that may still run
        junk = mb.Tensor(gpu, dt, (512, 512))
        mb.check(L.magb200_fill(gpu, C.byref(junk.view_struct()), 7.0))
        got2 = r2.to_bits()
        first = (tx @ tw.T)
        assert np.array_equal(first.to_bits(), want)
        ref2 = (first @ tw.T).to_bits()
        assert np.array_equal(got2, ref2)
        for t in (r2, junk, first):
            t.release()
    mb.check(L.magb200_pool_trim(gpu))
    assert stats()[1] == 0
    for t in (tx, tw):
        t.release()


def test_non_finite_operands_float32(gpu):
    """float32 goes through the compensated FFMA kernel, whose error-free summation must not turn an infinite sum into NaN."""
    dt = O.FLOAT32
    rng = np.random.default_rng(14)
    for (M, N, K) in ((96, 80, 200), (64, 64, 4096)):     # the second shape splits K over CTAs
        xb, wb = bits(dt, rng, (M, K), 1.0), bits(dt, rng, (N, K), 0.1)
        xb[1, 7] = 0x7FC00000
        xb[2, 9] = 0x7F800000
        wb[5, K - 3] = 0xFF800000
        tx, tw = mb.Tensor.from_bits(gpu, dt, xb), mb.Tensor.from_bits(gpu, dt, wb)
        r = tx @ tw.T
        assert mb.last_kernel() == "simt"
        f = O.bits_to_f64(dt, r.to_bits())
        with np.errstate(all="ignore"):
            truth = O.bits_to_f64(dt, xb) @ O.bits_to_f64(dt, wb).T
        assert np.array_equal(np.isnan(f), np.isnan(truth))
        assert np.array_equal(np.isposinf(f), np.isposinf(truth)) and np.array_equal(np.isneginf(f), np.isneginf(truth))
        fin = np.isfinite(truth)
        assert np.max(np.abs(f[fin] - truth[fin])) <= 1e-5 * np.max(np.abs(truth[fin]))
        for t in (r, tx, tw):
            t.release()


def test_float32_operands_that_cannot_be_split(gpu):
    """The float32 tensor-core path writes every element as three bf16 values, which cannot hold an infinity, a NaN, a value
    that rounds to a bf16 infinity or one so small that its lower parts leave the normal range. The split pass flags such an
    operand, the tensor-core launch then does nothing and the FFMA kernel that stands by behind it computes the product:
    the result is bit for bit what the FFMA kernel gives when it is asked for directly. A clean product afterwards takes
    the tensor-core kernel again (the flag is per call)."""
    dt = O.FLOAT32
    rng = np.random.default_rng(15)
    M, N, K = 256, 384, 512
    clean_x, clean_w = bits(dt, rng, (M, K), 1.0), bits(dt, rng, (N, K), 0.1)
    patterns = {"inf": 0x7F800000, "nan": 0x7FC00000, "rounds_to_bf16_inf": 0x7F7FFFFF, "tiny": 0x0A000000, "subnormal": 0x00000001}
    for label, pat in patterns.items():
        for where in ("x", "w"):
            xb, wb = clean_x.copy(), clean_w.copy()
            (xb if where == "x" else wb)[3, K - 5] = pat
            tx, tw = mb.Tensor.from_bits(gpu, dt, xb), mb.Tensor.from_bits(gpu, dt, wb)
            results = {}
            for kernel in ("tcgen05_f32x3", "simt"):
                mb.force_kernel(kernel)
                try:
                    r = tx @ tw.T
                    assert mb.last_kernel() == kernel
                    results[kernel] = r.to_bits()
                    r.release()
                finally:
                    mb.force_kernel(None)
            assert np.array_equal(results["tcgen05_f32x3"], results["simt"]), (label, where)
            for t in (tx, tw):
                t.release()
    # clean operands: the two kernels differ in the last place somewhere, which shows that the tensor-core kernel ran
    tx, tw = mb.Tensor.from_bits(gpu, dt, clean_x), mb.Tensor.from_bits(gpu, dt, clean_w)
    out = {}
    for kernel in ("tcgen05_f32x3", "simt"):
        mb.force_kernel(kernel)
        try:
            r = tx @ tw.T
            out[kernel] = O.bits_to_f64(dt, r.to_bits())
            r.release()
        finally:
            mb.force_kernel(None)
    truth = O.bits_to_f64(dt, clean_x) @ O.bits_to_f64(dt, clean_w).T
    scale = np.abs(O.bits_to_f64(dt, clean_x)) @ np.abs(O.bits_to_f64(dt, clean_w)).T
    for kernel in out:
        assert (np.abs(out[kernel] - truth) / scale).max() <= 2.0 ** -24 * 1.5, kernel
    assert not np.array_equal(out["tcgen05_f32x3"], out["simt"])
    for t in (tx, tw):
        t.release()


def test_float32_split_operand_kernel_in_a_graph(gpu):
    """The planes live in the device workspace, so the float32 tensor-core path can be recorded into a CUDA graph once the
    workspace has its size (one plain call first); replays give the same bits as the plain call."""
    dt = O.FLOAT32
    rng = np.random.default_rng(16)
    M, N, K = 384, 512, 1024
    xb, wb = bits(dt, rng, (M, K), 1.0), bits(dt, rng, (N, K), 0.1)
    tx, tw, out = mb.Tensor.from_bits(gpu, dt, xb), mb.Tensor.from_bits(gpu, dt, wb), mb.Tensor(gpu, dt, (M, N))
    L = mb.lib()
    xv, wv, ov = tx.view_struct(), tw.T.view_struct(), out.view_struct()
    mb.force_kernel("tcgen05_f32x3")
    try:
        mb.check(L.magb200_matmul(gpu, C.byref(xv), C.byref(wv), C.byref(ov)))
        plain = out.to_bits()
        mb.check(L.magb200_fill(gpu, C.byref(ov), C.c_double(0.0)))
        graph = C.c_void_p()
        mb.check(L.magb200_graph_begin_capture(gpu))
        mb.check(L.magb200_matmul(gpu, C.byref(xv), C.byref(wv), C.byref(ov)))
        assert mb.last_kernel() == "tcgen05_f32x3"
        mb.check(L.magb200_graph_end_capture(gpu, C.byref(graph)))
        for _ in range(3):
            mb.check(L.magb200_graph_launch(gpu, graph))
        mb.synchronize(gpu)
        assert np.array_equal(out.to_bits(), plain)
        mb.check(L.magb200_graph_destroy(graph))
    finally:
        mb.force_kernel(None)
    for t in (tx, tw, out):
        t.release()


@pytest.mark.parametrize("kernel", ["tcgen05", "tcgen05_2sm", "skinny", "simt"])
def test_non_finite_operands(gpu, kernel):
    """NaN and infinities in the operands: rows / columns that meet them are NaN or infinite in the result, every other
    element is unaffected. Recorded here: the tensor-core and decode kernels round with the hardware converters and
    produce 0x7FFF for a NaN result, the FFMA kernel the canonical 0x7FC0; the reference's own NaN pattern depends on
    the CPU specialisation, so only NaN-ness is asserted."""
    dt = O.BFLOAT16
    M, N, K = (4, 512, 512) if kernel == "skinny" else (256, 256, 256)
    rng = np.random.default_rng(13)
    xb, wb = bits(dt, rng, (M, K), 1.0), bits(dt, rng, (N, K), 0.1)
    xb[1, 7] = 0x7FC0            # NaN in activation row 1
    xb[2, 9] = 0x7F80            # +inf in activation row 2
    wb[5, 11] = 0xFF80           # -inf in weight row 5 (output column 5)
    tx, tw = mb.Tensor.from_bits(gpu, dt, xb), mb.Tensor.from_bits(gpu, dt, wb)
    mb.force_kernel(kernel)
    try:
        r = tx @ tw.T
        assert mb.last_kernel().startswith(kernel)
    finally:
        mb.force_kernel(None)
    got = r.to_bits()
    f = O.bits_to_f64(dt, got)
    with np.errstate(all="ignore"):
        truth = O.bits_to_f64(dt, xb) @ O.bits_to_f64(dt, wb).T
    assert np.array_equal(np.isnan(f), np.isnan(truth))
    assert np.array_equal(np.isposinf(f), np.isposinf(truth)) and np.array_equal(np.isneginf(f), np.isneginf(truth))
    fin = np.isfinite(truth)
    assert np.max(np.abs(f[fin] - truth[fin])) <= 2.0 ** -7 * np.max(np.abs(truth[fin]))
    nan_patterns = set(np.unique(got[np.isnan(f)]).tolist())
    assert nan_patterns <= {0x7FFF, 0x7FC0, 0xFFC0, 0xFFFF}, [hex(p) for p in nan_patterns]
    for t in (r, tx, tw):
        t.release()


def test_every_visible_device_runs_the_big_shared_memory_kernels(gpu):
    """The opt-in to more than 48 KB of dynamic shared memory is per device: one tensor-core and one decode matmul on
    every visible device of this process."""
    dt = O.BFLOAT16
    L = mb.lib()
    rng = np.random.default_rng(3)
    xb, wb = bits(dt, rng, (256, 512), 1.0), bits(dt, rng, (512, 512), 0.1)
    xf, wf = O.bits_to_f64(dt, xb), O.bits_to_f64(dt, wb)
    for dev in range(mb.device_count()):
        mb.check(L.magb200_device_init(dev))
        tx, tw = mb.Tensor.from_bits(dev, dt, xb), mb.Tensor.from_bits(dev, dt, wb)
        for kernel, rows in (("tcgen05_2sm", 256), ("tcgen05", 256), ("skinny", 8)):
            mb.force_kernel(kernel)
            try:
                r = tx.slice(0, 0, rows) @ tw.T
            finally:
                mb.force_kernel(None)
            m = O.error_metrics(dt, r.to_bits(), xf[:rows] @ wf.T, np.abs(xf[:rows]) @ np.abs(wf).T)
            assert m["e"] <= unit_roundoff(dt) + 512 * 2.0 ** -24, (dev, kernel, m)
            r.release()
        tx.release(); tw.release()
