"""GPU parity tests of MAG_OP_MATMUL through the C ABI.

Every case is checked three ways: (1) the accuracy gate against the reference CPU backend's golden
result (error vs fp64 not above 2x the reference's), (2) this library's own bar -- one rounding of an
fp32-accumulated sum, |err| <= (u + K 2^-24) sum_k|a||b| -- and (3) elementwise closeness to the
reference result in the reference tests' tolerances wherever the reference itself is right."""
import ctypes as C

import numpy as np
import pytest

import magnetron_b200 as mb
from oracle import mag_oracle as O
from oracle import ref_driver as R
from tests import cases
from tests.common import case_operands, case_truth, gate, golden, reference_defect_mask, unit_roundoff

pytestmark = pytest.mark.gpu
CASE_NAMES = [c[0] for c in cases.MATMUL_CASES]


def run_case(dev, name, dt, kernel=None):
    xb, yb = case_operands(name, dt)
    _, _, xops, _, yops = cases.case_by_name(name)
    tx, ty = mb.Tensor.from_bits(dev, dt, xb), mb.Tensor.from_bits(dev, dt, yb)
    vx, vy = cases.apply_ops(tx, xops), cases.apply_ops(ty, yops)
    mb.force_kernel(kernel)
    try:
        r = vx @ vy
        used = mb.last_kernel()
        mb.synchronize(dev)
    finally:
        mb.force_kernel(None)
    got = r.to_bits()
    for t in (r, tx, ty):
        t.release()
    return xb, yb, got, used, vx.shape[-1]


def check_case(name, dname, dt, xb, yb, got, K):
    truth, scale = case_truth(name, dt, xb, yb)
    ref = golden("matmul_golden.npz")[f"{name}.{dname}.r"]
    assert got.shape == truth.shape == tuple(golden("matmul_golden.npz")[f"{name}.{dname}.rshape"])
    mg, _ = gate(dt, got, ref, truth, scale, K)
    assert mg["e"] <= unit_roundoff(dt) + K * 2.0 ** -24, mg        # single rounding of an fp32 sum
    ok = ~reference_defect_mask(name, dt, truth.shape)
    a, r = O.bits_to_f64(dt, got), O.bits_to_f64(dt, ref)
    atol, rtol = ((1e-5, 1e-5) if dt == O.FLOAT32 else (1e-2, 1e-2))
    assert np.all((np.abs(a - r) <= atol * max(1.0, np.abs(truth).max()) + rtol * np.abs(r))[ok])


@pytest.mark.parametrize("name", CASE_NAMES)
@pytest.mark.parametrize("dname", list(cases.DTYPES))
def test_case_auto_route(gpu, name, dname):
    dt = cases.DTYPES[dname]
    xb, yb, got, used, K = run_case(gpu, name, dt)
    assert used in ("tcgen05", "skinny", "skinny_splitk", "simt")
    check_case(name, dname, dt, xb, yb, got, K)


@pytest.mark.parametrize("name", CASE_NAMES)
@pytest.mark.parametrize("dname", list(cases.DTYPES))
def test_case_simt_kernel(gpu, name, dname):
    dt = cases.DTYPES[dname]
    xb, yb, got, used, K = run_case(gpu, name, dt, "simt")
    assert used == "simt"
    check_case(name, dname, dt, xb, yb, got, K)


@pytest.mark.parametrize("name", CASE_NAMES)
def test_case_float32_split_operand_kernel(gpu, name):
    """Every float32 case through the tensor-core kernel that splits the operands into three bf16 planes: same gate, same
    own bar and same closeness to the reference as the FFMA kernel (strided, transposed, batched and broadcast operands go
    through the split pass, ragged shapes through the tile tails)."""
    dt = O.FLOAT32
    xb, yb, got, used, K = run_case(gpu, name, dt, "tcgen05_f32x3")
    assert used == "tcgen05_f32x3"
    check_case(name, "f32", dt, xb, yb, got, K)


TC_CASES = ["sq64", "rect_big", "linear_wT", "linear_wT_tail", "x_T_al", "both_T_al", "batch_y_T", "gqa_scores", "gqa_pv",
            "slice_k", "slice_n", "big_k", "tile_edge", "batch_same", "batch_bcast_y", "batch_mixed", "permute_x"]


@pytest.mark.parametrize("name", TC_CASES)
@pytest.mark.parametrize("dname", ["bf16", "f16"])
def test_case_tcgen05_kernel(gpu, name, dname):
    """Small and ragged shapes forced through the tensor-core kernel: tails in M, N and K, both operand
    major-nesses, batch and broadcast coordinates."""
    dt = cases.DTYPES[dname]
    xb, yb, got, used, K = run_case(gpu, name, dt, "tcgen05")
    assert used == "tcgen05"
    check_case(name, dname, dt, xb, yb, got, K)


SKINNY_CASES = ["gemv_wT", "gemv_kn", "skinny4_wT", "skinny8_kn", "big_k"]


@pytest.mark.parametrize("name", SKINNY_CASES)
@pytest.mark.parametrize("dname", list(cases.DTYPES))
def test_case_skinny_kernel(gpu, name, dname):
    dt = cases.DTYPES[dname]
    xb, yb, got, used, K = run_case(gpu, name, dt, "skinny")
    assert used in ("skinny", "skinny_splitk")
    check_case(name, dname, dt, xb, yb, got, K)


def bits(dt, rng, shape, scale):
    return O.f32_to_bits(dt, cases.gen_storage(rng, shape, scale))


def sampled_check(dt, xb, wb_nk, got, rows, K):
    """fp64 truth on a sample of output rows of x @ W.T (full-size shapes)."""
    x = O.bits_to_f64(dt, xb[rows]); w = O.bits_to_f64(dt, wb_nk)
    truth = x @ w.T
    scale = np.abs(x) @ np.abs(w).T
    m = O.error_metrics(dt, got[rows], truth, scale)
    assert m["e"] <= unit_roundoff(dt) + K * 2.0 ** -24, m
    return m


@pytest.mark.parametrize("dname", ["bf16", "f32"])
def test_single_op_workload_512x2048x2048(gpu, dname):
    """C[512,2048] = A[512,2048] @ W[2048,2048]^T with W a transposed strided view, seed 0; checked
    against fp64 and, when the reference library is on this machine, against its error in the same run."""
    dt = cases.DTYPES[dname]
    rng = np.random.default_rng(0)
    xb, wb = bits(dt, rng, (512, 2048), 1.0), bits(dt, rng, (2048, 2048), 0.02)
    tx, tw = mb.Tensor.from_bits(gpu, dt, xb), mb.Tensor.from_bits(gpu, dt, wb)
    r = tx @ tw.T
    assert mb.last_kernel() == ("tcgen05" if dt == O.BFLOAT16 else "tcgen05_f32x3")   # 16 tiles of 256x256: the one-CTA kernel
    got = r.to_bits()
    truth = O.bits_to_f64(dt, xb) @ O.bits_to_f64(dt, wb).T
    scale = np.abs(O.bits_to_f64(dt, xb)) @ np.abs(O.bits_to_f64(dt, wb)).T
    mg = O.error_metrics(dt, got, truth, scale)
    assert mg["e"] <= unit_roundoff(dt) + 2048 * 2.0 ** -24, mg
    if R.available():
        api = R.MagApi("cpu", log_level=1)
        try:
            ra, rw = api.from_bits(dt, xb), api.from_bits(dt, wb)
            rwt = api.transpose(rw, 0, 1)
            rr = api.matmul(ra, rwt)
            mr = O.error_metrics(dt, api.to_bits(rr), truth, scale)
            for h in (rr, rwt, ra, rw):
                h.release()
        finally:
            api.close(True)
        assert mg["e"] <= 2.0 * mr["e"], (mg, mr)


@pytest.mark.parametrize("M,N,K", [(4096, 4096, 4096), (4096, 1024, 4096), (1000, 12288, 4096), (4096, 4096, 12288)])
def test_prefill_shapes_sampled(gpu, M, N, K):
    """Qwen3-8B-shaped prefill GEMMs (seed 3) at full size; fp64 truth on 48 sampled rows, plus the
    size-independent checks: identical result when rerun, and zero rows of A give zero rows of C."""
    dt = O.BFLOAT16
    rng = np.random.default_rng(3)
    xb, wb = bits(dt, rng, (M, K), 1.0), bits(dt, rng, (N, K), 0.02)
    xb[5] = 0; xb[M - 1] = 0
    tx, tw = mb.Tensor.from_bits(gpu, dt, xb), mb.Tensor.from_bits(gpu, dt, wb)
    r = tx @ tw.T
    assert mb.last_kernel() == ("tcgen05_2sm" if (M // 256) * (N // 256) >= 74 else "tcgen05")
    got = r.to_bits()
    rows = np.unique(np.concatenate([[0, 5, 127, 128, M - 1], rng.integers(0, M, 43)]))
    sampled_check(dt, xb, wb, got, rows, K)
    assert not got[5].any() and not got[M - 1].any()
    again = (tx @ tw.T).to_bits()
    assert np.array_equal(got, again)


@pytest.mark.parametrize("M", [1, 2, 4, 8])
@pytest.mark.parametrize("N,K", [(2048, 1024), (1024, 1024), (3072, 1024), (1024, 3072), (151936, 1024), (5120, 25600)])
def test_decode_shapes(gpu, M, N, K):
    """Qwen3-0.6B decode projections and lm_head (and the long-K down projection of the 32B model),
    batch sweep M in {1,2,4,8}, weights through the `W.T` view; fp64 truth on sampled output columns."""
    dt = O.BFLOAT16
    rng = np.random.default_rng(2)
    xb, wb = bits(dt, rng, (M, K), 1.0), bits(dt, rng, (N, K), 0.02)
    tx, tw = mb.Tensor.from_bits(gpu, dt, xb), mb.Tensor.from_bits(gpu, dt, wb)
    r = tx @ tw.T
    assert mb.last_kernel() in ("skinny", "skinny_splitk")
    got = r.to_bits()
    cols = np.unique(np.concatenate([[0, 1, N - 1], rng.integers(0, N, 500)]))
    x = O.bits_to_f64(dt, xb); w = O.bits_to_f64(dt, wb[cols])
    truth = x @ w.T
    m = O.error_metrics(dt, got[:, cols], truth, np.abs(x) @ np.abs(w).T)
    assert m["e"] <= unit_roundoff(dt) + K * 2.0 ** -24, m


@pytest.mark.parametrize("dname", ["bf16", "f16"])
def test_attention_broadcast_shapes(gpu, dname):
    """Scores Q @ K^T and outputs P @ V with K/V broadcast over 4 query heads per KV head through views
    (reduced batch and sequence so the fp64 truth stays cheap)."""
    dt = cases.DTYPES[dname]
    B, KV, G, T, D = 2, 2, 4, 256, 128
    rng = np.random.default_rng(4)
    q, k, v = bits(dt, rng, (B, KV, G, T, D), 1.0), bits(dt, rng, (B, KV, T, D), 1.0), bits(dt, rng, (B, KV, T, D), 1.0)
    tq, tk, tv = (mb.Tensor.from_bits(gpu, dt, a) for a in (q, k, v))
    kt = tk.transpose(2, 3).view((B, KV, 1, D, T))
    s = tq @ kt
    assert mb.last_kernel().startswith("tcgen05") and s.shape == (B, KV, G, T, T)
    qf, kf, vf = (O.bits_to_f64(dt, a) for a in (q, k, v))
    truth = np.einsum("bhgtd,bhsd->bhgts", qf, kf)
    scale = np.einsum("bhgtd,bhsd->bhgts", np.abs(qf), np.abs(kf))
    m = O.error_metrics(dt, s.to_bits(), truth, scale)
    assert m["e"] <= unit_roundoff(dt) + D * 2.0 ** -24, m
    # P = softmax(scaled logits) rounded to the storage dtype, then P @ V
    logits = truth / np.sqrt(D)
    p = np.exp(logits - logits.max(-1, keepdims=True)); p /= p.sum(-1, keepdims=True)
    pb = O.f32_to_bits(dt, p.astype(np.float32))
    tp = mb.Tensor.from_bits(gpu, dt, pb)
    o = tp @ tv.view((B, KV, 1, T, D))
    assert mb.last_kernel().startswith("tcgen05") and o.shape == (B, KV, G, T, D)
    pf = O.bits_to_f64(dt, pb)
    truth2 = np.einsum("bhgts,bhsd->bhgtd", pf, vf)
    m2 = O.error_metrics(dt, o.to_bits(), truth2, np.einsum("bhgts,bhsd->bhgtd", np.abs(pf), np.abs(vf)))
    assert m2["e"] <= unit_roundoff(dt) + T * 2.0 ** -24, m2


TWO_SM_SHAPES = [
    # (x storage shape, x transposed?, y storage shape, y is W.T?)  -- M, N >= 256 with tails in M, N and K
    ((512, 256), False, (512, 256), True),
    ((300, 200), False, (260, 200), True),          # ragged M, N, K
    ((1024, 4096), False, (768, 4096), True),       # several tiles per pair, long K
    ((384, 320), False, (320, 520), False),         # contiguous [K,N] weight (N-major B)
    ((192, 640), True, (512, 192), True),           # transposed activation (M-major A)
    ((3, 256, 128), False, (3, 128, 512), False),   # batched
    ((2, 257, 72), False, (384, 72), True),         # batch folds into M = 514
]


@pytest.mark.parametrize("xs,xT,ys,wT", TWO_SM_SHAPES)
@pytest.mark.parametrize("dname", ["bf16", "f16"])
def test_two_sm_kernel(gpu, xs, xT, ys, wT, dname):
    """The CTA-pair kernel (tcgen05.mma.cta_group::2) forced on shapes with tails, both major-nesses and batches;
    full fp64 truth."""
    dt = cases.DTYPES[dname]
    rng = np.random.default_rng(17)
    xb, yb = bits(dt, rng, xs, 1.0), bits(dt, rng, ys, 0.1)
    tx, ty = mb.Tensor.from_bits(gpu, dt, xb), mb.Tensor.from_bits(gpu, dt, yb)
    vx = tx.transpose(len(xs) - 2, len(xs) - 1) if xT else tx
    vy = ty.transpose(len(ys) - 2, len(ys) - 1) if wT else ty
    mb.force_kernel("tcgen05_2sm")
    try:
        r = vx @ vy
        assert mb.last_kernel() == "tcgen05_2sm"
        mb.synchronize(gpu)
    finally:
        mb.force_kernel(None)
    xf, yf = O.bits_to_f64(dt, xb), O.bits_to_f64(dt, yb)
    xf = np.swapaxes(xf, -1, -2) if xT else xf
    yf = np.swapaxes(yf, -1, -2) if wT else yf
    truth = np.matmul(xf, yf)
    m = O.error_metrics(dt, r.to_bits(), truth, np.matmul(np.abs(xf), np.abs(yf)))
    assert m["e"] <= unit_roundoff(dt) + xf.shape[-1] * 2.0 ** -24, m
    for t in (r, tx, ty):
        t.release()


@pytest.mark.parametrize("ranks,M,N,K", [(2, 512, 512, 512), (4, 1024, 384, 2048), (8, 2048, 5120, 1024)])
def test_fused_row_sharded_linear_emulated_ranks(gpu, ranks, M, N, K):
    """The fused row-sharded linear (scatter epilogue + reduce-broadcast) with all ranks emulated on one GPU: rank r
    multiplies its K slice and pushes row block o of the partial product into rank o's staging slot r; every owner then sums
    its slots and writes its rows into every rank's output. All outputs must be identical and match the unsharded product."""
    dt = O.BFLOAT16
    L = mb.lib()
    rng = np.random.default_rng(23)
    xb, wb = bits(dt, rng, (M, K), 1.0), bits(dt, rng, (N, K), 0.05)
    tx, tw = mb.Tensor.from_bits(gpu, dt, xb), mb.Tensor.from_bits(gpu, dt, wb)
    R_ = M // ranks
    stages = [mb.Tensor(gpu, dt, (ranks, R_, N)) for _ in range(ranks)]
    outs = [mb.Tensor(gpu, dt, (M, N)) for _ in range(ranks)]
    stage_ptrs = (C.c_void_p * ranks)(*[t.ptr for t in stages])
    out_ptrs = (C.c_void_p * ranks)(*[t.ptr for t in outs])
    kp = K // ranks
    for r in range(ranks):
        xr = tx.slice(1, r * kp, kp)                 # this rank's K slice of the activations: a strided view
        wr = tw.slice(1, r * kp, kp).T               # and of the weight, seen as W.T
        mb.check(L.magb200_matmul_scatter(gpu, C.byref(xr.view_struct()), C.byref(wr.view_struct()), stage_ptrs, ranks, r))
        assert mb.last_kernel().startswith("tcgen05")
    for o in range(ranks):
        mb.check(L.magb200_reduce_broadcast(gpu, None, stages[o].ptr, out_ptrs, ranks, o, R_, N, dt))
    mb.synchronize(gpu)
    got = [t.to_bits() for t in outs]
    for g in got[1:]:
        assert np.array_equal(g, got[0])
    xf, wf = O.bits_to_f64(dt, xb), O.bits_to_f64(dt, wb)
    m = O.error_metrics(dt, got[0], xf @ wf.T, np.abs(xf) @ np.abs(wf).T)
    assert m["e"] <= (ranks + 1) * unit_roundoff(dt) + K * 2.0 ** -24, m      # one rounding per partial + one for the sum
    for t in stages + outs + [tx, tw]:
        t.release()


@pytest.mark.parametrize("dname", ["bf16", "f16"])
def test_attention_scores_full_size(gpu, dname):
    """Q[8x32x2048x128] @ K^T with K [8x8x2048x128] broadcast over 4 query heads per KV head (seed 4), at full size:
    549 GFLOP, a 2.1 GB result. fp64 truth on sampled (batch, head, row) triples; the 4 query heads of a group really
    read the same K (row of head g against K of its KV head)."""
    dt = cases.DTYPES[dname]
    B, KV, G, T, D = 8, 8, 4, 2048, 128
    rng = np.random.default_rng(4)
    q = bits(dt, rng, (B, KV, G, T, D), 1.0)
    k = bits(dt, rng, (B, KV, T, D), 1.0)
    tq, tk = mb.Tensor.from_bits(gpu, dt, q), mb.Tensor.from_bits(gpu, dt, k)
    s = tq @ tk.transpose(2, 3).view((B, KV, 1, D, T))
    assert s.shape == (B, KV, G, T, T) and mb.last_kernel().startswith("tcgen05")
    mb.synchronize(gpu)
    for _ in range(24):
        b, h, g, t = (int(rng.integers(0, n)) for n in (B, KV, G, T))
        row = mb.Tensor(gpu, dt, (T,), base_ptr=s.ptr, offset=(((b * KV + h) * G + g) * T + t) * T, storage_elems=s.numel).to_bits()
        qf, kf = O.bits_to_f64(dt, q[b, h, g, t]), O.bits_to_f64(dt, k[b, h])
        truth = kf @ qf
        m = O.error_metrics(dt, row, truth, np.abs(kf) @ np.abs(qf))
        assert m["e"] <= unit_roundoff(dt) + D * 2.0 ** -24, (b, h, g, t, m)
    for t_ in (s, tq, tk):
        t_.release()


@pytest.mark.parametrize("dname", ["bf16", "f16"])
def test_attention_pv_full_size(gpu, dname):
    """P[8x32x2048x2048] @ V with V [8x8x2048x128] broadcast over 4 query heads per KV head, at full size: P is 2.1 GB of
    softmax rows (scaled N(0,1) logits, seed 4). The logits of one batch entry are drawn and soft-maxed on the host; batch
    entry b holds the same rows rolled by 37 b keys, so every entry is different and still a softmax. fp64 truth on sampled
    (batch, head, row) triples."""
    dt = cases.DTYPES[dname]
    B, KV, G, T, D = 8, 8, 4, 2048, 128
    rng = np.random.default_rng(4)
    v = bits(dt, rng, (B, KV, T, D), 1.0)
    tv = mb.Tensor.from_bits(gpu, dt, v)
    logits = rng.standard_normal((KV, G, T, T), dtype=np.float32) / np.float32(np.sqrt(D))
    logits -= logits.max(-1, keepdims=True)
    np.exp(logits, out=logits)
    logits /= logits.sum(-1, keepdims=True)
    p0 = O.f32_to_bits(dt, logits)
    del logits
    tp = mb.Tensor(gpu, dt, (B, KV, G, T, T))
    per = KV * G * T * T
    for b in range(B):
        chunk = np.ascontiguousarray(np.roll(p0, 37 * b, axis=-1))
        mb.check(mb.lib().magb200_upload(gpu, tp.ptr + b * per * 2, chunk.ctypes.data, chunk.nbytes))
    o = tp @ tv.view((B, KV, 1, T, D))
    assert o.shape == (B, KV, G, T, D) and mb.last_kernel().startswith("tcgen05")
    got = o.to_bits()
    for _ in range(32):
        b, h, g, t = (int(rng.integers(0, n)) for n in (B, KV, G, T))
        pf = O.bits_to_f64(dt, np.roll(p0[h, g, t], 37 * b))
        vf = O.bits_to_f64(dt, v[b, h])
        m = O.error_metrics(dt, got[b, h, g, t], pf @ vf, np.abs(pf) @ np.abs(vf))
        assert m["e"] <= unit_roundoff(dt) + T * 2.0 ** -24, (b, h, g, t, m)
    for t_ in (o, tp, tv):
        t_.release()


# per-rank problems of the Qwen3-32B layer sharded 8 ways: (M, N_local, K_local, K_full); K_full > K_local means the operands
# are the rank's K slice of a wider activation and weight (row sharding: strided views)
TP_RANK_SHAPES = [(8192, 1280, 5120, 5120), (8192, 5120, 1024, 2048), (8192, 6400, 5120, 5120), (8192, 5120, 3200, 6400),
                  (512, 1280, 5120, 5120), (512, 5120, 1024, 2048), (512, 6400, 5120, 5120), (512, 5120, 3200, 6400)]


@pytest.mark.parametrize("M,N,K,KF", TP_RANK_SHAPES)
def test_tensor_parallel_per_rank_shapes(gpu, M, N, K, KF):
    """What one of eight ranks multiplies for qkv / o / gate+up / down at 8192 and 512 tokens (seed 5): column shards are
    plain x @ W_shard.T, row shards take the second K slice of x and of W as strided views. fp64 truth on sampled rows."""
    dt = O.BFLOAT16
    rng = np.random.default_rng(5)
    xb, wb = bits(dt, rng, (M, KF), 1.0), bits(dt, rng, (N, KF), 0.02)
    tx, tw = mb.Tensor.from_bits(gpu, dt, xb), mb.Tensor.from_bits(gpu, dt, wb)
    k0 = KF - K
    r = tx.slice(1, k0, K) @ tw.slice(1, k0, K).T
    assert mb.last_kernel().startswith("tcgen05")
    got = r.to_bits()
    rows = np.unique(np.concatenate([[0, 255, 256, M - 1], rng.integers(0, M, 28)]))
    sampled_check(dt, xb[:, k0:], wb[:, k0:], got, rows, K)
    for t in (r, tx, tw):
        t.release()


@pytest.mark.parametrize("dname", list(cases.DTYPES))
@pytest.mark.parametrize("shapes,dim", [([(2, 8, 5, 64), (2, 8, 1, 64)], 2),          # KV-cache append: one new position
                                        ([(3, 7), (4, 7), (1, 7)], 0), ([(6, 5), (6, 1), (6, 9)], 1),
                                        ([(2, 3, 4), (2, 3, 4)], 2), ([(1, 2, 2048, 128), (1, 2, 2048, 128)], 2)])
def test_cat_matches_concatenate(gpu, dname, shapes, dim):
    """MAG_OP_CAT on the device against numpy.concatenate on the same bit patterns (a pure copy: bit exact)."""
    dt = cases.DTYPES[dname]
    rng = np.random.default_rng(6)
    hosts = [O.f32_to_bits(dt, cases.gen_storage(rng, sh, 1.0)) for sh in shapes]
    tensors = [mb.Tensor.from_bits(gpu, dt, h) for h in hosts]
    out = mb.Tensor.cat(tensors, dim)
    assert np.array_equal(out.to_bits(), np.concatenate(hosts, axis=dim))
    wrong = list(shapes[0])
    wrong[(dim + 1) % len(wrong)] += 1                    # differs on an axis that is not the concat axis
    bad = mb.Tensor.from_bits(gpu, dt, np.zeros(wrong, hosts[0].dtype))
    with pytest.raises(mb.MagB200Error):
        mb.Tensor.cat([tensors[0], bad], dim)
    for t in tensors + [out, bad]:
        t.release()


def test_host_buffer_matmul(gpu):
    dt = O.BFLOAT16
    rng = np.random.default_rng(8)
    xb, wb = bits(dt, rng, (64, 256), 1.0), bits(dt, rng, (96, 256), 0.1)
    out = np.empty((64, 96), np.uint16)
    xv = mb.make_view(xb.ctypes.data, dt, (64, 256))
    wv = mb.make_view(wb.ctypes.data, dt, (256, 96), (1, 256))   # W.T view of the host buffer
    rv = mb.make_view(out.ctypes.data, dt, (64, 96))
    mb.check(mb.lib().magb200_matmul_host(gpu, C.byref(xv), xb.nbytes, C.byref(wv), wb.nbytes, C.byref(rv)))
    truth = O.bits_to_f64(dt, xb) @ O.bits_to_f64(dt, wb).T
    m = O.error_metrics(dt, out, truth, np.abs(O.bits_to_f64(dt, xb)) @ np.abs(O.bits_to_f64(dt, wb)).T)
    assert m["e"] <= unit_roundoff(dt) + 256 * 2.0 ** -24


def test_overlapped_transfers_keep_operator_order(gpu):
    """Uploads and downloads on the copy streams: a chain upload -> matmul -> download, repeated with the same device
    buffers and different host data, returns for every round exactly what the plain path returns."""
    dt = O.BFLOAT16
    rng = np.random.default_rng(21)
    L = mb.lib()
    M, K, N = 512, 1024, 768
    wb = bits(dt, rng, (N, K), 0.05)
    tw = mb.Tensor.from_bits(gpu, dt, wb)
    tx, to = mb.Tensor(gpu, dt, (M, K)), mb.Tensor(gpu, dt, (M, N))
    rounds = 4
    pin_x, pin_o = C.c_void_p(), C.c_void_p()
    mb.check(L.magb200_host_alloc_pinned(C.byref(pin_x), rounds * M * K * 2))
    mb.check(L.magb200_host_alloc_pinned(C.byref(pin_o), rounds * M * N * 2))
    try:
        hx = np.ctypeslib.as_array(C.cast(pin_x, C.POINTER(C.c_uint16)), shape=(rounds, M, K))
        ho = np.ctypeslib.as_array(C.cast(pin_o, C.POINTER(C.c_uint16)), shape=(rounds, M, N))
        ho[:] = 0
        for r in range(rounds):
            hx[r] = bits(dt, rng, (M, K), 1.0)
        want = []
        for r in range(rounds):
            t = mb.Tensor.from_bits(gpu, dt, np.ascontiguousarray(hx[r]))
            want.append((t @ tw.T).to_bits())
            t.release()
        # all rounds are queued without a synchronisation in between, one result buffer per round
        outs = [mb.Tensor(gpu, dt, (M, N)) for _ in range(rounds)]
        for r in range(rounds):
            mb.check(L.magb200_upload_overlapped(gpu, tx.ptr, hx[r].ctypes.data, M * K * 2))
            mb.check(L.magb200_matmul(gpu, C.byref(tx.view_struct()), C.byref(tw.T.view_struct()), C.byref(outs[r].view_struct())))
            mb.check(L.magb200_download_overlapped(gpu, ho[r].ctypes.data, outs[r].ptr, M * N * 2))
        mb.synchronize(gpu)
        for r in range(rounds):
            np.testing.assert_array_equal(ho[r], want[r])
        for t in outs:
            t.release()
    finally:
        L.magb200_host_free_pinned(pin_x)
        L.magb200_host_free_pinned(pin_o)
        for t in (tw, tx, to):
            t.release()


def test_graph_replay_matches_direct_calls(gpu):
    """A recorded sequence of decode-shaped matmuls replays to the same bits as the direct calls."""
    dt = O.BFLOAT16
    rng = np.random.default_rng(12)
    xb = bits(dt, rng, (2, 1024), 1.0)
    ws = [bits(dt, rng, (n, 1024), 0.02) for n in (1024, 3072, 2048)]
    tx = mb.Tensor.from_bits(gpu, dt, xb)
    tws = [mb.Tensor.from_bits(gpu, dt, w) for w in ws]
    outs = [mb.Tensor(gpu, dt, (2, w.shape[0])) for w in ws]
    L = mb.lib()

    def run():
        for w, o in zip(tws, outs):
            mb.check(L.magb200_matmul(gpu, C.byref(tx.view_struct()), C.byref(w.T.view_struct()), C.byref(o.view_struct())))

    run()
    direct = [o.to_bits() for o in outs]
    for o in outs:
        mb.check(L.magb200_fill(gpu, C.byref(o.view_struct()), 0.0))
    graph = C.c_void_p()
    mb.check(L.magb200_graph_begin_capture(gpu))
    run()
    mb.check(L.magb200_graph_end_capture(gpu, C.byref(graph)))
    assert not any(o.to_bits().any() for o in outs)          # capture records, it does not run
    mb.check(L.magb200_graph_launch(gpu, graph))
    mb.synchronize(gpu)
    for d, o in zip(direct, outs):
        assert np.array_equal(d, o.to_bits())
    mb.check(L.magb200_graph_destroy(graph))


def test_errors(gpu):
    a = mb.Tensor.from_bits(gpu, O.BFLOAT16, np.zeros((4, 5), np.uint16))
    b = mb.Tensor.from_bits(gpu, O.BFLOAT16, np.zeros((6, 7), np.uint16))
    with pytest.raises(mb.MagB200Error) as e:
        a @ b
    assert e.value.code == mb.ERR_SHAPE
    c = mb.Tensor.from_bits(gpu, O.FLOAT16, np.zeros((5, 7), np.uint16))
    out = mb.Tensor(gpu, O.BFLOAT16, (4, 7))
    rc = mb.lib().magb200_matmul(gpu, C.byref(a.view_struct()), C.byref(c.view_struct()), C.byref(out.view_struct()))
    assert rc == mb.ERR_INVALID_ARG      # both inputs must share one dtype (core/mag_op_stubs.c:224-247)


# ---- gated MLP: silu(x @ Wg.T) * (x @ Wu.T) ------------------------------------------------------------------------------
def _swiglu_inputs(dt, M, N, K, seed):
    rng = np.random.default_rng(seed)
    return (O.f32_to_bits(dt, cases.gen_storage(rng, (M, K), 1.0)), O.f32_to_bits(dt, cases.gen_storage(rng, (N, K), 0.05)),
            O.f32_to_bits(dt, cases.gen_storage(rng, (N, K), 0.05)))


@pytest.mark.parametrize("dname", ["bf16", "f16"])
@pytest.mark.parametrize("M,N,K,transposed", [(512, 1024, 512, True), (300, 200, 328, True), (1024, 384, 256, False), (64, 256, 128, True)])
def test_gated_mlp_fused_equals_operator_sequence(gpu, dname, M, N, K, transposed):
    """magb200_matmul_swiglu against (1) the same product computed on the device as two matmuls and the elementwise pass
    (bit for bit: the fused drain applies the same roundings), (2) the reference CPU backend running MATMUL, MATMUL, SILU,
    MUL, in the reference tests' 16-bit tolerance, (3) fp64. Shapes: whole tiles, ragged M / N / K, weights as [K, N]
    instead of W.T views, and one too small for the fused kernel (falls back to the operator sequence by itself)."""
    dt = cases.DTYPES[dname]
    xb, gb, ub = _swiglu_inputs(dt, M, N, K, 21)
    if not transposed:
        gb, ub = np.ascontiguousarray(gb.T), np.ascontiguousarray(ub.T)
    tx, tg, tu = (mb.Tensor.from_bits(gpu, dt, b) for b in (xb, gb, ub))
    wg, wu = (tg.T, tu.T) if transposed else (tg, tu)
    fused = tx.matmul_swiglu(wg, wu)
    fused_kernel = mb.last_kernel()
    mb.force_kernel("tcgen05")          # any forced kernel takes the operator-sequence route; this one sums K in the same order
    try:
        plain = tx.matmul_swiglu(wg, wu)
    finally:
        mb.force_kernel(None)
    fb, pb = fused.to_bits(), plain.to_bits()
    if M >= 256:
        assert fused_kernel == "tcgen05_2sm"
        assert np.array_equal(fb, pb)
    xf = O.bits_to_f64(dt, xb)
    gf, uf = (O.bits_to_f64(dt, b) for b in (gb, ub))
    g64, u64 = (xf @ gf.T, xf @ uf.T) if transposed else (xf @ gf, xf @ uf)
    truth = g64 / (1.0 + np.exp(-g64)) * u64
    got = O.bits_to_f64(dt, fb)
    u = unit_roundoff(dt)
    assert np.all(np.abs(got - truth) <= 6 * u * np.abs(truth) + 4 * u * np.abs(u64) * (np.abs(xf) @ np.abs(gf.T if transposed else gf)) + 1e-30)
    if R.available():
        api = R.MagApi("cpu", log_level=1)
        try:
            ra, rg, ru = api.from_bits(dt, xb), api.from_bits(dt, gb), api.from_bits(dt, ub)
            vg, vu = (api.transpose(rg, 0, 1), api.transpose(ru, 0, 1)) if transposed else (rg, ru)
            mg, mu = api.matmul(ra, vg), api.matmul(ra, vu)
            sg = api.silu(mg)
            rr = api.mul(sg, mu)
            ref = O.bits_to_f64(dt, api.to_bits(rr))
            for h in (rr, sg, mu, mg) + ((vg, vu) if transposed else ()) + (ru, rg, ra):
                h.release()
        finally:
            api.close(True)
        # reference operator tests: atol 1e-2, rtol 1e-2 for 16-bit dtypes (test/python/operators/test_matmul.py:7-11)
        if True:
            assert np.all(np.abs(got - ref) <= 1e-2 * max(1.0, np.abs(truth).max()) + 1e-2 * np.abs(ref))
    for t in (fused, plain, tx, tg, tu):
        t.release()
