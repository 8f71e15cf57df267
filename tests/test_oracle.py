"""CPU tests: the numpy restatement in oracle/ against the golden vectors made by the reference,
and (where oracle/_ref is present) against the live reference library."""
import numpy as np
import pytest

from oracle import mag_oracle as O
from oracle import ref_driver as R
from tests import cases
from tests.common import case_operands, case_truth, golden, reference_defect_mask

# Known answers read off the reference CPU backend (F16C host): input -> (bf16, fp16)
KAT_F32 = {
    0x7FC00000: (0x7FC0, 0x7E00), 0xFFC00000: (0x7FC0, 0xFE00), 0x7F800001: (0x7FC0, 0x7E00),
    0xFF800001: (0x7FC0, 0xFE00), 0x7F80FFFF: (0x7FC0, 0x7E07), 0x7FA00000: (0x7FC0, 0x7F00),
    0x00000001: (0x0000, 0x0000), 0x007FFFFF: (0x0080, 0x0000), 0x00008000: (0x0000, 0x0000),
    0x00018000: (0x0002, 0x0000), 0x7F7FFFFF: (0x7F80, 0x7C00), 0x3F808000: (0x3F80, 0x3C04),
    0x3F818000: (0x3F82, 0x3C0C), 0x33800000: (0x3380, 0x0001), 0x33000000: (0x3300, 0x0000),
    0x477FE000: (0x4780, 0x7BFF), 0x477FF000: (0x4780, 0x7C00), 0x38800000: (0x3880, 0x0400),
    0x387FC000: (0x3880, 0x03FF),
}
KAT_F16_TO_F32 = {0x7E00: 0x7FC00000, 0xFE00: 0xFFC00000, 0x7C01: 0x7FC02000, 0xFC01: 0xFFC02000,
                  0x7DFF: 0x7FFFE000, 0x0001: 0x33800000, 0x03FF: 0x387FC000, 0x8001: 0xB3800000,
                  0x7BFF: 0x477FE000, 0x3C00: 0x3F800000}
KAT_BF16_TO_F32 = {0x7F81: 0x7F810000, 0xFF81: 0xFF810000, 0x7FFF: 0x7FFF0000, 0x0001: 0x00010000,
                   0x007F: 0x007F0000, 0x8001: 0x80010000, 0x7F7F: 0x7F7F0000, 0x3F80: 0x3F800000}
KAT_BF16_TO_F16 = {0x7F81: 0x7E08, 0x7FFF: 0x7FF8, 0x0001: 0x0000, 0x7F7F: 0x7C00}


def test_cast_known_answers():
    x = np.array(list(KAT_F32), dtype=np.uint32)
    assert O.f32_to_bf16_bits(x).tolist() == [v[0] for v in KAT_F32.values()]
    assert O.f32_to_f16_bits(x).tolist() == [v[1] for v in KAT_F32.values()]
    h = np.array(list(KAT_F16_TO_F32), dtype=np.uint16)
    assert O.f16_to_f32_bits(h).tolist() == list(KAT_F16_TO_F32.values())
    b = np.array(list(KAT_BF16_TO_F32), dtype=np.uint16)
    assert O.bf16_to_f32_bits(b).tolist() == list(KAT_BF16_TO_F32.values())
    b = np.array(list(KAT_BF16_TO_F16), dtype=np.uint16)
    assert O.cast_bits(O.BFLOAT16, O.FLOAT16, b).tolist() == list(KAT_BF16_TO_F16.values())


def test_cast_golden_vectors():
    g = golden("cast_golden.npz")
    x = g["f32_in"]
    assert np.array_equal(O.cast_bits(O.FLOAT32, O.BFLOAT16, x), g["f32_to_bf16"])
    assert np.array_equal(O.cast_bits(O.FLOAT32, O.FLOAT16, x), g["f32_to_f16"])
    all16 = np.arange(65536, dtype=np.uint16)
    assert np.array_equal(O.cast_bits(O.FLOAT16, O.FLOAT32, all16), g["f16_to_f32"])
    assert np.array_equal(O.cast_bits(O.BFLOAT16, O.FLOAT32, all16), g["bf16_to_f32"])
    assert np.array_equal(O.cast_bits(O.FLOAT16, O.BFLOAT16, all16), g["f16_to_bf16"])
    assert np.array_equal(O.cast_bits(O.BFLOAT16, O.FLOAT16, all16), g["bf16_to_f16"])
    assert np.array_equal(O.cast_bits(O.FLOAT32, O.BFLOAT16, g["strided_in"].T), g["strided_T_to_bf16"])


def test_gather_view_matches_numpy():
    a = np.arange(2 * 3 * 4).reshape(2, 3, 4)
    v = O.gather_view(a, (4, 2, 3), (1, 12, 4), 0)
    assert np.array_equal(v, a.transpose(2, 0, 1))
    assert np.array_equal(O.gather_view(a, (2, 5), (12, 0), 3), np.repeat(a.reshape(2, 12)[:, 3:4], 5, axis=1))


@pytest.mark.parametrize("xs,ys,expect", [
    ((4,), (4,), ()), ((4,), (4, 5), (5,)), ((3, 4), (4,), (3,)), ((3, 4), (4, 5), (3, 5)),
    ((2, 3, 4), (4, 5), (2, 3, 5)), ((3, 4), (7, 4, 5), (7, 3, 5)), ((2, 1, 3, 4), (1, 6, 4, 5), (2, 6, 3, 5)),
])
def test_result_shape_rules(xs, ys, expect):
    assert O.matmul_result_shape(xs, ys) == expect


@pytest.mark.parametrize("xs,ys", [((3, 4), (5, 6)), ((2, 3, 4), (3, 4, 5)), ((4,), (5,))])
def test_result_shape_errors(xs, ys):
    with pytest.raises(O.MatmulShapeError):
        O.matmul_result_shape(xs, ys)


@pytest.mark.parametrize("name", [c[0] for c in cases.MATMUL_CASES])
@pytest.mark.parametrize("dname", list(cases.DTYPES))
def test_matmul_restatement_vs_golden(name, dname):
    """The restated rounding structure reproduces the reference's result shape and error level."""
    dt = cases.DTYPES[dname]
    g = golden("matmul_golden.npz")
    xb, yb = case_operands(name, dt)
    truth, scale = case_truth(name, dt, xb, yb)
    ref = g[f"{name}.{dname}.r"]
    assert tuple(g[f"{name}.{dname}.rshape"]) == truth.shape
    _, _, xops, _, yops = cases.case_by_name(name)
    xv = cases.apply_ops(cases.NpView(xb), xops).a
    yv = cases.apply_ops(cases.NpView(yb), yops).a
    mine = O.matmul_like_reference(dt, np.ascontiguousarray(xv), np.ascontiguousarray(yv))
    ok = ~reference_defect_mask(name, dt, truth.shape)
    if not ok.any():
        pytest.skip("the reference itself is wrong on every element of this case (see reference_defect_mask)")
    a, r = O.bits_to_f64(dt, mine), O.bits_to_f64(dt, ref)
    K = xv.shape[-1]
    u = {O.FLOAT32: 2.0 ** -24, O.FLOAT16: 2.0 ** -11, O.BFLOAT16: 2.0 ** -8}[dt]
    floor = u + K * 2.0 ** -24
    em = (np.abs(a - truth) / np.maximum(scale, 1e-300))[ok].max()
    er = (np.abs(r - truth) / np.maximum(scale, 1e-300))[ok].max()
    # same error class: within 2x of each other, or both at the single-rounding floor
    assert em <= max(2 * er, floor) and er <= max(2 * em, 4 * floor), (em, er, floor)
    # and elementwise close within the reference tests' own tolerances (test/python/operators/test_matmul.py:7-11)
    atol, rtol = ((1e-5, 1e-5) if dt == O.FLOAT32 else (1e-2, 1e-2))
    assert np.all((np.abs(a - r) <= atol * max(1.0, np.abs(truth).max()) + rtol * np.abs(r))[ok])


@pytest.mark.skipif(not R.available(), reason="oracle/_ref not built (reference sources absent)")
def test_live_reference_agrees_with_golden_and_restatement():
    api = R.MagApi("cpu", log_level=1)
    try:
        x = cases.cast_inputs_f32(11, 1 << 16)
        for dst in (O.BFLOAT16, O.FLOAT16):
            t = api.from_bits(O.FLOAT32, x)
            o = api.cast(t, dst)
            assert np.array_equal(api.to_bits(o), O.cast_bits(O.FLOAT32, dst, x))
            t.release(); o.release()
        name, dt = "linear_wT", O.BFLOAT16
        xb, yb = case_operands(name, dt)
        _, _, xops, _, yops = cases.case_by_name(name)
        tx, ty = api.from_bits(dt, xb), api.from_bits(dt, yb)
        vy = cases.apply_ops(ty, yops)
        tr = api.matmul(tx, vy)
        assert np.array_equal(api.to_bits(tr), golden("matmul_golden.npz")[f"{name}.bf16.r"])
        for h in (tr, vy, tx, ty):
            h.release()
    finally:
        api.close(True)
