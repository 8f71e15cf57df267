"""Helpers shared by the test modules (golden loaders, case materialisation, error gate)."""
from __future__ import annotations

import os
import zlib

import numpy as np

from oracle import mag_oracle as O
from tests import cases

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
_cache = {}


def golden(name: str):
    if name not in _cache:
        _cache[name] = np.load(os.path.join(GOLDEN, name))
    return _cache[name]


def case_operands(name: str, dtype: int):
    """Seeded operand storages (bit patterns) of a matmul case; checked against the CRCs that were
    recorded when the golden results were made."""
    _, xs, _, ys, _ = cases.case_by_name(name)
    rng = np.random.default_rng(cases.seed_of(name, dtype))
    xb = O.f32_to_bits(dtype, cases.gen_storage(rng, xs, 1.0))
    yb = O.f32_to_bits(dtype, cases.gen_storage(rng, ys, 0.25))
    dname = [k for k, v in cases.DTYPES.items() if v == dtype][0]
    crc = golden("matmul_golden.npz")[f"{name}.{dname}.crc"]
    assert zlib.crc32(xb.tobytes()) == crc[0] and zlib.crc32(yb.tobytes()) == crc[1], \
        "seeded operands differ from the ones the golden results were made from"
    return xb, yb


def case_truth(name: str, dtype: int, xb, yb):
    """fp64 product of the rounded operands through the case's views, plus sum_k |a||b|."""
    _, _, xops, _, yops = cases.case_by_name(name)
    xv = cases.apply_ops(cases.NpView(O.bits_to_f64(dtype, xb)), xops).a
    yv = cases.apply_ops(cases.NpView(O.bits_to_f64(dtype, yb)), yops).a
    shape = O.matmul_result_shape(xv.shape, yv.shape)
    x2 = xv[None, :] if xv.ndim == 1 else xv
    y2 = yv[:, None] if yv.ndim == 1 else yv
    truth = np.matmul(x2, y2).reshape(shape)
    scale = np.matmul(np.abs(x2), np.abs(y2)).reshape(shape)
    return truth, scale


def unit_roundoff(dtype: int) -> float:
    return {O.FLOAT32: 2.0 ** -24, O.FLOAT16: 2.0 ** -11, O.BFLOAT16: 2.0 ** -8}[dtype]


def gate(dtype: int, got_bits, ref_bits, truth, scale, K: int):
    """The accuracy gate of this path: the error against the fp64 truth, measured as
    e = max |got - truth| / sum_k |a||b|, must not exceed twice the reference CPU kernel's own error
    on the same inputs. For tiny problems the reference can be exact to the last bit, so the bound
    never drops below what a single correctly rounded result may show (one unit roundoff of the output
    plus the fp32 accumulation bound)."""
    mg = O.error_metrics(dtype, got_bits, truth, scale)
    mr = O.error_metrics(dtype, ref_bits, truth, scale)
    floor = unit_roundoff(dtype) + K * 2.0 ** -24
    assert mg["e"] <= max(2.0 * mr["e"], floor), (mg, mr, floor)
    return mg, mr


def reference_defect_mask(name: str, dtype: int, result_shape) -> np.ndarray:
    """Result elements on which the reference CPU backend itself is wrong at this snapshot (found by
    comparing it with the fp64 truth on plain contiguous inputs):
      * float32 / bfloat16 blocked kernel: when N is not a multiple of 8, the scalar loop that handles
        the last N % 8 columns reads the packed A panel as if it were row-major
        (magnetron/cpu/mag_cpu_impl_ops_matmul.inl:2744-2754, :2785-2796 against the k-major 8-row
        panels written by mag_mm_pack_A_mc_kc_panel8_*), so those columns are wrong for every row
        that sits in a full 8-row panel; a rank-1 y (N = 1) is the extreme case;
      * bfloat16 GEMV fast path (M = 1, N >= 4096, contiguous [K,N] weight, :2940) returns values far
        from the product;
      * float16 with a rank-1 y.
    Golden comparisons skip these elements; the GPU results are still checked there against the fp64
    truth."""
    _, xs, xops, ys, yops = cases.case_by_name(name)
    xv = cases.apply_ops(cases.NpView(np.zeros(xs, np.uint8)), xops).a
    yv = cases.apply_ops(cases.NpView(np.zeros(ys, np.uint8)), yops).a
    mask = np.zeros(result_shape, dtype=bool)
    if yv.ndim == 1 and xv.ndim >= 2 and dtype == O.FLOAT16:
        mask[...] = True
        return mask
    N = 1 if yv.ndim == 1 else yv.shape[-1]
    M = 1 if xv.ndim == 1 else xv.shape[-2]
    K = xv.shape[-1]
    if dtype in (O.FLOAT32, O.BFLOAT16) and N % 8:
        full = M - M % 8                      # rows that sit in full 8-row A panels
        if yv.ndim == 1 and xv.ndim == 1:
            pass                              # dot product: a single row
        elif yv.ndim == 1:
            mask[..., :full] = True           # result has no N axis: (M,K)x(K) -> (M)
        elif xv.ndim == 1:
            pass                              # one row: never a full panel
        else:
            mask[..., :full, N - N % 8:] = True
    if dtype == O.BFLOAT16 and M == 1 and K >= 128 and N >= 4096 and yv.ndim == 2 and yv.strides[-1] == 1:
        mask[...] = True
    return mask
