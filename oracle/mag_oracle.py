"""CPU restatement (numpy) of magnetron's MATMUL and fp32<->bf16/fp16 CAST semantics.

TEST INFRASTRUCTURE ONLY. Nothing in the product path imports this file; tests, the smoke check and
the bench's CPU-baseline leg use it as the checker. It restates, in plain numpy integer / float
arithmetic, what the reference computes for this path, each function naming the reference lines it
follows. Pinning: `tests/test_oracle.py` checks every function here against golden vectors that were
produced by running the unmodified reference CPU backend (built by `oracle/Makefile`), and, where
`oracle/_ref` is present, against the live reference as well.

Conversions operate on raw bit patterns (uint16 / uint32 arrays) so NaN payloads survive numpy.
"""
from __future__ import annotations

import numpy as np

FLOAT32, FLOAT16, BFLOAT16 = 0, 1, 2  # mag_dtype_t, include/magnetron/magnetron.h:171-174
DTYPE_NAME = {FLOAT32: "float32", FLOAT16: "float16", BFLOAT16: "bfloat16"}
BITS_DTYPE = {FLOAT32: np.uint32, FLOAT16: np.uint16, BFLOAT16: np.uint16}
MAX_DIMS = 16


# ------------------------------------------------------------------------------------------------
# conversions
# ------------------------------------------------------------------------------------------------
def f32_to_bf16_bits(u: np.ndarray) -> np.ndarray:
    """magnetron/core/mag_bfloat16.h:47-58 -- every NaN becomes 0x7FC0, otherwise integer RNE
    `(bits + 0x7fff + ((bits>>16)&1)) >> 16` (subnormals rounded, overflow to inf)."""
    u = np.asarray(u, dtype=np.uint32)
    r = ((u.astype(np.uint64) + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return np.where((u & 0x7FFFFFFF) > 0x7F800000, np.uint16(0x7FC0), r)


def bf16_to_f32_bits(h: np.ndarray) -> np.ndarray:
    """magnetron/core/mag_bfloat16.h:60-65 -- `bits << 16`, exact, payloads and sNaN preserved."""
    return np.asarray(h, dtype=np.uint16).astype(np.uint32) << 16


def f32_to_f16_bits(u: np.ndarray) -> np.ndarray:
    """magnetron/cpu/mag_cpu_impl_cast.inl:12-28 on a host with F16C (`vcvtps2ph`, rounding mode 0):
    round-to-nearest-even, gradual underflow, overflow to inf; NaN keeps its sign and the top ten
    payload bits and gets the quiet bit."""
    u = np.asarray(u, dtype=np.uint32)
    sign = ((u >> 16) & 0x8000).astype(np.uint32)
    a = u & 0x7FFFFFFF
    exp = (a >> 23).astype(np.int64)
    man = (a & 0x7FFFFF).astype(np.uint64)
    # results in fp16's normal range (fp32 biased exponent >= 113); a carry out of the mantissa moves
    # into the exponent field, which is the correctly rounded answer (up to and including inf)
    base = (np.maximum(exp - 112, 0).astype(np.uint64) << np.uint64(10)) | (man >> np.uint64(13))
    rem = man & np.uint64(0x1FFF)
    normal = base + ((rem > 0x1000) | ((rem == 0x1000) & ((base & np.uint64(1)) == 1)))
    normal = np.minimum(normal, 0x7C00)
    # results below the normal range: |x| = full * 2^(exp-150); express in units of 2^-24 and round
    full = man | np.uint64(0x800000)
    shift = np.clip(126 - exp, 14, 40).astype(np.uint64)
    q = full >> shift
    r = full & ((np.uint64(1) << shift) - np.uint64(1))
    half = np.uint64(1) << (shift - np.uint64(1))
    sub = q + ((r > half) | ((r == half) & ((q & np.uint64(1)) == 1)))
    sub = np.where(exp == 0, 0, sub)  # fp32 subnormals are far below 2^-25
    out = np.where(exp >= 113, normal, sub).astype(np.uint32)
    out = np.where(a > 0x7F800000, 0x7E00 | ((a >> 13) & 0x3FF), out)  # NaN: quiet bit + top payload bits
    return (out | sign).astype(np.uint16)


def f16_to_f32_bits(h: np.ndarray) -> np.ndarray:
    """magnetron/cpu/mag_cpu_impl_cast.inl:30-46 on a host with F16C (`vcvtph2ps`): exact widening;
    a signalling NaN comes out quiet with its payload shifted up."""
    h = np.asarray(h, dtype=np.uint16).astype(np.uint32)
    sign = (h & 0x8000) << 16
    exp = (h >> 10) & 0x1F
    man = h & 0x3FF
    normal = ((exp + 112) << 23) | (man << 13)
    # subnormal: man * 2^-24, normalise
    with np.errstate(divide="ignore"):
        msb = np.where(man > 0, np.floor(np.log2(np.maximum(man, 1))).astype(np.int64), 0)
    sub = (((msb + 103).astype(np.uint32)) << 23) | ((man << (23 - msb).astype(np.uint32)) & 0x7FFFFF)
    out = np.where(exp == 0, np.where(man == 0, 0, sub), normal)
    out = np.where(exp == 31, np.where(man == 0, 0x7F800000, 0x7FC00000 | (man << 13)), out)
    return (out | sign).astype(np.uint32)


def cast_bits(src: int, dst: int, bits: np.ndarray) -> np.ndarray:
    """mag_cast_table_2D for the fp32/fp16/bf16 pairs (magnetron/cpu/mag_cpu_impl_cast.inl:56-72):
    16-bit <-> 16-bit pairs go through fp32."""
    bits = np.asarray(bits, dtype=BITS_DTYPE[src])
    if src == dst:
        return bits.copy()
    if src == FLOAT32:
        return f32_to_bf16_bits(bits) if dst == BFLOAT16 else f32_to_f16_bits(bits)
    wide = bf16_to_f32_bits(bits) if src == BFLOAT16 else f16_to_f32_bits(bits)
    if dst == FLOAT32:
        return wide
    return f32_to_bf16_bits(wide) if dst == BFLOAT16 else f32_to_f16_bits(wide)


def bits_to_f64(dtype: int, bits: np.ndarray) -> np.ndarray:
    """Exact numeric value of each bit pattern, as float64."""
    if dtype == FLOAT32:
        return np.asarray(bits, dtype=np.uint32).view(np.float32).astype(np.float64)
    wide = bf16_to_f32_bits(bits) if dtype == BFLOAT16 else f16_to_f32_bits(bits)
    return wide.view(np.float32).astype(np.float64)


def f32_to_bits(dtype: int, x: np.ndarray) -> np.ndarray:
    """Round float32 values into the storage dtype with the reference's conversion."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return cast_bits(FLOAT32, dtype, u)


# ------------------------------------------------------------------------------------------------
# strided views (what the backend receives: base buffer, element offset, shape, strides)
# ------------------------------------------------------------------------------------------------
def gather_view(storage: np.ndarray, shape, strides, offset: int = 0) -> np.ndarray:
    """Materialise a (shape, strides, offset) view of a flat storage array; strides in elements,
    0 allowed (magnetron/core/mag_tensor.c:122-157, :217-219)."""
    storage = np.asarray(storage).reshape(-1)
    idx = np.full(tuple(shape) if len(shape) else (), offset, dtype=np.int64)
    for d, (n, s) in enumerate(zip(shape, strides)):
        ax = np.arange(n, dtype=np.int64) * s
        idx = idx + ax.reshape([-1 if i == d else 1 for i in range(len(shape))])
    return storage[idx]


def contiguous_strides(shape) -> tuple:
    st, acc = [], 1
    for n in reversed(shape):
        st.append(acc)
        acc *= n
    return tuple(reversed(st))


# ------------------------------------------------------------------------------------------------
# matmul
# ------------------------------------------------------------------------------------------------
class MatmulShapeError(ValueError):
    """Mirrors MAG_STATUS_ERR_OPERATOR_IMPOSSIBLE from mag_matmul (core/mag_op_stubs.c:1256-1290)."""


def matmul_result_shape(xs, ys) -> tuple:
    """Result shape rules of `mag_matmul` (magnetron/core/mag_op_stubs.c:1249-1310):
    (K)x(K)->() (a rank-0 scalar), (K)x(K,N)->(N), (M,K)x(K)->(M), otherwise batched with
    batch dims broadcast iff equal or 1."""
    xs, ys = tuple(xs), tuple(ys)
    if len(xs) < 1 or len(ys) < 1:
        raise MatmulShapeError("rank")
    kx = xs[-1]
    ky = ys[0] if len(ys) == 1 or (len(ys) == 2 and len(xs) == 1) else ys[-2]
    if kx != ky:
        raise MatmulShapeError(f"K mismatch {kx} != {ky}")
    xb = xs[:-2] if len(xs) > 2 else ()
    yb = ys[:-2] if len(ys) > 2 else ()
    rbd = max(len(xb), len(yb))
    xb = (1,) * (rbd - len(xb)) + xb
    yb = (1,) * (rbd - len(yb)) + yb
    for a, b in zip(xb, yb):
        if a != b and a != 1 and b != 1:
            raise MatmulShapeError(f"batch dims {a} vs {b}")
    if len(xs) == 1 and len(ys) == 1:
        return ()
    if len(xs) == 1 and len(ys) == 2:
        return (ys[1],)
    if len(xs) == 2 and len(ys) == 1:
        return (xs[0],)
    m = 1 if len(xs) == 1 else xs[-2]
    n = 1 if len(ys) == 1 else ys[-1]
    return tuple(max(a, b) for a, b in zip(xb, yb)) + (m, n)


def _as_batched(x: np.ndarray, y: np.ndarray):
    """Promote operands to (..., M, K) and (..., K, N) like the CPU kernels do
    (magnetron/cpu/mag_cpu_impl_ops_matmul.inl:2933-2939: rank-1 x is one row, rank-1 y one column)."""
    if x.ndim == 1:
        x = x[None, :]
    if y.ndim == 1:
        y = y[:, None]
    return x, y


def matmul_f64(dtype: int, x_bits: np.ndarray, y_bits: np.ndarray) -> np.ndarray:
    """fp64 ground truth of the product of the ROUNDED operands; result shape per matmul_result_shape."""
    shape = matmul_result_shape(x_bits.shape, y_bits.shape)
    x, y = _as_batched(bits_to_f64(dtype, x_bits), bits_to_f64(dtype, y_bits))
    return np.matmul(x, y).reshape(shape)


def abs_product_sum(dtype: int, x_bits: np.ndarray, y_bits: np.ndarray) -> np.ndarray:
    """Sum_k |a_ik| |b_kj| -- the scale of the rounding-error bound of one output element."""
    shape = matmul_result_shape(x_bits.shape, y_bits.shape)
    x, y = _as_batched(np.abs(bits_to_f64(dtype, x_bits)), np.abs(bits_to_f64(dtype, y_bits)))
    return np.matmul(x, y).reshape(shape)


def matmul_like_reference(dtype: int, x_bits: np.ndarray, y_bits: np.ndarray, kc: int = 856) -> np.ndarray:
    """Restatement of the reference's rounding structure, returned as bit patterns of `dtype`.

    bf16 (magnetron/cpu/mag_cpu_impl_ops_matmul.inl:2921-3019): fp32 accumulation inside one K panel
    of `kc` elements; between panels the partial C is stored as bf16 and re-read (`acc` = pc, :3015,
    loads at :805-810). fp32 (:2821-2919): fp32 accumulation across panels. fp16 (:3062-3116): one
    fp32 accumulator per output element, one rounding at the end.
    The summation order inside a panel is not restated (it depends on the SIMD width in use), so this
    function pins the error LEVEL of the reference, not its bits."""
    shape = matmul_result_shape(x_bits.shape, y_bits.shape)
    x, y = _as_batched(bits_to_f64(dtype, x_bits).astype(np.float32),
                       bits_to_f64(dtype, y_bits).astype(np.float32))
    K = x.shape[-1]
    if dtype != BFLOAT16:
        acc = np.matmul(x, y).astype(np.float32)
        return f32_to_bits(dtype, acc).reshape(shape)
    c = None
    for pc in range(0, K, kc):
        part = np.matmul(x[..., pc:pc + kc], y[..., pc:pc + kc, :]).astype(np.float32)
        if c is not None:
            part = part + bf16_to_f32_bits(c).view(np.float32)
        c = f32_to_bf16_bits(np.ascontiguousarray(part, dtype=np.float32).view(np.uint32))
    return c.reshape(shape)


def error_metrics(dtype: int, got_bits: np.ndarray, truth: np.ndarray, scale: np.ndarray) -> dict:
    """Accuracy figures used by the gate: `e` = max |got-truth| / sum_k|a||b| (scale-aware form of
    max-relative), `max_rel_floor` = max |got-truth| / max(|truth|, 2^-8 rms(truth)), `max_abs`."""
    got = bits_to_f64(dtype, got_bits).reshape(truth.shape)
    err = np.abs(got - truth)
    tau = 2.0 ** -8 * float(np.sqrt(np.mean(truth ** 2))) if truth.size else 0.0
    return {
        "e": float((err / np.maximum(scale, 1e-300)).max()) if err.size else 0.0,
        "max_rel_floor": float((err / np.maximum(np.abs(truth), max(tau, 1e-300))).max()) if err.size else 0.0,
        "max_abs": float(err.max()) if err.size else 0.0,
    }
