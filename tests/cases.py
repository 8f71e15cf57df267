"""Problem lists shared by the golden-vector generator and the parity tests.

A matmul case names dtype, the STORAGE shapes of both operands and the recipe that turns each
storage into the operand view (transposes, permutes, slices, reshapes), so the same case can be
stated against the reference C API and against the B200 C ABI. Shapes follow the reference's own
operator tests (test/python/operators/test_matmul.py: squares, rectangles, matrix-vector,
vector-matrix, transposed operands, every broadcastable batch pattern), kept small so the CPU side
finishes in seconds.
"""
from __future__ import annotations

import numpy as np

F32, F16, BF16 = 0, 1, 2
DTYPES = {"f32": F32, "f16": F16, "bf16": BF16}

# (name, x storage shape, x ops, y storage shape, y ops); ops: ("T", d0, d1) | ("permute", dims) |
# ("slice", dim, start, length, step) | ("view", shape)
MATMUL_CASES = [
    ("sq4", (4, 4), [], (4, 4), []),
    ("sq33", (33, 33), [], (33, 33), []),
    ("sq64", (64, 64), [], (64, 64), []),
    ("rect", (17, 40), [], (40, 9), []),
    ("rect_big", (130, 72), [], (72, 200), []),
    ("linear_wT", (24, 64), [], (48, 64), [("T", 0, 1)]),                  # x @ W.T  (nn.Linear)
    ("linear_wT_tail", (19, 72), [], (37, 72), [("T", 0, 1)]),
    ("x_T", (40, 17), [("T", 0, 1)], (40, 9), []),                        # x transposed
    ("both_T", (40, 17), [("T", 0, 1)], (9, 40), [("T", 0, 1)]),
    ("x_T_al", (64, 24), [("T", 0, 1)], (64, 16), []),                    # transposed x with a 16-byte-multiple pitch
    ("both_T_al", (64, 136), [("T", 0, 1)], (16, 64), [("T", 0, 1)]),
    ("mat_vec", (12, 32), [], (32,), []),
    ("vec_mat", (32,), [], (32, 12), []),
    ("vec_vec", (48,), [], (48,), []),
    ("gemv_wT", (1, 256), [], (96, 256), [("T", 0, 1)]),                  # decode through W.T
    ("gemv_kn", (1, 128), [], (128, 4096), []),                          # reference GEMV path (N>=4096)
    ("skinny4_wT", (4, 256), [], (64, 256), [("T", 0, 1)]),
    ("skinny8_kn", (8, 64), [], (64, 72), []),
    ("batch_same", (3, 5, 16), [], (3, 16, 8), []),
    ("batch_bcast_y", (2, 3, 5, 16), [], (16, 24), []),
    ("batch_bcast_x", (9, 16), [], (2, 3, 16, 7), []),
    ("batch_mixed", (2, 1, 5, 16), [], (1, 3, 16, 16), []),
    ("batch_rank6", (2, 1, 2, 3, 4, 8), [], (3, 1, 1, 8, 8), []),
    ("batch_y_T", (2, 3, 8, 16), [], (2, 3, 24, 16), [("T", 2, 3)]),       # q @ k.transpose(2,3)
    ("gqa_scores", (1, 2, 2, 16, 8), [], (1, 2, 16, 8), [("T", 2, 3), ("view", (1, 2, 1, 8, 16))]),
    ("gqa_pv", (1, 2, 2, 16, 16), [], (1, 2, 16, 8), [("view", (1, 2, 1, 16, 8))]),
    ("slice_k", (10, 64), [("slice", 1, 16, 32, 1)], (64, 16), [("slice", 0, 16, 32, 1)]),   # row-sharded K slice
    ("slice_n", (10, 32), [], (32, 48), [("slice", 1, 8, 24, 1)]),                           # column shard
    ("stride2", (6, 32), [("slice", 1, 0, 16, 2)], (16, 10), []),                            # inner stride 2
    ("permute_x", (4, 3, 16), [("permute", (1, 0, 2))], (16, 40), []),
    ("k1", (9, 1), [], (1, 11), []),
    ("big_k", (8, 2200), [], (24, 2200), [("T", 0, 1)]),                  # K spans several reference K panels
    ("tile_edge", (129, 96), [], (257, 96), [("T", 0, 1)]),
]


def case_by_name(name):
    for c in MATMUL_CASES:
        if c[0] == name:
            return c
    raise KeyError(name)


def seed_of(name: str, dtype: int) -> int:
    return (sum(ord(ch) * (i + 1) for i, ch in enumerate(name)) * 7 + dtype) % (2 ** 31)


def gen_storage(rng, shape, scale: float) -> np.ndarray:
    """fp32 values ~ N(0, scale^2)."""
    return (rng.standard_normal(shape, dtype=np.float32) * np.float32(scale)).astype(np.float32)


def apply_ops(t, ops):
    """Apply a view recipe to any tensor handle with transpose/permute/slice/view methods."""
    for op in ops:
        if op[0] == "T":
            t = t.transpose(op[1], op[2])
        elif op[0] == "permute":
            t = t.permute(op[1])
        elif op[0] == "slice":
            t = t.slice(op[1], op[2], op[3], op[4])
        elif op[0] == "view":
            t = t.view(op[1])
        else:
            raise ValueError(op)
    return t


class NpView:
    """numpy stand-in with the same view methods, to compute the fp64 truth of a case."""

    def __init__(self, a):
        self.a = a

    def transpose(self, d0, d1):
        return NpView(np.swapaxes(self.a, d0, d1))

    def permute(self, dims):
        return NpView(np.transpose(self.a, dims))

    def slice(self, dim, start, length, step):
        idx = [slice(None)] * self.a.ndim
        idx[dim] = slice(start, start + length * step, step)
        return NpView(self.a[tuple(idx)])

    def view(self, shape):
        return NpView(self.a.reshape(shape))


# fp32 bit patterns every cast test includes (NaNs of both signs and payloads, infinities, zeros,
# subnormals, rounding ties of both target formats, overflow boundaries)
CAST_SPECIAL_F32 = np.array([
    0x00000000, 0x80000000, 0x7F800000, 0xFF800000, 0x7FC00000, 0xFFC00000, 0x7F800001, 0xFF800001,
    0x7F80FFFF, 0x7FA00000, 0x7F801234, 0xFFFFFFFF, 0x7FFFFFFF, 0x00000001, 0x007FFFFF, 0x80000001,
    0x00008000, 0x00018000, 0x00008001, 0x7F7FFFFF, 0xFF7FFFFF, 0x7F7F8000, 0x7F7F7FFF, 0x3F808000,
    0x3F818000, 0x3F808001, 0x3F807FFF, 0x33800000, 0x33000000, 0x33000001, 0x32FFFFFF, 0x477FE000,
    0x477FF000, 0x477FEFFF, 0x47800000, 0x38800000, 0x387FC000, 0x387FE000, 0x387FF000, 0x38000000,
    0x33800001, 0x3F800000, 0xBF800000, 0x3F801000, 0x3F803000, 0x3F802000, 0x3F800FFF, 0x3F801001,
    0x00800000, 0x80800000, 0x34000000, 0x337FFFFF,
], dtype=np.uint32)


def cast_inputs_f32(seed: int, n: int) -> np.ndarray:
    """N(0,1) values with ~1% specials mixed in at seeded positions, as fp32 bit patterns."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal(n, dtype=np.float32).view(np.uint32).copy()
    k = max(n // 100, min(n, len(CAST_SPECIAL_F32)))
    pos = rng.choice(n, size=k, replace=False)
    x[pos] = CAST_SPECIAL_F32[np.arange(k) % len(CAST_SPECIAL_F32)]
    return x
