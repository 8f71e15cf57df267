"""GPU parity tests of MAG_OP_CAST through the C ABI: bit-exact against the golden vectors made by the
reference CPU backend and against the numpy oracle."""
import ctypes as C

import numpy as np
import pytest

import magnetron_b200 as mb
from oracle import mag_oracle as O
from tests import cases
from tests.common import golden

pytestmark = pytest.mark.gpu
PAIRS = [(s, d) for s in (O.FLOAT32, O.FLOAT16, O.BFLOAT16) for d in (O.FLOAT32, O.FLOAT16, O.BFLOAT16)]


def gpu_cast(dev, src, dst, bits):
    t = mb.Tensor.from_bits(dev, src, bits)
    o = t.cast(dst)
    r = o.to_bits()
    t.release(); o.release()
    return r


def test_golden_vectors_bit_exact(gpu):
    g = golden("cast_golden.npz")
    x = g["f32_in"]
    assert np.array_equal(gpu_cast(gpu, O.FLOAT32, O.BFLOAT16, x), g["f32_to_bf16"])
    assert np.array_equal(gpu_cast(gpu, O.FLOAT32, O.FLOAT16, x), g["f32_to_f16"])
    all16 = np.arange(65536, dtype=np.uint16)
    assert np.array_equal(gpu_cast(gpu, O.FLOAT16, O.FLOAT32, all16), g["f16_to_f32"])
    assert np.array_equal(gpu_cast(gpu, O.BFLOAT16, O.FLOAT32, all16), g["bf16_to_f32"])
    assert np.array_equal(gpu_cast(gpu, O.FLOAT16, O.BFLOAT16, all16), g["f16_to_bf16"])
    assert np.array_equal(gpu_cast(gpu, O.BFLOAT16, O.FLOAT16, all16), g["bf16_to_f16"])


def test_strided_source_golden(gpu):
    g = golden("cast_golden.npz")
    t = mb.Tensor.from_bits(gpu, O.FLOAT32, g["strided_in"])
    o = t.T.cast(O.BFLOAT16)
    assert np.array_equal(o.to_bits(), g["strided_T_to_bf16"])


@pytest.mark.parametrize("src,dst", PAIRS)
@pytest.mark.parametrize("n", [1, 7, 8, 9, 255, 1023, 65537])
def test_ragged_sizes_vs_oracle(gpu, src, dst, n):
    x32 = cases.cast_inputs_f32(100 + n, n)
    x = O.cast_bits(O.FLOAT32, src, x32) if src != O.FLOAT32 else x32
    assert np.array_equal(gpu_cast(gpu, src, dst, x), O.cast_bits(src, dst, x))


@pytest.mark.parametrize("src,dst", [(O.FLOAT32, O.BFLOAT16), (O.BFLOAT16, O.FLOAT32), (O.FLOAT32, O.FLOAT16), (O.FLOAT16, O.FLOAT32)])
def test_full_size_16m_with_specials(gpu, src, dst):
    """The 16 Mi-element cast of the single-op workload: N(0,1) with 1% specials, seed 1."""
    n = 1 << 24
    x32 = cases.cast_inputs_f32(1, n)
    x = O.cast_bits(O.FLOAT32, src, x32) if src != O.FLOAT32 else x32
    got = gpu_cast(gpu, src, dst, x)
    assert np.array_equal(got, O.cast_bits(src, dst, x))


def test_exhaustive_upper_halves_f32(gpu):
    """All 65536 upper halves of fp32 crossed with low halves around both rounding ties."""
    lows = np.array([0, 1, 0x0FFF, 0x1000, 0x1001, 0x1FFF, 0x2000, 0x3000, 0x7FFF, 0x8000, 0x8001, 0xFFFF], dtype=np.uint32)
    x = ((np.arange(65536, dtype=np.uint32)[:, None] << 16) | lows[None, :]).reshape(-1)
    for dst in (O.BFLOAT16, O.FLOAT16):
        assert np.array_equal(gpu_cast(gpu, O.FLOAT32, dst, x), O.cast_bits(O.FLOAT32, dst, x))


def test_unaligned_offset_view(gpu):
    """A view that starts at an odd element offset cannot use 128-bit accesses; same bits expected."""
    x = cases.cast_inputs_f32(5, 4099)
    t = mb.Tensor.from_bits(gpu, O.FLOAT32, x)
    v = t.slice(0, 3, 4096)
    assert np.array_equal(v.cast(O.BFLOAT16).to_bits(), O.cast_bits(O.FLOAT32, O.BFLOAT16, x[3:4099]))


def test_permuted_3d_source(gpu):
    x = O.cast_bits(O.FLOAT32, O.BFLOAT16, cases.cast_inputs_f32(9, 6 * 10 * 14)).reshape(6, 10, 14)
    t = mb.Tensor.from_bits(gpu, O.BFLOAT16, x)
    got = t.permute((2, 0, 1)).cast(O.FLOAT32).to_bits()
    assert np.array_equal(got, O.cast_bits(O.BFLOAT16, O.FLOAT32, np.ascontiguousarray(x.transpose(2, 0, 1))))


def test_round_trip_properties(gpu):
    all16 = np.arange(65536, dtype=np.uint16)
    # widening then narrowing returns every non-NaN pattern; NaNs come back canonical (bf16) / quieted (fp16)
    back = gpu_cast(gpu, O.FLOAT32, O.BFLOAT16, gpu_cast(gpu, O.BFLOAT16, O.FLOAT32, all16))
    nan = (all16 & 0x7FFF) > 0x7F80
    assert np.array_equal(back[~nan], all16[~nan]) and np.all(back[nan] == 0x7FC0)
    back = gpu_cast(gpu, O.FLOAT32, O.FLOAT16, gpu_cast(gpu, O.FLOAT16, O.FLOAT32, all16))
    nan = (all16 & 0x7FFF) > 0x7C00
    assert np.array_equal(back[~nan], all16[~nan]) and np.array_equal(back[nan], all16[nan] | 0x0200)


def test_clone_and_fill(gpu):
    x = O.cast_bits(O.FLOAT32, O.FLOAT16, cases.cast_inputs_f32(3, 33 * 65)).reshape(33, 65)
    t = mb.Tensor.from_bits(gpu, O.FLOAT16, x)
    assert np.array_equal(t.T.contiguous().to_bits(), np.ascontiguousarray(x.T))
    f = mb.Tensor(gpu, O.BFLOAT16, (5, 7))
    mb.check(mb.lib().magb200_fill(gpu, C.byref(f.view_struct()), 1.5))
    assert np.all(f.to_bits() == 0x3FC0)


def test_host_buffer_entry_point(gpu):
    x = cases.cast_inputs_f32(21, 100000)
    out = np.empty(x.shape, np.uint16)
    src = mb.make_view(x.ctypes.data, O.FLOAT32, x.shape)
    dst = mb.make_view(out.ctypes.data, O.BFLOAT16, out.shape)
    mb.check(mb.lib().magb200_cast_host(gpu, C.byref(src), x.nbytes, C.byref(dst)))
    assert np.array_equal(out, O.cast_bits(O.FLOAT32, O.BFLOAT16, x))
