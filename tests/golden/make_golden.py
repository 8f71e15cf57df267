"""Generates the golden vectors under tests/golden/ by running the UNMODIFIED reference CPU backend.

    make -C oracle REF=<magnetron source tree>   # builds oracle/_ref from the reference sources (needs them on disk)
    python tests/golden/make_golden.py

Outputs (committed):
  cast_golden.npz    fp32 inputs (specials + seeded normals) with the reference's bf16 / fp16 results,
                     and the reference's results for ALL 65536 fp16 and bf16 bit patterns
                     (-> fp32, and the fp16<->bf16 pair).
  matmul_golden.npz  for every case of tests/cases.py and dtype: CRC32 of the seeded operand storages, the
                     reference result (bit patterns), and the reference's error against fp64.
The file records the CPU specialisation the reference picked, because its bf16 rounding depends on it
(magnetron/cpu/mag_cpu_impl_ops_matmul.inl:655-662 vs :772-778).
"""
import os
import sys
import zlib

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(HERE))

from oracle import mag_oracle as O      # noqa: E402
from oracle import ref_driver as R      # noqa: E402
import cases                            # noqa: E402


def main():
    api = R.MagApi("cpu", log_level=1)
    out_cast = {}

    def ref_cast(src, dst, bits):
        t = api.from_bits(src, bits)
        o = api.cast(t, dst)
        r = api.to_bits(o)
        t.release(); o.release()
        return r

    x = np.concatenate([cases.CAST_SPECIAL_F32, cases.cast_inputs_f32(1, 1 << 15)])
    out_cast["f32_in"] = x
    out_cast["f32_to_bf16"] = ref_cast(O.FLOAT32, O.BFLOAT16, x)
    out_cast["f32_to_f16"] = ref_cast(O.FLOAT32, O.FLOAT16, x)
    all16 = np.arange(65536, dtype=np.uint16)
    out_cast["f16_to_f32"] = ref_cast(O.FLOAT16, O.FLOAT32, all16)
    out_cast["bf16_to_f32"] = ref_cast(O.BFLOAT16, O.FLOAT32, all16)
    out_cast["f16_to_bf16"] = ref_cast(O.FLOAT16, O.BFLOAT16, all16)
    out_cast["bf16_to_f16"] = ref_cast(O.BFLOAT16, O.FLOAT16, all16)
    # strided source: cast of a transposed view
    m = cases.cast_inputs_f32(7, 24 * 40).reshape(24, 40)
    t = api.from_bits(O.FLOAT32, m)
    tt = api.transpose(t, 0, 1)
    o = api.cast(tt, O.BFLOAT16)
    out_cast["strided_in"] = m
    out_cast["strided_T_to_bf16"] = api.to_bits(o)
    for h in (t, tt, o):
        h.release()
    np.savez_compressed(os.path.join(HERE, "cast_golden.npz"), **out_cast)

    out_mm = {}
    for name, xs, xops, ys, yops in cases.MATMUL_CASES:
        for dname, dt in cases.DTYPES.items():
            rng = np.random.default_rng(cases.seed_of(name, dt))
            xb = O.f32_to_bits(dt, cases.gen_storage(rng, xs, 1.0))
            yb = O.f32_to_bits(dt, cases.gen_storage(rng, ys, 0.25))
            tx, ty = api.from_bits(dt, xb), api.from_bits(dt, yb)
            vx, vy = cases.apply_ops(tx, xops), cases.apply_ops(ty, yops)
            tr = api.matmul(vx, vy)
            rb = api.to_bits(tr)
            key = f"{name}.{dname}"
            # operands are regenerated from the case seed by the tests; the CRCs detect a drifted generator
            out_mm[key + ".crc"] = np.array([zlib.crc32(xb.tobytes()), zlib.crc32(yb.tobytes())], dtype=np.uint32)
            out_mm[key + ".r"] = rb
            out_mm[key + ".rshape"] = np.array(tr.shape, dtype=np.int64)
            out_mm[key + ".xv"] = np.array([vx.shape, vx.strides], dtype=np.int64)
            out_mm[key + ".yv"] = np.array([vy.shape, vy.strides], dtype=np.int64)
            for h in {id(v): v for v in (tr, vx, vy, tx, ty)}.values():
                h.release()
    out_mm["_cpu"] = np.array(api.cpu_name)
    np.savez_compressed(os.path.join(HERE, "matmul_golden.npz"), **out_mm)
    api.close(True)
    for f in ("cast_golden.npz", "matmul_golden.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    main()
