"""Builds the sm_100a shared libraries of this package with nvcc (in-tree, no JIT cache).

    python -m magnetron_b200.build            # libmagnetron_b200.so (+ the backend module when the
                                              #  magnetron headers are available)

Outputs land in `magnetron_b200/lib/`:
  libmagnetron_b200.so   the C ABI of include/magnetron_b200.h (kernels + host front-end)
  libmagnetron_cuda.so   the same objects plus the magnetron backend module (C host code compiled
                         against the magnetron headers found under $MAGNETRON_SRC, or in a directory named
                         `reference` beside this repository); skipped with a note when those headers are absent.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "lib")
OBJ = os.path.join(PKG, "build")
CU_SOURCES = ["cabi.cu", "cast.cu", "gemv.cu", "gemm_simt.cu", "gemm_tcgen05.cu", "skinny_noalloc.cu", "tp_reduce.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr"]


def magnetron_source_tree() -> str | None:
    """Where the magnetron sources lie: $MAGNETRON_SRC, else a directory named `reference` beside this repository.
    None when neither holds the backend header; nothing of that tree is ever copied, it is only compiled against."""
    for cand in (os.environ.get("MAGNETRON_SRC"), os.path.join(os.path.dirname(ROOT), "reference")):
        if cand and os.path.exists(os.path.join(cand, "magnetron", "core", "mag_backend.h")):
            return cand
    return None


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _run(cmd, verbose):
    if verbose:
        print("  " + " ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("command failed: " + " ".join(cmd))
    return res.stdout + res.stderr


def _stale(out: str, deps) -> bool:
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(verbose: bool = False, ptxas_info: bool = False) -> dict:
    os.makedirs(LIB, exist_ok=True)
    os.makedirs(OBJ, exist_ok=True)
    nvcc = _nvcc()
    headers = [os.path.join(CSRC, "common.cuh"), os.path.join(ROOT, "include", "magnetron_b200.h")]
    objs, log = [], ""
    for src in CU_SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ, src.replace(".cu", ".o"))
        if _stale(o, [s] + headers) or ptxas_info:
            extra = ["-Xptxas", "-v"] if ptxas_info else []
            log += _run([nvcc] + NVCC_FLAGS + extra + ["-DMAGB200_BUILDING", "-c", s, "-o", o], verbose)
        objs.append(o)
    out = {"log": log}
    lib = os.path.join(LIB, "libmagnetron_b200.so")
    if _stale(lib, objs):
        _run([nvcc, "-shared", "-o", lib] + objs + ["-cudart", "static", "-lpthread", "-ldl", "-lrt"], verbose)
    out["cabi"] = lib

    # backend module: C host code against the magnetron headers (never copied into this tree)
    ref = magnetron_source_tree() or ""
    backend_src = os.path.join(CSRC, "backend", "mag_b200_backend.c")
    plugin = os.path.join(LIB, "libmagnetron_cuda.so")
    core_dir = os.path.join(ROOT, "oracle", "_ref")
    if os.path.exists(os.path.join(ref, "magnetron", "core", "mag_backend.h")) and os.path.exists(backend_src) \
            and os.path.exists(os.path.join(core_dir, "libmagnetron_core.so")):
        bobj = os.path.join(OBJ, "mag_b200_backend.o")
        if _stale(bobj, [backend_src] + headers):
            _run(["/usr/bin/gcc", "-std=gnu99", "-O2", "-fPIC", "-fvisibility=hidden", "-DNDEBUG", "-D_GNU_SOURCE=1",
                  "-Wall", "-Wno-unused-function", "-I" + os.path.join(ref, "include"), "-I" + os.path.join(ref, "magnetron"),
                  "-I" + os.path.join(ROOT, "include"), "-c", backend_src, "-o", bobj], verbose)
        if _stale(plugin, objs + [bobj]):
            _run([nvcc, "-shared", "-o", plugin] + objs + [bobj] +
                 ["-cudart", "static", "-lpthread", "-ldl", "-lrt", "-L" + core_dir, "-lmagnetron_core",
                  "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"], verbose)
        out["plugin"] = plugin
    else:
        out["plugin"] = plugin if os.path.exists(plugin) else None
        if verbose:
            print("  backend module not rebuilt (magnetron headers or the reference core are not present here)")
    return out


if __name__ == "__main__":
    r = build(verbose=True, ptxas_info="--ptxas" in sys.argv)
    if "--ptxas" in sys.argv:
        print(r["log"])
    print({k: v for k, v in r.items() if k != "log"})
