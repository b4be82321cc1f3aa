"""Builds the test-only variant of the block-scaled GEMM used by ``test_gpu_wait_limit.py``.

``csrc/mxq_gemm.cu`` is compiled once more with ``-DMXQ_TEST_SPIN_LIMIT=2048`` (every bounded wait gives
up after two thousand polls instead of four million) and ``-DMXQ_TEST_DROP_ACCUM_COMMIT`` (the MMA warp never
signals "accumulators complete", so the epilogue's wait can only run out), and linked with the product's other
objects into ``tests/_build/libmxq_waittest.so``.  Nothing in the product loads this library.
"""

from __future__ import annotations

import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

OUT_DIR = Path(__file__).resolve().parent / "_build"
LIB = OUT_DIR / "libmxq_waittest.so"
FLAGS = ["-DMXQ_TEST_SPIN_LIMIT=2048", "-DMXQ_TEST_DROP_ACCUM_COMMIT"]


def build(force: bool = False) -> Path:
    from mase_triton_b200 import build as lib_build

    csrc = lib_build.CSRC
    newest = max(p.stat().st_mtime for p in list(csrc.glob("*.cu")) + list(csrc.glob("*.h")) + list(csrc.glob("*.cuh")))
    if not force and LIB.exists() and LIB.stat().st_mtime >= newest:
        return LIB
    lib_build.build()                                   # the product objects this variant is linked with
    OUT_DIR.mkdir(exist_ok=True)
    obj = OUT_DIR / "mxq_gemm_waittest.o"
    nvcc = lib_build._nvcc()
    r = subprocess.run([nvcc, *lib_build.NVCC_FLAGS, *FLAGS, "-c", str(csrc / "mxq_gemm.cu"), "-o", str(obj)], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on the wait-limit variant:\n{r.stdout}\n{r.stderr}")
    others = [str(csrc / f"{name}.o") for name in ("mxq_api", "mxq_elementwise", "mxq_bitpack")]
    r = subprocess.run([nvcc, "-shared", "-o", str(LIB), str(obj), *others], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
