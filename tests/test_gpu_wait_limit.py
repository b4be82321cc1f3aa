"""A bounded wait inside the GEMM kernel that runs out: the kernel must return with a status code, free its
tensor memory and leave the device usable.

The failure is produced without faulting anything: a test-only build of the kernel (``waittest_build.py``)
whose MMA warp never signals "accumulators complete", with the wait limit cut to two thousand polls.  The
epilogue warps give up, record their code in the status word, every other warp unwinds through its own
bounded waits, and the launch ends by itself within milliseconds.
"""

from __future__ import annotations

import ctypes

import pytest
import torch

from mase_triton_b200 import _lib
from mase_triton_b200.mxfp import gemm as G
from mase_triton_b200.mxfp.meta import MXFP8_E4M3_fn

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


@pytest.fixture(scope="module")
def waitlib():
    from waittest_build import build

    L = ctypes.CDLL(str(build()))
    L.mxq_mx_gemm.argtypes = _lib.SIGNATURES["mxq_mx_gemm"]
    L.mxq_mx_gemm.restype = ctypes.c_int
    return L


@pytest.mark.parametrize("shape", [(256, 448, 256), (512, 224 * 100, 128)], ids=["one-tile-per-cta", "two-tiles-per-cta"])
def test_wait_that_runs_out_reports_and_recovers(lib, waitlib, shape):
    M, N, K = shape
    torch.manual_seed(1)
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (0.05 * torch.randn(N, K, device=DEV)).to(torch.bfloat16)
    a = G.quantize_pack(x, MXFP8_E4M3_fn)
    b = G.quantize_pack(w, MXFP8_E4M3_fn, G.OPERAND_B)
    good = G.mx_gemm(a, b, torch.bfloat16)
    G.check_status(DEV)

    word = G.status_word(DEV)                           # pinned host memory the kernel writes directly
    assert int(word[0]) == 0
    out = torch.zeros((M, N), dtype=torch.bfloat16, device=DEV)
    rc = waitlib.mxq_mx_gemm(a.codes.data_ptr(), a.sf.data_ptr(), a.hw_format, b.codes.data_ptr(), b.sf.data_ptr(), b.hw_format,
                             b.tile_rows, out.data_ptr(), _lib.DTYPE_ID[torch.bfloat16], None, M, N, K, word.data_ptr(),
                             torch.cuda.current_stream(DEV).cuda_stream)
    assert rc == 0
    torch.cuda.synchronize(DEV)                         # the launch ends by itself: no hang, no CUDA error
    assert int(word[0]) in (1, 2, 3), int(word[0])

    # the failure surfaces on the next GEMM call of the Python layer, once, without any synchronising check
    with pytest.raises(_lib.MXQError, match="gave up"):
        G.mx_gemm(a, b, torch.bfloat16)
    assert int(word[0]) == 0
    # tensor memory was released and the context is intact: the product kernel runs and gives the same bytes
    again = G.mx_gemm(a, b, torch.bfloat16)
    G.check_status(DEV)
    assert torch.equal(again, good)
