"""mxq_mx_linear_static: the linear entry point for hosts that cannot allocate device memory.

Such hosts (a serving loop that owns all device memory through its own arena, a plugin that must
not touch the process allocator, code running while a CUDA graph is being captured elsewhere) give
the library no scratch buffer; the library uses a fixed 8 MiB array of its own instead.  The test
drives both entry points through the C ABI on the same inputs and expects identical bytes, twice in
a row with different data, because the array is shared by every call and keeps old contents.
This file is collected last on purpose: it is the only test that depends on library-global state.
"""

from __future__ import annotations

import pytest
import torch

from mase_triton_b200 import _lib
from mase_triton_b200.mxfp import gemm as G
from mase_triton_b200.mxfp.meta import MXFP8_E4M3_fn, OCP_MXFP6_E3M2

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _linear(L, fn_name, x, w: G.PackedOperand, bias, extra_scratch=None, x_meta=MXFP8_E4M3_fn):
    M, K = x.shape
    out = torch.empty((M, w.rows), dtype=x.dtype, device=x.device)
    status = torch.zeros(1, dtype=torch.int32, device=x.device)
    head = [x.data_ptr(), _lib.DTYPE_ID[x.dtype], M, K, x_meta.element_exp_bits, x_meta.element_frac_bits,
            w.codes.data_ptr(), w.sf.data_ptr(), w.hw_format, w.tile_rows, w.rows, out.data_ptr(), _lib.DTYPE_ID[out.dtype],
            None if bias is None else bias.data_ptr()]
    tail = [status.data_ptr(), torch.cuda.current_stream(x.device).cuda_stream]
    if extra_scratch is not None:
        head += [extra_scratch.data_ptr(), extra_scratch.numel()]
    rc = getattr(L, fn_name)(*head, *tail)
    torch.cuda.synchronize()
    return rc, out, int(status.item())


def test_static_scratch_linear_matches_caller_scratch_linear(lib):
    L = lib
    assert L.mxq_mx_linear_static_capacity() == 8 << 20
    torch.manual_seed(123)
    K, N = 1024, 1536
    w = (0.02 * torch.randn(N, K, device=DEV)).to(torch.bfloat16)
    wq = G.quantize_pack(w, OCP_MXFP6_E3M2, G.OPERAND_B)
    bias = torch.randn(N, device=DEV).to(torch.bfloat16)
    # calls in a row with different shapes and data: a later one must not see an earlier one's leftovers.
    # MXFP8 activations are quantised and packed in one kernel; the 6-bit activation takes the other route
    # inside the library (extract into the scratch, then an in-place re-encode), which uses more of the array.
    for M, use_bias, x_meta in ((512, True, MXFP8_E4M3_fn), (200, False, MXFP8_E4M3_fn), (384, True, OCP_MXFP6_E3M2),
                                (130, False, MXFP8_E4M3_fn)):
        x = (torch.randn(M, K, device=DEV) * 2).to(torch.bfloat16)
        scratch = torch.empty(L.mxq_mx_linear_scratch_bytes(M, K), dtype=torch.uint8, device=DEV)
        b = bias if use_bias else None
        rc_ref, y_ref, st_ref = _linear(L, "mxq_mx_linear", x, wq, b, extra_scratch=scratch, x_meta=x_meta)
        rc_new, y_new, st_new = _linear(L, "mxq_mx_linear_static", x, wq, b, x_meta=x_meta)
        assert (rc_ref, st_ref) == (0, 0) and (rc_new, st_new) == (0, 0)
        assert torch.equal(y_new.view(torch.int16), y_ref.view(torch.int16)), f"M={M}: outputs differ"
        assert y_new.float().abs().max() > 0


def test_static_scratch_rejects_oversized_activation(lib):
    L = lib
    K, N = 4096, 256
    M = 4096                      # 16 Mi elements: more than the 8 MiB scratch can hold
    assert L.mxq_mx_linear_scratch_bytes(M, K) > L.mxq_mx_linear_static_capacity()
    x = torch.zeros(M, K, dtype=torch.bfloat16, device=DEV)
    wq = G.quantize_pack(torch.ones(N, K, dtype=torch.bfloat16, device=DEV), MXFP8_E4M3_fn, G.OPERAND_B)
    rc, _, _ = _linear(L, "mxq_mx_linear_static", x, wq, None)
    assert rc == -3               # MXQ_ESIZE
    assert L.mxq_status_string(rc) == b"size not supported by this entry point"
