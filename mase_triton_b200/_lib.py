"""ctypes binding of ``csrc/libmxq.so`` (the C ABI declared in ``include/mxq.h``).

There is no fallback: if the shared object is missing or a call fails, the error
is raised to the caller.
"""

from __future__ import annotations

import ctypes
from pathlib import Path

import torch

LIB_PATH = Path(__file__).resolve().parent / "csrc" / "libmxq.so"

DTYPE_ID = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
ROUND_ID = {"rn": 0, "ru": 1, "rd": 2, "rz": 3}

_p, _i, _i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
# name -> argument types; every function returns an int status unless noted
SIGNATURES = {
    "mxq_minifloat_extract": [_p, _i, _p, _i64, _i, _i, _i, _i, _p],
    "mxq_minifloat_compose": [_p, _p, _i, _i64, _i, _i, _i, _p],
    "mxq_minifloat_qdq": [_p, _i, _p, _i, _i64, _i, _i, _i, _i, _p],
    "mxq_mxfp_extract": [_p, _i, _p, _p, _i64, _i, _i, _i, _i, _i, _p],
    "mxq_mxfp_compose": [_p, _p, _p, _i, _i64, _i, _i, _i, _i, _p],
    "mxq_mxfp_qdq": [_p, _i, _p, _i, _i64, _i, _i, _i, _i, _i, _p],
    "mxq_mxfp_extract_strided": [_p, _i, _p, _p, _i64, _i64, _i64, _i, _i, _i, _i, _i, _p],
    "mxq_mxfp_compose_strided": [_p, _p, _p, _i, _i64, _i64, _i64, _i, _i, _i, _i, _p],
    "mxq_mxfp_qdq_strided": [_p, _i, _p, _i, _i64, _i64, _i64, _i, _i, _i, _i, _i, _p],
    "mxq_mx_pack_operand": [_p, _p, _i64, _i64, _i, _i, _i, _i, _p, _p, _p, _p],
    "mxq_mx_pack_operand_native": [_p, _p, _i64, _i64, _i, _i, _i, _i, _p, _p, _p, _p],
    "mxq_mx_best_tile_rows": [_i64],
    "mxq_mx_quantize_pack": [_p, _i, _i64, _i64, _i, _i, _p, _p, _p, _p],
    "mxq_minifloat_quantize_pack": [_p, _i, _i64, _i64, _i, _i, _i, _p, _p, _p, _p],
    "mxq_mx_gemm": [_p, _p, _i, _p, _p, _i, _i, _p, _i, _p, _i64, _i64, _i64, _p, _p],
    "mxq_mx_gemm_qbias": [_p, _p, _i, _p, _p, _i, _i, _p, _i, _p, _p, _i, _i, _i64, _i64, _i64, _p, _p],
    "mxq_mx_gemm_gather": [_p, _p, _i, _p, _p, _i, _i, _p, _i, _i, _i64, _i64, _i, _p, _i64, _i64, _i64, _p, _p],
    "mxq_mx_linear": [_p, _i, _i64, _i64, _i, _i, _p, _p, _i, _i, _i64, _p, _i, _p, _p, _i64, _p, _p],
    "mxq_mx_linear_static": [_p, _i, _i64, _i64, _i, _i, _p, _p, _i, _i, _i64, _p, _i, _p, _p, _p],
    "mxq_dense_linear": [_p, _p, _i, _p, _p, _i64, _i64, _i64, _p, _p],
    "mxq_mxfp_weight_linear": [_p, _i, _p, _p, _i, _i, _p, _p, _i64, _i64, _i64, _p, _p],
    "mxq_minifloat_weight_linear": [_p, _i, _p, _i, _i, _i, _p, _p, _i64, _i64, _i64, _p, _p],
    "mxq_pack_codes": [_p, _p, _i64, _i, _p],
    "mxq_unpack_codes": [_p, _p, _i64, _i, _p],
    "mxq_version": [],
}
_I64_FUNCS = {"mxq_mx_sf_bytes": [_i64, _i64, _i, _i], "mxq_packed_bytes": [_i64, _i], "mxq_mx_linear_scratch_bytes": [_i64, _i64],
              "mxq_mx_linear_static_capacity": []}
_STRING_FUNCS = {"mxq_status_string": [_i], "mxq_last_cuda_error": []}

_lib = None


class MXQError(RuntimeError):
    """A libmxq entry point returned a non-zero status."""


def load() -> ctypes.CDLL:
    """Load libmxq.so once and declare its signatures. Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise MXQError(f"{LIB_PATH} is missing: build it with `python -m mase_triton_b200.build` "
                           "(there is no CPU or PyTorch fallback)")
        L = ctypes.CDLL(str(LIB_PATH))
        for name, args in SIGNATURES.items():
            fn = getattr(L, name)
            fn.argtypes, fn.restype = args, _i
        for name, args in _I64_FUNCS.items():
            fn = getattr(L, name)
            fn.argtypes, fn.restype = args, _i64
        for name, args in _STRING_FUNCS.items():
            fn = getattr(L, name)
            fn.argtypes, fn.restype = args, ctypes.c_char_p
        _lib = L
    return _lib


def check(status: int, what: str) -> None:
    if status != 0:
        L = load()
        msg = L.mxq_status_string(status).decode()
        if status == -2:
            msg += ": " + L.mxq_last_cuda_error().decode()
        raise MXQError(f"{what} failed: {msg} (status {status})")


def require_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise MXQError(f"{what}: tensor is on {t.device}; this library only runs on CUDA devices (no CPU fallback)")


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def fmt_args(meta) -> tuple[int, int, int, int]:
    """(exp_bits, frac_bits, is_finite, round mode id) of a MinifloatMeta."""
    return meta.exp_bits, meta.frac_bits, int(bool(meta.is_finite)), ROUND_ID[meta.round_mode]
