"""CPU oracle for the MXFP / minifloat fake-quantisation path (TEST INFRASTRUCTURE).

A ctypes front end over ``oracle/mxq_oracle.c``, which restates the reference's
pure-PyTorch fake path (``src/mase_triton/minifloat/fake.py``,
``src/mase_triton/mxfp/fake.py``) in scalar C.  The functions here keep the
fake path's signatures so parity tests read like the reference's own tests.

Only tests, the smoke check and the benchmark's CPU legs may import this
package; the product package never does.

Parity pin: ``oracle/validate_against_reference.py`` compares every function
here bit-for-bit with the reference's fake path, and ``tests/golden`` holds
vectors generated from the reference.
"""

from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import torch

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "_build" / "libmxq_oracle.so"
_ROUND_MODES = {"rn": 0, "ru": 1, "rd": 2, "rz": 3}
_lib = None


def build(force: bool = False) -> Path:
    """Compile the C oracle with the Makefile beside it (gcc, a second or two)."""
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < (_HERE / "mxq_oracle.c").stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "-B"], check=True, capture_output=True)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(str(_LIB_PATH))
        p, i64, i = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
        L.mxq_oracle_minifloat_extract.argtypes = [p, p, i64, i, i, i, i]
        L.mxq_oracle_minifloat_compose.argtypes = [p, p, i64, i, i, i]
        L.mxq_oracle_minifloat_qdq.argtypes = [p, p, i64, i, i, i, i]
        L.mxq_oracle_mxfp_extract.argtypes = [p, p, p, i64, i, i, i, i, i]
        L.mxq_oracle_mxfp_compose.argtypes = [p, p, p, i64, i, i, i, i]
        L.mxq_oracle_log2_roundup_count.argtypes = [i]
        L.mxq_oracle_log2_roundup_count.restype = i
        L.mxq_oracle_num_threads.restype = i
        L.mxq_oracle_set_num_threads.argtypes = [i]
        L.mxq_oracle_set_num_threads.restype = None
        for name in ("minifloat_extract", "minifloat_compose", "minifloat_qdq", "mxfp_extract", "mxfp_compose"):
            getattr(L, f"mxq_oracle_{name}").restype = None
        _lib = L
    return _lib


def num_threads() -> int:
    return lib().mxq_oracle_num_threads()


def set_num_threads(n: int) -> None:
    """OpenMP threads used by the oracle (launchers such as torchrun export OMP_NUM_THREADS=1)."""
    lib().mxq_oracle_set_num_threads(int(n))


def _fmt(meta):
    """(exp_bits, frac_bits, is_finite, round_mode id) of a MinifloatMeta-like object."""
    return int(meta.exp_bits), int(meta.frac_bits), int(bool(meta.is_finite)), _ROUND_MODES[meta.round_mode]


def _mx_fmt(m):
    return (int(m.block_size), int(m.element_exp_bits), int(m.element_frac_bits),
            int(bool(m.element_is_finite)), _ROUND_MODES[m.round_mode])


def _f32(x: torch.Tensor) -> torch.Tensor:
    assert x.device.type == "cpu", "the oracle runs on CPU tensors"
    return x.detach().to(torch.float32).contiguous()


def log2_roundup_count(e: int) -> int:
    """How many fp32 values just below 2**(e+1) have floor(log2f(v)) == e+1."""
    return lib().mxq_oracle_log2_roundup_count(int(e))


# --- minifloat (reference: src/mase_triton/minifloat/fake.py) ----------------------------------

def extract_minifloat_component(x: torch.Tensor, minifloat_meta) -> torch.Tensor:
    """fp tensor -> uint16 codes of the same shape (fake.py:7-78)."""
    eb, fb, fin, rm = _fmt(minifloat_meta)
    xf = _f32(x)
    out = torch.empty(xf.shape, dtype=torch.uint16)
    lib().mxq_oracle_minifloat_extract(xf.data_ptr(), out.data_ptr(), xf.numel(), eb, fb, fin, rm)
    return out


def compose_minifloat_component(elements: torch.Tensor, minifloat_meta, output_dtype: torch.dtype) -> torch.Tensor:
    """uint16 codes -> tensor of ``output_dtype`` (fake.py:81-125)."""
    assert elements.dtype == torch.uint16
    eb, fb, fin, _ = _fmt(minifloat_meta)
    el = elements.contiguous()
    out = torch.empty(el.shape, dtype=torch.float32)
    lib().mxq_oracle_minifloat_compose(el.data_ptr(), out.data_ptr(), el.numel(), eb, fb, fin)
    return out.to(output_dtype)


def quantize_dequantize_minifloat(x: torch.Tensor, minifloat_meta, output_dtype: torch.dtype | None = None) -> torch.Tensor:
    """extract then compose in one pass (minifloat/functional/cast.py:72-90)."""
    eb, fb, fin, rm = _fmt(minifloat_meta)
    xf = _f32(x)
    out = torch.empty(xf.shape, dtype=torch.float32)
    lib().mxq_oracle_minifloat_qdq(xf.data_ptr(), out.data_ptr(), xf.numel(), eb, fb, fin, rm)
    return out.to(x.dtype if output_dtype is None else output_dtype)


# --- MXFP (reference: src/mase_triton/mxfp/fake.py) -------------------------------------------

def extract_mxfp_components(tensor: torch.Tensor, mxfp_meta) -> tuple[torch.Tensor, torch.Tensor]:
    """flattened fp tensor -> (scales u8 [n_blocks,1], elements u8 [n_blocks,B]) (fake.py:11-59)."""
    B, eb, fb, fin, rm = _mx_fmt(mxfp_meta)
    xf = _f32(tensor).flatten()
    n = xf.numel()
    assert n % B == 0
    scales = torch.empty((n // B, 1), dtype=torch.uint8)
    elements = torch.empty((n // B, B), dtype=torch.uint8)
    lib().mxq_oracle_mxfp_extract(xf.data_ptr(), scales.data_ptr(), elements.data_ptr(), n, B, eb, fb, fin, rm)
    return scales, elements


def compose_mxfp_tensor(scales: torch.Tensor, elements: torch.Tensor, mxfp_meta, output_dtype: torch.dtype) -> torch.Tensor:
    """(scales, elements) -> flat tensor of ``output_dtype`` (fake.py:62-79)."""
    assert scales.dtype == torch.uint8
    assert elements.dtype == torch.uint8
    B, eb, fb, fin, _ = _mx_fmt(mxfp_meta)
    sc, el = scales.contiguous(), elements.contiguous()
    n = el.numel()
    out = torch.empty(n, dtype=torch.float32)
    lib().mxq_oracle_mxfp_compose(sc.data_ptr(), el.data_ptr(), out.data_ptr(), n, B, eb, fb, fin)
    return out.to(output_dtype)
