"""Generate the golden vectors under tests/golden/ from the reference's own fake path.

Run where the reference checkout is available:

    python tests/golden/make_golden.py path/to/mase-triton/src

Writes
  * golden_small.npz  - inputs and the reference's outputs for small adversarial cases
                        (minifloat extract / compose, MXFP extract / compose, every preset);
  * golden_digests.json - SHA-256 digests of the reference's outputs on the full-size benchmark
                        configurations 1-3 (inputs come from mase_triton_b200.synthetic), so the CUDA
                        path can be pinned to the reference at full size without shipping the data.
The tests only read these files; nothing reads the reference at test time.
"""

from __future__ import annotations

import hashlib
import json
import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))
if len(sys.argv) < 2 and "MASE_TRITON_SRC" not in os.environ:
    raise SystemExit("usage: python " + sys.argv[0] + " <path to the src/ folder of a mase-triton checkout> (or set MASE_TRITON_SRC)")
REF_SRC = sys.argv[1] if len(sys.argv) > 1 else os.environ["MASE_TRITON_SRC"]
sys.path.insert(0, REF_SRC)

from helpers import PRESETS, adversarial_fp32, adversarial_mx_blocks  # noqa: E402
from mase_triton.minifloat import fake as ref_mf  # noqa: E402
from mase_triton.minifloat import functional as ref_mf_F  # noqa: E402
from mase_triton.minifloat.meta import MinifloatMeta  # noqa: E402
from mase_triton.mxfp import fake as ref_mx  # noqa: E402
from mase_triton.mxfp.meta import MXFPMeta  # noqa: E402

from mase_triton_b200 import synthetic  # noqa: E402


def as_np(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy()
    return t.numpy()


def digest(t: torch.Tensor) -> str:
    t = t.contiguous()
    raw = t.view(torch.uint8) if t.dtype != torch.uint8 else t
    return hashlib.sha256(raw.numpy().tobytes()).hexdigest()


def small() -> dict:
    out = {}
    x = adversarial_fp32(4096, seed=2024)
    out["mf_x"] = as_np(x)
    codes = torch.arange(0, 2048, dtype=torch.int32).to(torch.uint16)
    out["mf_codes"] = codes.numpy()
    for name, (eb, fb) in PRESETS.items():
        for fin in (True, False):
            for rm in ("rn", "ru", "rd", "rz"):
                meta = MinifloatMeta(exp_bits=eb, frac_bits=fb, is_finite=fin, round_mode=rm)
                out[f"mf_extract/{name}/{int(fin)}/{rm}"] = ref_mf.extract_minifloat_component(x, meta).numpy()
            meta = MinifloatMeta(exp_bits=eb, frac_bits=fb, is_finite=fin, round_mode="rn")
            for dt in (torch.float32, torch.bfloat16, torch.float16):
                out[f"mf_compose/{name}/{int(fin)}/{str(dt)[6:]}"] = as_np(ref_mf.compose_minifloat_component(codes, meta, dt))
    for eb, fb in ((5, 10), (8, 7), (3, 4)):
        meta = MinifloatMeta(exp_bits=eb, frac_bits=fb, is_finite=True, round_mode="rn")
        out[f"mf_extract/e{eb}m{fb}/1/rn"] = ref_mf.extract_minifloat_component(x, meta).numpy()
    # MXFP: 96 blocks of 32 plus 96 blocks of 8, three input dtypes
    for B in (32, 8):
        base = adversarial_mx_blocks(96, B, seed=77)
        for dt in (torch.float32, torch.bfloat16, torch.float16):
            xin = base.to(dt).flatten()
            dn = str(dt)[6:]
            out[f"mx_x/{B}/{dn}"] = as_np(xin)
            for name, (eb, fb) in PRESETS.items():
                for fin in (True, False):
                    for rm in (("rn", "rz") if B == 32 else ("rn",)):
                        meta = MXFPMeta(block_size=B, scale_exp_bits=8, element_exp_bits=eb, element_frac_bits=fb,
                                        element_is_finite=fin, round_mode=rm)
                        s, e = ref_mx.extract_mxfp_components(xin, meta)
                        key = f"{B}/{dn}/{name}/{int(fin)}/{rm}"
                        out[f"mx_scales/{key}"] = s.numpy()
                        out[f"mx_elements/{key}"] = e.numpy()
                        if rm == "rn":
                            out[f"mx_composed/{key}"] = as_np(ref_mx.compose_mxfp_tensor(s, e, meta, dt))
    # MXFP compose on hand-picked scales x every code
    sc_vals = [0, 1, 2, 23, 100, 126, 127, 128, 150, 200, 230, 253, 254, 255, 64, 192]
    sc = torch.tensor(sc_vals, dtype=torch.uint8).repeat_interleave(8).reshape(-1, 1)
    el = torch.arange(256, dtype=torch.int32).to(torch.uint8).repeat(len(sc_vals)).reshape(-1, 32)
    out["mxc_scales"], out["mxc_elements"] = sc.numpy(), el.numpy()
    for name, (eb, fb) in PRESETS.items():
        for fin in (True, False):
            meta = MXFPMeta(block_size=32, scale_exp_bits=8, element_exp_bits=eb, element_frac_bits=fb,
                            element_is_finite=fin, round_mode="rn")
            for dt in (torch.float32, torch.bfloat16, torch.float16):
                out[f"mxc_out/{name}/{int(fin)}/{str(dt)[6:]}"] = as_np(ref_mx.compose_mxfp_tensor(sc, el, meta, dt))
    return out


def digests() -> dict:
    d = {"torch": torch.__version__}
    # config 1: MXFP8 E4M3, fp32 [4096, 4096]
    x = synthetic.cfg1_mxfp8_fp32()
    meta = MXFPMeta(32, 8, 4, 3, True, "rn")
    s, e = ref_mx.extract_mxfp_components(x.flatten(), meta)
    y = ref_mx.compose_mxfp_tensor(s, e, meta, torch.float32)
    d["cfg1"] = {"input": digest(x), "scales": digest(s), "elements": digest(e), "composed": digest(y)}
    # config 2: minifloat E5M2 quantize_dequantize, fp32 [8192, 8192] (is_finite True and False)
    x = synthetic.cfg2_minifloat_fp32()
    d["cfg2"] = {"input": digest(x)}
    for fin in (True, False):
        meta = MinifloatMeta(5, 2, fin, "rn")
        h = hashlib.sha256()
        hc = hashlib.sha256()
        for r0 in range(0, x.shape[0], 1024):
            c = ref_mf.extract_minifloat_component(x[r0:r0 + 1024], meta)
            hc.update(c.contiguous().view(torch.uint8).numpy().tobytes())
            h.update(ref_mf.compose_minifloat_component(c, meta, torch.float32).contiguous().view(torch.uint8).numpy().tobytes())
        d["cfg2"][f"codes_fin{int(fin)}"] = hc.hexdigest()
        d["cfg2"][f"qdq_fin{int(fin)}"] = h.hexdigest()
    # config 3: MXFP4 E2M1, bf16 [16384, 8192], hashed in row chunks (rows are independent)
    x = synthetic.cfg3_mxfp4_bf16()
    meta = MXFPMeta(32, 8, 2, 1, True, "rn")
    hs, he, hy = hashlib.sha256(), hashlib.sha256(), hashlib.sha256()
    for r0 in range(0, x.shape[0], 2048):
        s, e = ref_mx.extract_mxfp_components(x[r0:r0 + 2048].flatten(), meta)
        y = ref_mx.compose_mxfp_tensor(s, e, meta, torch.bfloat16)
        hs.update(s.numpy().tobytes())
        he.update(e.numpy().tobytes())
        hy.update(y.view(torch.int16).numpy().tobytes())
    d["cfg3"] = {"input": digest(x), "scales": hs.hexdigest(), "elements": he.hexdigest(), "composed": hy.hexdigest()}
    return d


if __name__ == "__main__":
    s = small()
    np.savez_compressed(HERE / "golden_small.npz", **s)
    print("golden_small.npz:", (HERE / "golden_small.npz").stat().st_size, "bytes,", len(s), "arrays")
    d = digests()
    (HERE / "golden_digests.json").write_text(json.dumps(d, indent=1) + "\n")
    print(json.dumps(d, indent=1))
