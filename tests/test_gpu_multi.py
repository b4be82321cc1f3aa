"""Two-GPU checks of the gather-fused column-parallel linear.  They run only where two GPUs are
visible (child processes, one per GPU, NCCL over 127.0.0.1) and are skipped elsewhere."""

from __future__ import annotations

import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

CHILD = r"""
import os, sys
import torch, torch.distributed as dist
sys.path.insert(0, os.environ["MXQ_ROOT"])
from mase_triton_b200 import parallel
from mase_triton_b200.mxfp import gemm as G
from mase_triton_b200.mxfp.layers import MXFPLinearPTQ
from mase_triton_b200.mxfp.meta import MXFP8_E4M3_fn, OCP_MXFP6_E3M2

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
g = torch.Generator().manual_seed(3)
K, N = 512, 1792 + 448
fc = torch.nn.Linear(K, N, bias=True, dtype=torch.bfloat16)
with torch.no_grad():
    fc.weight.copy_((0.05 * torch.randn(N, K, generator=g)).bfloat16())
    fc.bias.copy_(torch.randn(N, generator=g).bfloat16())
layer = MXFPLinearPTQ.from_linear(fc.to(dev), MXFP8_E4M3_fn, OCP_MXFP6_E3M2, None, "XqWqB", "fused")
fused = parallel.GatherFusedMXFPLinear(layer, max_rows=600, dtype=torch.bfloat16)
gathered = parallel.column_parallel_mxfp_linear(layer)
for step, rows in enumerate((600, 257, 64, 600)):
    x = torch.randn(rows, K, generator=g).bfloat16().to(dev)       # same seed on every rank: replicated activation
    want = layer(x)                                                # the whole layer on one GPU
    got = fused(x)
    G.check_status(dev)
    torch.cuda.synchronize()
    assert got.shape == want.shape, (got.shape, want.shape)
    assert torch.equal(got.view(torch.uint8), want.view(torch.uint8)), f"rank {rank} step {step}: fused gather differs"
    via_nccl = gathered(x)
    assert torch.equal(via_nccl.contiguous().view(torch.uint8), want.view(torch.uint8)), f"rank {rank} step {step}: NCCL gather differs"
dist.barrier(device_ids=[rank])
dist.destroy_process_group()
print(f"rank {rank} ok")
"""


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_gather_fused_linear_matches_single_gpu(tmp_path):
    script = tmp_path / "child.py"
    script.write_text(CHILD)
    port = str(_free_port())
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=port,
                   MXQ_ROOT=str(ROOT), NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n[timed out]"
        outs.append(out)
    for rank, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"rank {rank} ok" in out, out[-3000:]
