"""Multi-GPU checks of the gather-fused column-parallel linear at 2, 4 and 8 ranks (child processes, one per
GPU, NCCL over 127.0.0.1; each size is skipped where fewer GPUs are visible), and of one process that drives
two GPUs through the same library."""

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
K, N = 512, 1792 + 448 + 64 * world
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


@pytest.mark.parametrize("world", [2, 4, 8])
def test_gather_fused_linear_matches_single_gpu(tmp_path, world):
    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    script = tmp_path / "child.py"
    script.write_text(CHILD)
    port = str(_free_port())
    procs = []
    for rank in range(world):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=port,
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


def test_one_process_two_devices(lib):
    """The per-device set-up of the GEMM kernels (shared-memory limit, SM count, scratch, status word) is
    kept per device: the same process runs a fused linear on cuda:0 and then on cuda:1."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from mase_triton_b200 import tc_linear
    from mase_triton_b200.mxfp import gemm as G
    from mase_triton_b200.mxfp.layers import MXFPLinearPTQ
    from mase_triton_b200.mxfp.meta import MXFP8_E4M3_fn

    torch.manual_seed(0)
    fc = torch.nn.Linear(512, 768, bias=True, dtype=torch.bfloat16)
    x = torch.randn(300, 512).bfloat16()
    outs, dense = [], []
    for dev in ("cuda:0", "cuda:1"):
        layer = MXFPLinearPTQ.from_linear(fc.to(dev), MXFP8_E4M3_fn, MXFP8_E4M3_fn, None, "XqWqB", "fused")
        outs.append(layer(x.to(dev)).cpu())
        dense.append(tc_linear.dense_linear(x.to(dev), fc.weight.detach().to(dev), fc.bias.detach().to(dev)).cpu())
        G.check_status(torch.device(dev))
    assert torch.equal(outs[0], outs[1]) and torch.equal(dense[0], dense[1])
    assert outs[0].float().abs().max() > 0
