"""Host-side logic of the multi-GPU path with two gloo ranks on CPU: shard bounds, slicing a
quantised weight by output feature, and the gathered layout of a column-parallel linear."""

from __future__ import annotations

import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from mase_triton_b200 import parallel
from mase_triton_b200.mxfp.meta import MXFP8_E4M3_fn, MXFPTensorMeta


def test_shard_bounds_cover_everything():
    for n, world, mult in ((16384, 8, 1), (10, 3, 1), (14336, 8, 1), (7, 8, 1), (4096, 4, 32)):
        spans = [parallel.shard_bounds(n, r, world, mult) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert all((hi - lo) % mult == 0 for lo, hi in spans)
        assert max(hi - lo for lo, hi in spans) - min(hi - lo for lo, hi in spans) <= mult


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, uneven: bool):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)              # same data on every rank
        N, K, M = (96 if not uneven else 97), 64, 5
        w = torch.randn(N, K, generator=g)
        x = torch.randn(2, M, K, generator=g)
        scales, elements = oracle.extract_mxfp_components(w.flatten(), MXFP8_E4M3_fn)
        meta = MXFPTensorMeta(device="cpu", dtype=torch.float32, shape=(N, K), block_dim=1, meta=MXFP8_E4M3_fn)
        w_dq = oracle.compose_mxfp_tensor(scales, elements, MXFP8_E4M3_fn, torch.float32).reshape(N, K)

        s_r, e_r, meta_r, (n0, n1) = parallel.shard_quantised_weight(scales, elements, meta, rank, world)
        # the shard is what quantising the row slice on its own would give (row sharding needs no collective)
        s_own, e_own = oracle.extract_mxfp_components(w[n0:n1].flatten(), MXFP8_E4M3_fn)
        assert torch.equal(s_r, s_own) and torch.equal(e_r, e_own) and meta_r.shape == (n1 - n0, K)
        w_r = oracle.compose_mxfp_tensor(s_r.contiguous(), e_r.contiguous(), MXFP8_E4M3_fn, torch.float32).reshape(n1 - n0, K)

        layer = parallel.ColumnParallelLinear(lambda t: torch.nn.functional.linear(t, w_r), N)
        y = layer(x)
        assert y.shape == (2, M, N)
        assert torch.equal(y, torch.nn.functional.linear(x, w_dq)), "gathered column-parallel output differs from the full linear"
        assert layer(x, gather=False).shape == (2, M, n1 - n0)
        # row-sharded quantisation: each rank's rows, gathered along dim 0, reproduce the full result
        rows = parallel.shard_rows(w, rank, world)
        part = oracle.extract_mxfp_components(rows.flatten(), MXFP8_E4M3_fn)[1]
        if not uneven:
            full = torch.empty((world * part.shape[0], 32), dtype=part.dtype)
            dist.all_gather_into_tensor(full, part)
            assert torch.equal(full.reshape(-1, 32), elements)
    finally:
        dist.destroy_process_group()


def test_column_parallel_two_ranks_even():
    mp.spawn(_worker, args=(2, _free_port(), False), nprocs=2, join=True)


def test_column_parallel_two_ranks_uneven():
    mp.spawn(_worker, args=(2, _free_port(), True), nprocs=2, join=True)
