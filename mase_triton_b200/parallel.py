"""Single-node multi-GPU use of the path: one process per GPU over ``torch.distributed``.

* Quantisation (extract / compose / quantize_dequantize) shards by rows and needs no collective:
  with blocks along the last dim and ``cols % block_size == 0`` no block spans two rows, and the
  scales / elements of a row slice are exactly the matching slice of the full result.
* Linears are column-parallel by output feature: rank r owns rows ``[n0, n1)`` of the weight (a
  contiguous slice of ``w_elements.view(N, K)`` and ``w_scales.view(N, K/32)``), every rank
  quantises the (replicated) activation itself, and the ``[M, N/g]`` partial outputs are gathered
  with one all-gather (NCCL over NVLink on GPUs, gloo in the CPU tests).
* :class:`GatherFusedMXFPLinear` removes that collective for layers whose activation and weight are
  both quantised: the tensor-core GEMM kernel itself copies every finished output tile into the
  full ``[M, N]`` output of every rank (peer memory mapped through PyTorch symmetric memory, plain
  stores over NVLink, issued by extra warps of the same CTAs), so the gather overlaps the GEMM tile
  by tile.

The reference has no distributed code; this module is new functionality named by the benchmark
configurations (row-sharded quantisation, column-parallel linears).
"""

from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist
from torch import Tensor

from .mxfp.meta import MXFPTensorMeta


def shard_bounds(n: int, rank: int, world: int, multiple: int = 1) -> tuple[int, int]:
    """Half-open range of rank ``rank`` when ``n`` items (in units of ``multiple``) are split as evenly as
    possible over ``world`` ranks; earlier ranks take the remainder."""
    assert n % multiple == 0 and 0 <= rank < world
    units = n // multiple
    base, rem = divmod(units, world)
    lo = rank * base + min(rank, rem)
    hi = lo + base + (1 if rank < rem else 0)
    return lo * multiple, hi * multiple


def shard_rows(x: Tensor, rank: int, world: int) -> Tensor:
    """Row slice of ``x`` owned by ``rank`` (a view)."""
    lo, hi = shard_bounds(x.shape[0], rank, world)
    return x[lo:hi]


def shard_quantised_weight(w_scales: Tensor, w_elements: Tensor, w_tensor_meta: MXFPTensorMeta, rank: int, world: int):
    """Output-feature shard of a weight quantised with blocks along ``in_features``.

    Returns ``(scales, elements, tensor_meta, (n0, n1))`` where the tensors are contiguous slices of the
    inputs (no copy) shaped like a freshly quantised ``[n1-n0, K]`` weight."""
    N, K = w_tensor_meta.shape
    B = w_tensor_meta.meta.block_size
    assert w_tensor_meta.block_dim in (1, -1) and K % B == 0
    n0, n1 = shard_bounds(N, rank, world)
    blocks_per_row = K // B
    scales = w_scales.reshape(N * blocks_per_row, 1)[n0 * blocks_per_row:n1 * blocks_per_row]
    elements = w_elements.reshape(N * blocks_per_row, B)[n0 * blocks_per_row:n1 * blocks_per_row]
    meta = w_tensor_meta.create(shape=(n1 - n0, K))
    return scales, elements, meta, (n0, n1)


def gather_columns(y_local: Tensor, sizes: list[int], group=None) -> Tensor:
    """All-gather ``[..., n_r]`` partial outputs into ``[..., sum(n_r)]`` on every rank."""
    world = dist.get_world_size(group)
    assert len(sizes) == world
    lead = y_local.shape[:-1]
    if len(set(sizes)) == 1:
        # equal shards: one collective into a [world, M, n] buffer, then one strided copy
        flat = y_local.reshape(-1, sizes[0]).contiguous()
        buf = torch.empty((world * flat.shape[0], sizes[0]), dtype=flat.dtype, device=flat.device)
        dist.all_gather_into_tensor(buf, flat, group=group)          # rank r's rows land at [r*M, (r+1)*M)
        return buf.view(world, flat.shape[0], sizes[0]).permute(1, 0, 2).reshape(*lead, world * sizes[0])
    # uneven shards: pad every shard to the widest one, gather, drop the padding
    widest = max(sizes)
    flat = y_local.reshape(-1, y_local.shape[-1])
    padded = torch.zeros((flat.shape[0], widest), dtype=flat.dtype, device=flat.device)
    padded[:, : flat.shape[1]] = flat
    buf = torch.empty((world * flat.shape[0], widest), dtype=flat.dtype, device=flat.device)
    dist.all_gather_into_tensor(buf, padded, group=group)
    buf = buf.view(world, flat.shape[0], widest)
    return torch.cat([buf[r, :, :n] for r, n in enumerate(sizes)], dim=-1).reshape(*lead, sum(sizes))


class ColumnParallelLinear:
    """Column-parallel wrapper: ``local_forward(x) -> [..., n_r]`` runs this rank's shard (for example an
    ``MXFPLinearPTQ`` built from :func:`shard_quantised_weight`); ``__call__`` gathers the full output."""

    def __init__(self, local_forward: Callable[[Tensor], Tensor], out_features: int, group=None):
        self.local_forward = local_forward
        self.group = group
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        self.sizes = [hi - lo for lo, hi in (shard_bounds(out_features, r, world) for r in range(world))]
        self.bounds = shard_bounds(out_features, rank, world)

    def __call__(self, x: Tensor, gather: bool = True) -> Tensor:
        y = self.local_forward(x)
        assert y.shape[-1] == self.bounds[1] - self.bounds[0]
        return gather_columns(y, self.sizes, self.group) if gather else y


def column_parallel_mxfp_linear(layer, group=None) -> ColumnParallelLinear:
    """Shard an ``MXFPLinearPTQ`` whose weight is quantised (``Wq``) across the ranks of ``group``."""
    from .mxfp.layers import MXFPLinearPTQ

    world, rank = dist.get_world_size(group), dist.get_rank(group)
    assert layer.w_scales is not None, "column_parallel_mxfp_linear needs a quantised weight"
    s, e, meta, (n0, n1) = shard_quantised_weight(layer.w_scales.data, layer.w_elements.data, layer.w_tensor_meta, rank, world)
    bias = None if layer.bias is None else layer.bias.data[n0:n1]
    local = MXFPLinearPTQ.from_quantized(s.contiguous(), e.contiguous(), meta, bias, None, None, None, layer.x_mxfp_meta,
                                         layer.layer_type, layer.backend)
    return ColumnParallelLinear(local, layer.out_features, group)


class GatherFusedMXFPLinear:
    """Column-parallel ``XqWq`` MXFP linear with the all-gather fused into the GEMM epilogue.

    Every rank holds the packed weight rows ``[n0, n1)`` and two ``[max_rows, N]`` output buffers in
    symmetric memory (mapped into every process of ``group``).  A call quantises the replicated
    activation, runs ``mxq_mx_gemm_gather`` with the addresses of ALL ranks' current buffers as
    destinations, and then joins one tiny all-reduce that serves as the fence "every rank's stores have
    landed".  The two buffers alternate, so a fast rank never overwrites an output a slow rank is
    still reading: the returned tensor (a view of this rank's buffer) is valid until the call after
    the next one.
    """

    def __init__(self, layer, max_rows: int, dtype: torch.dtype = torch.bfloat16, group=None, tile_rows: int | None = None):
        import torch.distributed._symmetric_memory as symm_mem

        from .mxfp import gemm as _gemm

        self.group = group if group is not None else dist.group.WORLD
        world, rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        assert layer.w_scales is not None and layer.x_mxfp_meta is not None, "needs a quantised weight and activation"
        assert _gemm.supported(layer.x_mxfp_meta) and _gemm.supported(layer.w_tensor_meta.meta)
        N, K = layer.w_tensor_meta.shape
        unit = 4 if dtype == torch.float32 else 8
        assert N % unit == 0, "out_features must be a whole number of 16-byte units"
        B = layer.w_tensor_meta.meta.block_size
        self.n0, self.n1 = shard_bounds(N, rank, world, multiple=unit)
        bpr = K // B
        scales = layer.w_scales.data.reshape(N * bpr, 1)[self.n0 * bpr:self.n1 * bpr]
        elements = layer.w_elements.data.reshape(N * bpr, B)[self.n0 * bpr:self.n1 * bpr]
        # tile_rows: columns of the GEMM's CTA tile.  192 makes every forwarded row segment of a 16-bit output a whole
        # number of 128-byte lines, which the stores over NVLink prefer (+12 % egress on four GPUs); it is the default
        # where sending the shard to the peers takes longer than computing it (about (g - 1) * 1600 * bytes per element
        # > in_features), else the width with the least padded work is used.
        if tile_rows is None and (world - 1) * 1600 * (4 if dtype == torch.float32 else 2) > K and (self.n1 - self.n0) >= 192:
            tile_rows = 192
        self.weight = _gemm.pack_operand(scales, elements, self.n1 - self.n0, K, layer.w_tensor_meta.meta, _gemm.OPERAND_B, tile_rows)
        self.bias = None if layer.bias is None else layer.bias.data[self.n0:self.n1].to(dtype).contiguous()
        self.x_meta, self.N, self.K, self.dtype, self.max_rows = layer.x_mxfp_meta, N, K, dtype, max_rows
        dev = layer.w_elements.device
        self.bufs, self.ptrs, self._handles = [], [], []
        for _ in range(2):
            t = symm_mem.empty((max_rows, N), dtype=dtype, device=dev)
            h = symm_mem.rendezvous(t, self.group)
            self.bufs.append(t)
            self._handles.append(h)
            self.ptrs.append([int(p) for p in h.buffer_ptrs])
        self._fence = torch.zeros(1, device=dev)
        self.rank = rank
        self._turn = 0
        self._gemm = _gemm

    def __call__(self, x: Tensor) -> Tensor:
        g = self._gemm
        x2 = x.reshape(-1, self.K)
        M = x2.shape[0]
        assert M <= self.max_rows, "more rows than the output buffers were sized for"
        a = g.pack_activation(x2, self.x_meta)
        if self.n1 > self.n0:
            g.mx_gemm_gather(a, self.weight, self.ptrs[self._turn], self.rank, self.N, self.n0, self.dtype, self.bias)
        dist.all_reduce(self._fence, group=self.group)        # every rank's tiles are in every buffer after this
        out = self.bufs[self._turn][:M].view(*x.shape[:-1], self.N)
        self._turn ^= 1
        return out
