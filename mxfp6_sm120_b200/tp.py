"""Tensor-parallel sharding of dense W6A8 projections across the GPUs of one node.

Column-parallel = split the output features N (rows of the packed weight and of
its scale atoms) at multiples of 128: no collective, every rank owns a slice of
the output.  Row-parallel = split K at multiples of 128: every rank produces a
full ``[M, N]`` partial and the partials are summed with an NCCL all-reduce on
the compute stream.  The reference ships TP only as pre-sharded shapes
(benchmarks/model_shapes.py:9-15) and leaves the all-reduce to the serving
runtime; here both shardings are first-class.

The shard arithmetic is pure byte slicing and runs on any device, so it is
covered by CPU (gloo) tests.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

SCALE_VECTOR_SIZE = 32
# Up to this many output rows a row-parallel sum runs as one peer-memory kernel (latency
# bound); larger outputs are bandwidth-bound collectives and go through NCCL.
PEER_ALLREDUCE_MAX_ROWS = 256


def _packed_scale_offset(row: torch.Tensor, group: torch.Tensor, groups: int) -> torch.Tensor:
    atoms_per_rb = (groups + 3) // 4
    atom = (row // 128) * atoms_per_rb + group // 4
    r = row % 128
    return atom * 512 + (r % 32) * 16 + (r // 32) * 4 + group % 4


def unpack_scales_any(packed: torch.Tensor, rows: int, k: int) -> torch.Tensor:
    """Packed scale bytes -> logical ``[rows, k/32]`` with plain indexing (any device)."""
    groups = k // SCALE_VECTOR_SIZE
    r = torch.arange(rows, device=packed.device).view(-1, 1).expand(rows, groups)
    g = torch.arange(groups, device=packed.device).view(1, -1).expand(rows, groups)
    return packed[_packed_scale_offset(r, g, groups)]


def pack_scales_any(logical: torch.Tensor) -> torch.Tensor:
    """Logical ``[rows, k/32]`` -> packed bytes (padding 0x7f) with plain indexing."""
    rows, groups = logical.shape
    size = (rows + 127) // 128 * 128 * ((groups + 3) // 4 * 4)
    out = torch.full((size,), 0x7F, dtype=torch.uint8, device=logical.device)
    r = torch.arange(rows, device=logical.device).view(-1, 1).expand(rows, groups)
    g = torch.arange(groups, device=logical.device).view(1, -1).expand(rows, groups)
    out[_packed_scale_offset(r, g, groups)] = logical
    return out


def shard_bounds(total: int, world: int, rank: int, granule: int = 128) -> tuple[int, int]:
    """Contiguous ``[begin, end)`` of ``total`` for ``rank``, in units of ``granule``.

    Granules are dealt as evenly as possible; the first ``extra`` ranks get one more.
    """
    if total % granule:
        raise ValueError(f"{total} is not a multiple of the {granule}-element shard granule")
    units = total // granule
    base, extra = divmod(units, world)
    begin = rank * base + min(rank, extra)
    end = begin + base + (1 if rank < extra else 0)
    return begin * granule, end * granule


@dataclass(frozen=True)
class WeightShard:
    """One rank's slice of a packed MXFP6 weight (values, packed scales, rows, k)."""

    values: torch.Tensor
    scales: torch.Tensor
    rows: int
    k: int
    begin: int
    end: int


def shard_column_parallel(values: torch.Tensor, scales: torch.Tensor, n: int, k: int, world: int,
                          rank: int) -> WeightShard:
    """Rows ``[begin, end)`` of the weight: contiguous bytes of both buffers."""
    begin, end = shard_bounds(n, world, rank, 128)
    row_bytes = k * 3 // 4
    atom_row_bytes = ((k // SCALE_VECTOR_SIZE + 3) // 4) * 512  # bytes per 128-row block
    v = values.view(-1)[begin * row_bytes : end * row_bytes]
    s = scales.view(-1)[begin // 128 * atom_row_bytes : end // 128 * atom_row_bytes]
    return WeightShard(v.contiguous(), s.contiguous(), end - begin, k, begin, end)


def shard_row_parallel(values: torch.Tensor, scales: torch.Tensor, n: int, k: int, world: int,
                       rank: int) -> WeightShard:
    """K columns ``[begin, end)`` of every weight row, repacked to a dense shard."""
    begin, end = shard_bounds(k, world, rank, 128)
    row_bytes = k * 3 // 4
    v = values.view(n, row_bytes)[:, begin * 3 // 4 : end * 3 // 4].contiguous().view(-1)
    logical = unpack_scales_any(scales.view(-1), n, k)[:, begin // 32 : end // 32].contiguous()
    return WeightShard(v, pack_scales_any(logical), n, end - begin, begin, end)


class ColumnParallelLinear:
    """``out_local[M, N/world] = gemm(a, W[begin:end])``; no collective."""

    def __init__(self, ops, shard: WeightShard):
        self.ops = ops
        self.shard = shard
        self.weight = ops.PackedMXFP6Tensor(shard.values, shard.scales, shard.rows, shard.k)

    def __call__(self, a: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16,
                 out: torch.Tensor | None = None) -> torch.Tensor:
        return self.ops.gemm_from_float(a, self.weight, out_dtype=out_dtype, out=out)


class RowParallelLinear:
    """``out[M, N] = all_reduce_sum(gemm(a[:, begin:end], W[:, begin:end]))``."""

    def __init__(self, ops, shard: WeightShard, group=None, peer=None):
        self.ops = ops
        self.shard = shard
        self.group = group
        self.peer = peer
        self.weight = ops.PackedMXFP6Tensor(shard.values, shard.scales, shard.rows, shard.k)

    def __call__(self, a_local: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16,
                 out: torch.Tensor | None = None) -> torch.Tensor:
        rows = int(a_local.shape[0])
        if (self.peer is not None and self.peer.world > 1 and out_dtype == torch.bfloat16
                and rows <= PEER_ALLREDUCE_MAX_ROWS):
            # Decode-sized outputs: the GEMM writes into this rank's symmetric block and one
            # kernel sums all ranks' partials over peer memory (tp_fused.SymmetricBlocks).
            partial = self.peer.next_partial(rows, self.shard.rows)
            self.ops.gemm_from_float(a_local, self.weight, out_dtype=out_dtype, out=partial)
            if out is None:
                out = torch.empty((rows, self.shard.rows), dtype=out_dtype, device=a_local.device)
            return self.peer.allreduce(out)
        partial = self.ops.gemm_from_float(a_local, self.weight, out_dtype=out_dtype, out=out)
        if dist.is_initialized() and dist.get_world_size(self.group) > 1:
            dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=self.group)
        return partial
