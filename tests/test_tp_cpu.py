"""CPU (gloo, world_size 2) tests of the tensor-parallel shard arithmetic.

Each rank slices a packed MXFP6 weight column- or row-parallel with
``mxfp6_sm120_b200.tp``, computes its part with the CPU oracle and, for the
row-parallel case, all-reduces the partials; the result must equal the unsharded
oracle GEMM.
"""

from __future__ import annotations

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mxfp6_sm120_b200 import tp
from oracle import mx_oracle as o


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _problem():
    gen = torch.Generator(device="cpu").manual_seed(42)
    m, n, k = 5, 512, 768
    a = torch.randn((m, k), generator=gen).to(torch.bfloat16)
    w = (torch.randn((n, k), generator=gen) * 0.02).to(torch.bfloat16)
    a_q, a_s = o.quantize_mxfp8_torch(a)
    w_q, w_s = o.quantize_mxfp6(w)
    return m, n, k, a_q, a_s, w_q, w_s


def _worker(rank: int, world: int, port: int, results) -> None:
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m, n, k, a_q, a_s, w_q, w_s = _problem()
        values = torch.from_numpy(o.pack_fp6(w_q))
        scales = torch.from_numpy(o.pack_scales(w_s))
        full = o.gemm_w6a8(a_q, a_s, w_q, w_s, out_dtype=None)

        col = tp.shard_column_parallel(values, scales, n, k, world, rank)
        codes = o.unpack_fp6(col.values.numpy(), col.rows, col.k)
        logical = o.unpack_scales(col.scales.numpy(), col.rows, col.k)
        assert np.array_equal(codes, w_q[col.begin : col.end])
        assert np.array_equal(logical, w_s[col.begin : col.end])
        part = o.gemm_w6a8(a_q, a_s, codes, logical, out_dtype=None)
        gathered = [torch.empty_like(part) for _ in range(world)]
        dist.all_gather(gathered, part)
        ok_col = torch.equal(torch.cat(gathered, dim=1), full)

        row = tp.shard_row_parallel(values, scales, n, k, world, rank)
        codes = o.unpack_fp6(row.values.numpy(), row.rows, row.k)
        logical = o.unpack_scales(row.scales.numpy(), row.rows, row.k)
        assert np.array_equal(codes, w_q[:, row.begin : row.end])
        assert np.array_equal(logical, w_s[:, row.begin // 32 : row.end // 32])
        partial = o.gemm_w6a8(a_q[:, row.begin : row.end], a_s[:, row.begin // 32 : row.end // 32],
                              codes, logical, out_dtype=None)
        dist.all_reduce(partial)
        ok_row = torch.allclose(partial, full, rtol=1e-5, atol=1e-5)
        results[rank] = (ok_col, ok_row)
    finally:
        dist.destroy_process_group()


def test_column_and_row_parallel_shards_reproduce_the_full_gemm():
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    assert dict(results) == {0: (True, True), 1: (True, True)}


@pytest.mark.parametrize("total,world", [(34816, 8), (7168, 8), (2048, 8), (17408, 8), (6144, 4), (5120, 3)])
def test_shard_bounds_cover_everything_on_128_granules(total, world):
    edges = [tp.shard_bounds(total, world, r) for r in range(world)]
    assert edges[0][0] == 0 and edges[-1][1] == total
    for (b0, e0), (b1, _) in zip(edges, edges[1:]):
        assert e0 == b1 and b0 % 128 == 0 and e0 % 128 == 0
    sizes = [e - b for b, e in edges]
    assert max(sizes) - min(sizes) <= 128


def test_shard_bounds_reject_unaligned_totals():
    with pytest.raises(ValueError):
        tp.shard_bounds(1000, 2, 0)


def test_scale_repacking_helpers_match_oracle():
    rng = np.random.default_rng(0)
    logical = rng.integers(118, 130, size=(200, 24), dtype=np.uint8)
    packed = tp.pack_scales_any(torch.from_numpy(logical))
    assert np.array_equal(packed.numpy(), o.pack_scales(logical))
    assert np.array_equal(tp.unpack_scales_any(packed, 200, 768).numpy(), logical)
