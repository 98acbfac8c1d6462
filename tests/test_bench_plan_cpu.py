"""Host logic of the sharded benchmark step: launch order and which outputs an all-reduce sums.

The step the multi-GPU benchmark times is only valid if every (M, N, K) launch of the sweep
runs exactly once, every row-parallel output is summed exactly once, and an all-reduce is
issued only after the last GEMM that writes into its buffer.  These are properties of
``bench.plan_row_sums`` alone and need no GPU.
"""

from __future__ import annotations

import importlib.util
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
_spec = importlib.util.spec_from_file_location("bench_module", ROOT / "bench.py")
bench = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(bench)

ALL = {(m, n, k) for m in bench.M_VALUES for (n, k) in bench.NK_SHAPES}
ROWS = {(m, n, k) for (m, n, k) in ALL if (n, k) in bench.ROW_PARALLEL}


def test_one_gpu_keeps_the_listed_order_and_sums_nothing():
    groups, order = bench.plan_row_sums("auto", 1)
    assert groups == [] and order == [(m, n, k) for m in bench.M_VALUES for (n, k) in bench.NK_SHAPES]


@pytest.mark.parametrize("mode", ["nccl", "nccl_pair", "nccl_merged", "nccl_early", "peer"])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_every_launch_once_and_every_group_summed_after_its_last_gemm(mode, world):
    groups, order = bench.plan_row_sums(mode, world)
    assert len(order) == len(ALL) and set(order) == ALL            # every launch exactly once
    grouped = [key for group in groups for key in group]
    assert len(grouped) == len(set(grouped)) and set(grouped) <= ROWS   # a row output in one group at most
    position = {key: index for index, key in enumerate(order)}
    for group in groups:
        assert group, "no empty group"
        # the trigger (last key of the group) is the group's last launch in the step
        assert max(position[key] for key in group) == position[group[-1]]
    # large batches first: the first launch is a row-parallel GEMM of the largest batch
    assert order[0][0] == max(bench.M_VALUES) and order[0][1:] in bench.ROW_PARALLEL


def test_group_membership_of_each_mode():
    big = max(bench.M_VALUES)
    rows = [s for s in bench.NK_SHAPES if s in bench.ROW_PARALLEL]
    assert bench.plan_row_sums("nccl", 8)[0] == [] and bench.plan_row_sums("peer", 8)[0] == []
    pairs = bench.plan_row_sums("nccl_pair", 8)[0]
    assert len(pairs) == len(bench.M_VALUES) and all(len(g) == 2 and g[0][0] == g[1][0] for g in pairs)
    merged, order = bench.plan_row_sums("nccl_merged", 8)
    large = {key for key in ROWS if key[0] > 256}
    assert [len(g) for g in merged] == [2, len(large) - 2] and set(merged[0]) == {(big, *s) for s in rows}
    assert set(merged[0]) | set(merged[1]) == large
    # every prefill-sized row-parallel GEMM runs before any other launch
    assert set(order[: len(large)]) == large
    early, order_early = bench.plan_row_sums("nccl_early", 8)
    assert early[0] == [order_early[0]] == [(big, *rows[0])]        # the first sum waits for one GEMM only
    assert set(early[0]) | set(early[1]) == large and order_early == order
