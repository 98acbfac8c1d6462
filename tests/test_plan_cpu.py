"""The GEMM planner is host arithmetic behind the C ABI: tile, split-K form, grid and kernel
family for every shape of the named dense sweep, checked without a GPU (148 SMs assumed)."""

import pytest

import mxfp6_sm120_b200 as mx

NK = [(7168, 5120), (5120, 6144), (34816, 5120), (5120, 17408), (2048, 5120)]
M_VALUES = [1, 2, 4, 8, 16, 24, 32, 64, 96, 512, 1024, 2048, 4096, 8192]


@pytest.mark.parametrize("n,k", NK)
@pytest.mark.parametrize("m", M_VALUES)
def test_named_sweep_plans(m, n, k):
    plan = mx.gemm_w6a8_plan(m, n, k)
    tile = plan["tile_tokens"]
    assert tile >= min(m, 16) and tile in (16, 32, 64, 96, 128, 192, 256)
    assert plan["splits"] == 1 and plan["partial_bytes"] == 0      # cluster split-K needs no scratch
    if m <= 96:
        # one row tile of exactly the batch's width class, weights streamed once
        assert plan["cta_pair"] == 0 and tile >= m
        n_tiles = (n + 127) // 128
        if 2 * n_tiles <= 148:
            # too few tiles for the GPU: clusters split K, and every cluster fits the GPU
            assert 2 <= plan["cluster_k"] <= 8
            assert plan["grid"] == n_tiles * plan["cluster_k"] <= 148
        else:
            assert plan["cluster_k"] == 1 and plan["grid"] == min(n_tiles, 148)
    else:
        # prefill batches run on CTA pairs: 256 weight rows per tile, an even grid
        assert plan["cta_pair"] == 1 and tile in (128, 192, 256)
        assert plan["cluster_k"] == 1 and plan["grid"] % 2 == 0 and plan["grid"] <= 148
        pair_tiles = -(-m // tile) * -(-n // 256)
        assert plan["grid"] == 2 * min(pair_tiles, 74)


def test_explicit_choices_and_limits():
    assert mx.gemm_w6a8_plan(64, 1024, 2048, 64, 2)["splits"] == 2          # scratch split-K on request
    assert mx.gemm_w6a8_plan(64, 1024, 2048, 64, 2)["partial_bytes"] > 0
    assert mx.gemm_w6a8_plan(300, 1024, 2048, 64)["cta_pair"] == 0           # tile the pair kernel lacks
    assert mx.gemm_w6a8_plan(300, 1024, 2048, 128)["cta_pair"] == 1
    assert mx.gemm_w6a8_plan(300, 1000, 1024)["cta_pair"] == 0               # n % 128 != 0
    assert mx.gemm_w6a8_plan(300, 896, 1024)["cta_pair"] == 1                # last pair half empty
    with pytest.raises(ValueError):
        mx.gemm_w6a8_plan(0, 1024, 2048)
    with pytest.raises((ValueError, RuntimeError)):
        mx.gemm_w6a8_plan(16, 1024, 2000)                                     # k % 128 != 0
    with pytest.raises((ValueError, RuntimeError)):
        mx.gemm_w6a8_plan(64, 1024, 2048, 16)                                 # tile narrower than m


def test_split_k_mode_switch_changes_the_plan():
    try:
        mx.set_split_k_mode("workspace")
        plan = mx.gemm_w6a8_plan(16, 2048, 5120)
        assert plan["cluster_k"] == 1 and plan["splits"] > 1 and plan["partial_bytes"] > 0
        assert mx.is_stream_k_enabled()
        mx.set_split_k_mode("off")
        plan = mx.gemm_w6a8_plan(16, 2048, 5120)
        assert plan["cluster_k"] == 1 and plan["splits"] == 1
    finally:
        mx.set_split_k_mode("cluster")
    assert mx.gemm_w6a8_plan(16, 2048, 5120)["cluster_k"] == 8
    try:
        mx.set_cta_pair_mode(False)
        assert mx.gemm_w6a8_plan(4096, 7168, 5120)["cta_pair"] == 0
    finally:
        mx.set_cta_pair_mode(True)
    assert mx.gemm_w6a8_plan(4096, 7168, 5120)["cta_pair"] == 1
