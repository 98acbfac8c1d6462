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
    n_tiles = (n + 127) // 128
    if m <= 64 and not (m > 32 and 2 * n_tiles > 240):
        # decode batches: the weight-streaming kernel, two CTAs per SM
        assert plan["kernel"] == "stream" and plan["cta_pair"] == 0
        assert tile == (16 if m <= 16 else 32 if m <= 32 else 64)
        assert plan["smem_bytes"] <= (233472 // 2 - 1024) and plan["stages"] >= 3
        if 2 * n_tiles <= 240:
            # too few tiles: clusters split K; a launch fills at most 240 of the 296 CTA slots
            assert 2 <= plan["cluster_k"] <= 8
            assert plan["grid"] == n_tiles * plan["cluster_k"] <= 240
            assert n_tiles * (plan["cluster_k"] + 1) > 240 or plan["cluster_k"] == 8
        else:
            assert plan["cluster_k"] == 1 and plan["grid"] == n_tiles <= 288
    elif m <= 96:
        # 65..96 rows: two 64-row tiles per feature tile while the weights (read twice then)
        # fit the L2, else one 96-row tile; 64 rows of the widest matrix: one 64-row tile
        two_tiles = m > 64 and n * k * 3 // 4 <= 32 << 20
        assert plan["kernel"] == "persistent" and plan["cta_pair"] == 0
        assert tile == (64 if (two_tiles or m <= 64) else 96)
        tiles = n_tiles * -(-m // tile)
        if 2 * tiles <= 148:
            # too few tiles for the GPU: clusters split K, and every cluster fits the GPU
            assert 2 <= plan["cluster_k"] <= 8
            assert plan["grid"] == tiles * plan["cluster_k"] <= 148
        else:
            assert plan["cluster_k"] == 1 and plan["grid"] == min(tiles, 148)
    else:
        # prefill batches run on CTA pairs: 256 weight rows per tile, an even grid
        assert plan["cta_pair"] == 1 and plan["kernel"] == "cta_pair" and tile in (128, 192, 256)
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
        mx.set_stream_kernel_mode(False)
        plan = mx.gemm_w6a8_plan(16, 7168, 5120)
        assert plan["kernel"] == "persistent" and plan["cluster_k"] == 2 and plan["grid"] == 112
    finally:
        mx.set_stream_kernel_mode(True)
    assert mx.gemm_w6a8_plan(16, 7168, 5120)["kernel"] == "stream"
    try:
        mx.set_cta_pair_mode(False)
        assert mx.gemm_w6a8_plan(4096, 7168, 5120)["cta_pair"] == 0
    finally:
        mx.set_cta_pair_mode(True)
    assert mx.gemm_w6a8_plan(4096, 7168, 5120)["cta_pair"] == 1


def test_grid_of_the_streaming_kernel_without_a_split():
    # more tiles than CTA slots: equal shares, every CTA walks the same number of tiles
    plan = mx.gemm_w6a8_plan(8, 128 * 400, 1024)
    assert plan["kernel"] == "stream" and plan["cluster_k"] == 1 and plan["grid"] == 200
    plan = mx.gemm_w6a8_plan(8, 128 * 272, 5120)
    assert plan["grid"] == 272
    # k shorter than the cluster: the split stops at k / 128
    assert mx.gemm_w6a8_plan(8, 1024, 256)["cluster_k"] == 2


def test_explicit_configurations_are_described_and_validated():
    assert mx.w6a8_config_abi() == "b200-w6a8-58-v1"
    configs = mx.w6a8_configs()
    assert len(configs) == 58 and [c["config_id"] for c in configs] == list(range(58))
    assert configs[0] == {"config_id": 0, "kernel": "stream", "tile_tokens": 16, "cluster_k": 1,
                          "splits": 1}
    assert configs[15]["kernel"] == "stream" and configs[15]["tile_tokens"] == 32 and configs[15]["cluster_k"] == 8
    assert configs[16]["kernel"] == "persistent" and configs[31]["tile_tokens"] == 96
    assert {c["tile_tokens"] for c in configs if c["kernel"] == "cta_pair"} == {128, 192, 256}
    assert {c["splits"] for c in configs[38:50]} == {2, 4, 8}
    assert all(c["kernel"] == "stream" and c["tile_tokens"] == 64 for c in configs[50:])
    assert [c["cluster_k"] for c in configs[50:]] == list(range(1, 9))
    from mxfp6_sm120_b200._loader import library

    lib = library()
    out = (__import__("ctypes").c_int * 4)()
    assert lib.mxfp6_w6a8_config_describe(58, out) == 1          # out of range
    assert lib.mxfp6_w6a8_config_describe(-1, out) == 1


def test_decode_layer_schedule_choice_is_host_arithmetic():
    """Which decode schedule a routed-MoE batch takes is decided on the host from the two grids
    (148 SMs assumed): two launches need at most 16 blocks of 128 hidden values per W1 CTA and
    are taken wherever they fit."""
    named = dict(topk=8, experts=256, hidden_size=2048, intermediate=512)
    for tokens in (1, 2, 3, 4, 8, 16, 32, 64):
        assert mx.moe_decode_layer_supported(tokens, **named)
    assert all(mx.moe_decode_layer_preferred(t, **named) for t in (1, 2, 3, 4, 8, 32))
    # hidden 5120: 40 K blocks, so only launches that split K over a cluster fit the 16 slots
    assert mx.moe_decode_layer_supported(1, 8, 256, 5120, 512)
    assert not mx.moe_decode_layer_supported(8, 8, 256, 5120, 512)
    assert not mx.moe_decode_layer_preferred(8, 8, 256, 5120, 512)
    # more than nine routes per token, or a down projection wider than 2048 inputs
    assert not mx.moe_decode_layer_supported(1, 9, 256, 2048, 512)
    assert not mx.moe_decode_layer_supported(1, 8, 256, 2048, 4096)
    assert not mx.moe_decode_layer_supported(1, 8, 4, 2048, 512)      # fewer experts than top-k
