"""The allocation-free GEMM entry point against the ordinary one.

Some users of this library are not allowed to allocate device memory when they
call it: their call sits inside another framework's CUDA-graph capture, or the
process froze its memory pool at start-up, or they are a plugin that must leave
the host's allocator alone.  ``mxfp6_gemm_w6a8_static_scratch`` serves them with
split-K scratch that lives in a fixed array inside the library.  This file is
collected last on purpose, so a failure here cannot hide the other GPU tests.
"""

from __future__ import annotations

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _operands(mx, m, n, k, seed):
    gen = torch.Generator(device="cpu").manual_seed(seed)
    a = torch.randn((m, k), generator=gen).to(torch.bfloat16).to(DEV)
    w = (torch.randn((n, k), generator=gen) * 0.02).to(torch.bfloat16).to(DEV)
    return mx.quantize_mxfp8(a), mx.quantize_mxfp6(w)


def _call(lib, name, act, wgt, out, extra=()):
    stream = torch.cuda.current_stream().cuda_stream
    return getattr(lib, name)(
        act.values.data_ptr(), act.scales.data_ptr(), wgt.values.data_ptr(), wgt.scales.data_ptr(),
        act.rows, wgt.rows, act.k, ctypes.c_float(1.0), out.data_ptr(), 1, *extra, stream)


def test_static_scratch_gemm_matches_regular_entry_point(mx):
    from mxfp6_sm120_b200._loader import library

    lib = library()
    # 2048 x 5120 at M = 8 splits K nine ways, so the scratch array is really used.
    act, wgt = _operands(mx, 8, 2048, 5120, seed=5)
    mx.set_split_k_mode("workspace")  # the entry point under test always splits through scratch
    try:
        plan = mx.gemm_w6a8_plan(8, 2048, 5120)
        assert plan["splits"] > 1
        scratch = torch.zeros(plan["partial_bytes"] + plan["counter_bytes"], dtype=torch.uint8, device=DEV)
        want = torch.empty((8, 2048), dtype=torch.bfloat16, device=DEV)
        assert _call(lib, "mxfp6_gemm_w6a8_ex", act, wgt, want,
                     (0, 0, scratch.data_ptr(), scratch.numel())) == 0
    finally:
        mx.set_split_k_mode("cluster")
    for _ in range(2):  # two calls in a row share the array; the second must not see stale counters
        got = torch.full((8, 2048), float("nan"), dtype=torch.bfloat16, device=DEV)
        assert _call(lib, "mxfp6_gemm_w6a8_static_scratch", act, wgt, got) == 0
        torch.cuda.synchronize()
        assert torch.equal(got, want)  # same kernel, same plan: bit-identical
    # a problem with enough tiles takes the same entry point without any split or scratch
    mx.set_split_k_mode("workspace")
    try:
        plan2 = mx.gemm_w6a8_plan(40, 16384, 1024)
        assert plan2["splits"] == 1 and plan2["partial_bytes"] == 0
        act2, wgt2 = _operands(mx, 40, 16384, 1024, seed=6)
        want2 = torch.empty((40, 16384), dtype=torch.bfloat16, device=DEV)
        assert _call(lib, "mxfp6_gemm_w6a8_ex", act2, wgt2, want2, (0, 0, None, 0)) == 0
    finally:
        mx.set_split_k_mode("cluster")
    got2 = torch.empty_like(want2)
    assert _call(lib, "mxfp6_gemm_w6a8_static_scratch", act2, wgt2, got2) == 0
    torch.cuda.synchronize()
    assert torch.equal(got2, want2)
    # the headline property: a warmed-up call leaves the device's free memory as it found it
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        assert _call(lib, "mxfp6_gemm_w6a8_static_scratch", act, wgt, got) == 0
        assert _call(lib, "mxfp6_gemm_w6a8_static_scratch", act2, wgt2, got2) == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    assert torch.equal(got, want) and torch.equal(got2, want2)
    # and it captures: both shape classes have run eagerly above, so nothing is set up lazily
    side = torch.cuda.Stream()
    got.fill_(float("nan"))
    got2.fill_(float("nan"))
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            stream = torch.cuda.current_stream().cuda_stream
            assert getattr(lib, "mxfp6_gemm_w6a8_static_scratch")(
                act.values.data_ptr(), act.scales.data_ptr(), wgt.values.data_ptr(), wgt.scales.data_ptr(),
                act.rows, wgt.rows, act.k, ctypes.c_float(1.0), got.data_ptr(), 1, stream) == 0
            assert getattr(lib, "mxfp6_gemm_w6a8_static_scratch")(
                act2.values.data_ptr(), act2.scales.data_ptr(), wgt2.values.data_ptr(), wgt2.scales.data_ptr(),
                act2.rows, wgt2.rows, act2.k, ctypes.c_float(1.0), got2.data_ptr(), 1, stream) == 0
        for _ in range(5):
            graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(got, want) and torch.equal(got2, want2)
    assert mx.device_status() == 0


def test_static_scratch_rejects_oversized_problems(mx):
    from mxfp6_sm120_b200._loader import library

    lib = library()
    mx.set_split_k_mode("workspace")
    try:
        plan = mx.gemm_w6a8_plan(96, 5120, 17408)
    finally:
        mx.set_split_k_mode("cluster")
    assert plan["partial_bytes"] > 4 << 20  # needs more than the 4 MiB built in
    act, wgt = _operands(mx, 96, 5120, 17408, seed=7)
    out = torch.empty((96, 5120), dtype=torch.bfloat16, device=DEV)
    assert _call(lib, "mxfp6_gemm_w6a8_static_scratch", act, wgt, out) == 1
    message = lib.mxfp6_b200_last_error().decode()
    assert "built-in array" in message and str(plan["partial_bytes"]) in message
