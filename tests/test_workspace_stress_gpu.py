"""Ten thousand randomised launches on the frozen split-K arena, then two streams at once.

The reference's stress of its persistent workspace (tests/stress_persistent_workspace.py:
16-184): one 128 x 8704 weight, batch sizes at the tile boundaries, every problem run
through the dispatcher (``torch.ops.mxfp6.gemm_w6a8`` with a per-shape configuration pinned
by ``set_w6a8_config``, and the W6A6 form ``torch.ops.mxfp6.gemm`` as the control), planning,
freezing, 10 000 launches in random order that must reproduce the first results bit for bit,
two lanes in flight on two streams, all split-K counters back at zero and no launch that fell
back to a transient allocation.
"""

from __future__ import annotations

import random

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = torch.device("cuda", 0)
BOUNDARY_M = (1, 8, 9, 16, 17, 128)
ITERATIONS = 10_000
CONCURRENT_ITERATIONS = 1_000


def test_frozen_arena_survives_ten_thousand_random_launches(mx):
    from mxfp6_sm120_b200._loader import check, library

    n, k = 128, 8704
    gen = torch.Generator(device=DEV).manual_seed(1234)
    b_codes = torch.randint(0, 64, (n, k), generator=gen, device=DEV, dtype=torch.uint8)
    weight = mx.pack_operand(b_codes, torch.full((n, k // 32), 0x7F, device=DEV, dtype=torch.uint8))
    check(library().mxfp6_workspace_reset())
    mx.set_split_k_mode("workspace")     # K is split through arena scratch, as the reference's Stream-K is
    pinned = []
    try:
        problems = {}
        for index, m in enumerate(BOUNDARY_M):
            a_codes = torch.randint(0, 64, (m, k), generator=gen, device=DEV, dtype=torch.uint8)
            a6 = mx.pack_operand(a_codes, torch.full((m, k // 32), 0x7F, device=DEV, dtype=torch.uint8))
            a8 = torch.ops.mxfp6.expand_fp6_to_fp8(a6.values, m, k)
            out_dtype = torch.float16 if index % 2 == 0 else torch.bfloat16
            if m <= 32:
                # a pinned scratch split: 16- or 32-row tiles, K cut four ways
                config_id = 39 if m <= 16 else 42
                assert torch.ops.mxfp6.set_w6a8_config(a8, m, n, k, config_id, (1, 2, 4, 8)[index % 4],
                                                       index % 3, out_dtype)
                pinned.append((a8, m, out_dtype))
                if out_dtype == torch.bfloat16:   # the plan query reports the BF16 entry of the registry
                    assert mx.gemm_w6a8_plan(m, n, k)["splits"] == 4

            def run_w6a8(a8=a8, a6=a6, m=m, out_dtype=out_dtype):
                return torch.ops.mxfp6.gemm_w6a8(a8, weight.values, a6.scales, weight.scales, m, n, k, 1.0,
                                                 out_dtype)

            def run_w6a6(a6=a6, m=m, out_dtype=out_dtype):
                return torch.ops.mxfp6.gemm(a6.values, weight.values, a6.scales, weight.scales, m, n, k, 1.0,
                                            out_dtype)

            problems[(m, "w6a8")] = run_w6a8
            problems[(m, "w6a6")] = run_w6a6

        references = {key: run() for key, run in problems.items()}
        torch.cuda.synchronize()
        for m in BOUNDARY_M:   # both forms compute the same products exactly
            assert torch.equal(references[(m, "w6a8")], references[(m, "w6a6")])

        mx.begin_workspace_planning()
        for run in problems.values():
            run()
        torch.cuda.synchronize()
        planning = mx.workspace_stats()
        assert planning["layouts"] > 0 and planning["arena_bytes"] > 0, planning
        mx.finalize_workspace_planning()

        keys = list(problems)
        randomizer = random.Random(1234)
        latest = {}
        for _ in range(ITERATIONS):
            key = randomizer.choice(keys)
            latest[key] = problems[key]()
        torch.cuda.synchronize()
        for key, output in latest.items():
            assert torch.equal(output, references[key]), key

        stream_a, stream_b = torch.cuda.Stream(), torch.cuda.Stream()
        key_a, key_b = (1, "w6a8"), (17, "w6a8")
        with torch.cuda.stream(stream_a):
            out_a = problems[key_a]()      # the first eager launch on a stream takes a lane for it
        with torch.cuda.stream(stream_b):
            out_b = problems[key_b]()
        stream_a.synchronize()
        stream_b.synchronize()
        for _ in range(CONCURRENT_ITERATIONS):
            with torch.cuda.stream(stream_a):
                out_a = problems[key_a]()
            with torch.cuda.stream(stream_b):
                out_b = problems[key_b]()
        stream_a.synchronize()
        stream_b.synchronize()
        assert torch.equal(out_a, references[key_a]) and torch.equal(out_b, references[key_b])

        assert mx.workspace_barriers_zero()
        stats = mx.workspace_stats()
        assert stats["fallback_launches"] == 0, stats
        assert stats["persistent_launches"] >= ITERATIONS // 2
        assert stats["lanes"] >= 3
        assert mx.device_status() == 0
    finally:
        for a8, m, out_dtype in pinned:
            torch.ops.mxfp6.set_w6a8_config(a8, m, n, k, -1, 1, 0, out_dtype)
        mx.set_split_k_mode("cluster")
        torch.cuda.synchronize()
        check(library().mxfp6_workspace_reset())
