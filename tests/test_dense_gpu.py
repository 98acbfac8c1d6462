"""GPU parity tests of the dense path: layout tools, quantizers, W6A8 GEMM, arena.

Everything is called through the C ABI (via the ctypes-backed package) and
compared with the CPU oracle on CPU-seeded inputs.  Bit-exact for bytes;
rel-Frobenius <= 1e-3 against the oracle's output in the same dtype for the GEMM.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import mx_oracle as o

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
GEMM_REL_FRO = 1.0e-3  # tolerance named by the hot-path contract


def _cpu_gen(seed):
    return torch.Generator(device="cpu").manual_seed(seed)


def _rel_fro(got: torch.Tensor, want: torch.Tensor) -> float:
    got, want = got.float().cpu(), want.float().cpu()
    return float((got - want).norm() / want.norm().clamp_min(1e-30))


def _packed_operands(mx, a_bf16, w_bf16):
    a_q, a_s = o.quantize_mxfp8_torch(a_bf16)
    w_q, w_s = o.quantize_mxfp6(w_bf16)
    m, k = a_q.shape
    n = w_q.shape[0]
    act = mx.MXFP8Tensor(
        torch.from_numpy(a_q).reshape(-1).to(DEV), torch.from_numpy(o.pack_scales(a_s)).to(DEV), m, k
    )
    wgt = mx.PackedMXFP6Tensor(
        torch.from_numpy(o.pack_fp6(w_q)).to(DEV), torch.from_numpy(o.pack_scales(w_s)).to(DEV), n, k
    )
    return act, wgt, (a_q, a_s, w_q, w_s)


@pytest.fixture(scope="module", autouse=True)
def _status_clean(mx):
    yield
    assert mx.device_status() == 0, "a bounded device wait expired during the tests"


@pytest.mark.parametrize("rows,k", [(1, 128), (16, 128), (32, 256), (129, 128), (2048, 128)])
def test_fp6_pack_unpack_pad_expand(mx, rows, k):
    gen = _cpu_gen(rows + k)
    codes = torch.randint(0, 256, (rows, k), generator=gen, dtype=torch.uint8)
    packed = mx.pack_fp6(codes.to(DEV))
    want = o.pack_fp6(codes.numpy())
    assert np.array_equal(packed.cpu().numpy(), want)
    assert np.array_equal(mx.unpack_fp6(packed, rows, k).cpu().numpy(), codes.numpy() & 0x3F)
    assert np.array_equal(mx.pad_fp6(packed).cpu().numpy(), o.pad_fp6(want))
    expanded = mx.expand_fp6_to_fp8(packed, rows, k)
    assert torch.equal(expanded.float().cpu(), o.decode_e3m2(torch.from_numpy(codes.numpy() & 0x3F)))


def test_pack_fp6_unaligned_tail(mx):
    codes = torch.arange(0, 36, dtype=torch.uint8)  # 36 codes: two vectors + one scalar quad
    assert np.array_equal(mx.pack_fp6(codes.to(DEV)).cpu().numpy(), o.pack_fp6(codes.numpy()))


@pytest.mark.parametrize("rows,k", [(1, 64), (1, 128), (16, 128), (32, 256), (128, 128), (129, 256), (2048, 128)])
def test_scale_layout_tools(mx, rows, k):
    gen = _cpu_gen(rows * 7 + k)
    logical = torch.randint(120, 135, (rows, k // 32), generator=gen, dtype=torch.uint8)
    packed = mx.pack_scales(logical.to(DEV))
    assert np.array_equal(packed.cpu().numpy(), o.pack_scales(logical.numpy()))
    assert torch.equal(mx.unpack_scales(packed, rows, k).cpu(), logical)


def test_grouped_scale_packing(mx):
    counts = (1, 0, 3, 129, 2)
    offsets = torch.tensor((0, *np.cumsum(counts).tolist()), dtype=torch.int64)
    logical = torch.randint(120, 135, (sum(counts), 4), generator=_cpu_gen(5), dtype=torch.uint8)
    packed, soff = mx.pack_grouped_scales(logical.to(DEV), offsets.to(DEV))
    assert soff.cpu().tolist() == [0, 128, 128, 256, 512, 640]
    want, _ = o.pack_grouped_scales(logical.numpy(), offsets.numpy())
    assert np.array_equal(packed.cpu().numpy()[: want.size], want)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,k", [(1, 128), (7, 256), (129, 128), (33, 160)])
def test_quantizers_bit_exact_small(mx, dtype, rows, k):
    x = (torch.randn((rows, k), generator=_cpu_gen(rows + k)) * 6.0).to(dtype)
    x[0, :32] = 0
    x[0, 33] = -0.0
    codes, scales = o.quantize_mxfp8(x)
    q = mx.quantize_mxfp8(x.to(DEV))
    assert np.array_equal(q.values.cpu().numpy().reshape(rows, k), codes)
    assert np.array_equal(q.scales.cpu().numpy(), o.pack_scales(scales))
    v, logical = mx.quantize_mxfp8_logical(x.to(DEV))
    assert np.array_equal(v.view(torch.uint8).cpu().numpy(), codes)
    assert np.array_equal(logical.cpu().numpy(), scales)
    v2, l2, p2 = mx.quantize_mxfp8_dual(x.to(DEV))
    assert np.array_equal(l2.cpu().numpy(), scales) and np.array_equal(p2.cpu().numpy(), o.pack_scales(scales))
    c6, s6 = o.quantize_mxfp6((x * 0.02).to(dtype))
    w = mx.quantize_mxfp6((x * 0.02).to(dtype).to(DEV))
    assert np.array_equal(w.values.cpu().numpy(), o.pack_fp6(c6))
    assert np.array_equal(w.scales.cpu().numpy(), o.pack_scales(s6))


@pytest.mark.parametrize("m", [1, 8, 32, 512, 4096, 8192])
def test_activation_quantizer_named_config(mx, m):
    """BF16 [M, 5120], N(0,1) with 0.1% entries scaled x50, seed 100+M; bit-exact."""
    gen = _cpu_gen(100 + m)
    x = torch.randn((m, 5120), generator=gen)
    mask = torch.rand((m, 5120), generator=gen) < 0.001
    x = torch.where(mask, x * 50.0, x).to(torch.bfloat16)
    codes, scales = o.quantize_mxfp8_torch(x)
    q = mx.quantize_mxfp8(x.to(DEV))
    assert np.array_equal(q.values.cpu().numpy().reshape(m, 5120), codes)
    assert np.array_equal(q.scales.cpu().numpy(), o.pack_scales(scales))


def test_all_e3m2_codes_round_trip_on_device(mx):
    values = o.decode_e3m2(torch.arange(64, dtype=torch.uint8)).repeat(4, 2).to(torch.bfloat16)
    w = mx.quantize_mxfp6(values.to(DEV))
    codes, scales = mx.unpack_operand(w)
    assert bool((scales == 0x7F).all())
    assert torch.equal(o.decode_e3m2(codes.cpu()), values.float())


def test_correctness_gemm_against_golden(mx, golden_dir):
    """M=16, N=1024, K=2048, seed 0; output compared with the committed fixture."""
    ref = np.load(golden_dir / "reference_helpers.npz")
    gen = _cpu_gen(0)
    a = torch.randn((16, 2048), generator=gen).to(torch.bfloat16)
    w = (torch.randn((1024, 2048), generator=gen) * 0.02).to(torch.bfloat16)
    wq = mx.quantize_mxfp6(w.to(DEV))
    out = mx.gemm(a.to(DEV), wq, out_dtype=torch.bfloat16)
    want = torch.from_numpy(ref["c1_out_bf16_bits"]).view(torch.bfloat16)
    assert _rel_fro(out, want) <= GEMM_REL_FRO
    # FP32-level agreement before the BF16 cast: one BF16 ulp at most.
    want32 = torch.from_numpy(ref["c1_out_f32"])
    assert float((out.float().cpu() - want32).abs().max()) <= float(want32.abs().max()) * 2.0**-8
    aq = mx.quantize_mxfp8(a.to(DEV))
    assert np.array_equal(aq.values.cpu().numpy().reshape(16, 2048), ref["c1_a_codes_by_reference_formula"])
    assert torch.equal(mx.gemm(aq, wq, out_dtype=torch.bfloat16), out)


GEMM_CASES = [
    # m, n, k, tile_tokens, splits (0 = library's choice)
    (1, 1024, 2048, 0, 0),
    (16, 128, 128, 16, 1),
    (16, 1024, 2176, 16, 1),
    (16, 1024, 2048, 16, 4),
    (24, 1024, 1920, 32, 2),
    (32, 1024, 2048, 32, 1),
    (64, 1024, 2048, 64, 2),
    (96, 1024, 2176, 96, 1),
    (128, 1024, 2048, 128, 1),
    (200, 1024, 2048, 128, 1),
    (300, 1000, 1024, 64, 2),
    (400, 1024, 2048, 192, 1),
    (512, 2048, 2048, 256, 1),
    (1000, 1000, 1024, 0, 0),
    (33, 2048, 5120, 0, 0),
]


@pytest.mark.parametrize("m,n,k,tile,splits", GEMM_CASES)
def test_gemm_matches_oracle(mx, m, n, k, tile, splits):
    gen = _cpu_gen(m * 131 + n + k)
    a = torch.randn((m, k), generator=gen).to(torch.bfloat16)
    w = (torch.randn((n, k), generator=gen) * 0.02).to(torch.bfloat16)
    act, wgt, (a_q, a_s, w_q, w_s) = _packed_operands(mx, a, w)
    for dtype in (torch.bfloat16, torch.float16):
        want = o.gemm_w6a8(a_q, a_s, w_q, w_s, out_dtype=dtype)
        got = mx.gemm_w6a8_config(act, wgt, out_dtype=dtype, tile_tokens=tile, splits=splits)
        assert _rel_fro(got, want) <= GEMM_REL_FRO
    # alpha scales the FP32 accumulator before the cast
    want = o.gemm_w6a8(a_q, a_s, w_q, w_s, alpha=0.5, out_dtype=torch.bfloat16)
    got = mx.gemm_w6a8(act, wgt, 0.5, out_dtype=torch.bfloat16)
    assert _rel_fro(got, want) <= GEMM_REL_FRO


def test_gemm_from_float_equals_quantize_then_gemm(mx):
    gen = _cpu_gen(77)
    a = torch.randn((48, 1024), generator=gen).to(torch.bfloat16).to(DEV)
    w = mx.quantize_mxfp6((torch.randn((512, 1024), generator=gen) * 0.02).to(torch.bfloat16).to(DEV))
    fused = mx.gemm_from_float(a, w, out_dtype=torch.float16)
    staged = mx.gemm_w6a8(mx.quantize_mxfp8(a), w, out_dtype=torch.float16)
    assert torch.equal(fused, staged)


def test_w6a6_compatibility_path(mx, golden_dir):
    ref = np.load(golden_dir / "reference_helpers.npz")
    a_codes = np.tile(ref["w6a6_a_codes"], (1, 1))
    # K must be a multiple of 128 for the GEMM: the fixture has K = 256.
    out = mx.gemm_from_codes(
        torch.from_numpy(a_codes).to(DEV),
        torch.from_numpy(ref["w6a6_b_codes"]).to(DEV),
        torch.from_numpy(ref["w6a6_sfa"]).to(DEV),
        torch.from_numpy(ref["w6a6_sfb"]).to(DEV),
        out_dtype=torch.float16,
    )
    want = torch.from_numpy(ref["w6a6_out_f16_bits"]).view(torch.float16)
    # The fixture's random scales overflow FP16 in places: infinities must coincide.
    finite = torch.isfinite(want)
    assert torch.equal(torch.isfinite(out.cpu()), finite)
    assert torch.equal(out.cpu()[~finite], want[~finite])
    assert _rel_fro(out.cpu()[finite], want[finite]) <= GEMM_REL_FRO


def test_split_k_is_deterministic_and_config_independent(mx):
    gen = _cpu_gen(9)
    a = torch.randn((8, 5120), generator=gen).to(torch.bfloat16)
    w = (torch.randn((2048, 5120), generator=gen) * 0.02).to(torch.bfloat16)
    act, wgt, _ = _packed_operands(mx, a, w)
    first = mx.gemm_w6a8_config(act, wgt, out_dtype=torch.bfloat16, tile_tokens=16, splits=9)
    for _ in range(5):
        again = mx.gemm_w6a8_config(act, wgt, out_dtype=torch.bfloat16, tile_tokens=16, splits=9)
        assert torch.equal(first, again)
    single = mx.gemm_w6a8_config(act, wgt, out_dtype=torch.bfloat16, tile_tokens=16, splits=1)
    assert _rel_fro(first, single) <= GEMM_REL_FRO


def test_full_size_gemm_properties(mx):
    """Largest sweep shape (M=8192, N=34816, K=5120): sampled rows/columns against
    the oracle, and exact doubling when every weight scale exponent is raised by one."""
    m, n, k = 8192, 34816, 5120
    gen = torch.Generator(device=DEV).manual_seed(1)
    w_vals = torch.randint(0, 256, (n * k * 3 // 4,), generator=gen, dtype=torch.uint8, device=DEV)
    w_scales = torch.randint(118, 124, (mx.packed_scale_numel(n, k),), generator=gen, dtype=torch.uint8, device=DEV)
    a = torch.randn((m, k), generator=gen, device=DEV, dtype=torch.float32).to(torch.bfloat16)
    act = mx.quantize_mxfp8(a)
    wgt = mx.PackedMXFP6Tensor(w_vals, w_scales, n, k)
    out = mx.gemm_w6a8(act, wgt, out_dtype=torch.bfloat16)
    doubled = mx.gemm_w6a8(act, mx.PackedMXFP6Tensor(w_vals, w_scales + 1, n, k), out_dtype=torch.bfloat16)
    assert torch.equal(doubled.float(), out.float() * 2.0)
    rows = torch.tensor([0, 1, 191, 192, 4095, 8000, 8191])
    cols = torch.cat([torch.arange(0, 130), torch.arange(34816 - 130, 34816), torch.tensor([12345, 20000])])
    a_codes = act.values.view(m, k)[rows.to(DEV)].cpu().numpy()
    a_scales = mx.unpack_scales(act.scales, m, k)[rows.to(DEV)].cpu().numpy()
    w_codes = mx.unpack_fp6(w_vals, n, k)[cols.to(DEV)].cpu().numpy()
    w_sc = mx.unpack_scales(w_scales, n, k)[cols.to(DEV)].cpu().numpy()
    want = o.gemm_w6a8(a_codes, a_scales, w_codes, w_sc, out_dtype=torch.bfloat16)
    got = out[rows.to(DEV)][:, cols.to(DEV)]
    assert _rel_fro(got, want) <= GEMM_REL_FRO


def test_workspace_arena_planning_and_graph_replay(mx):
    from mxfp6_sm120_b200._loader import check, library

    check(library().mxfp6_workspace_reset())
    mx.set_split_k_mode("workspace")  # the arena serves the scratch-based split
    try:
        _arena_body(mx, check, library)
    finally:
        mx.set_split_k_mode("cluster")
        torch.cuda.synchronize()
        check(library().mxfp6_workspace_reset())


def _arena_body(mx, check, library):
    gen = _cpu_gen(21)
    w = mx.quantize_mxfp6((torch.randn((2048, 5120), generator=gen) * 0.02).to(torch.bfloat16).to(DEV))
    acts = {m: torch.randn((m, 5120), generator=gen).to(torch.bfloat16).to(DEV) for m in (1, 16, 32)}
    eager = {m: mx.gemm(a, w, out_dtype=torch.bfloat16) for m, a in acts.items()}
    assert mx.workspace_stats()["frozen"] == 0
    torch.cuda.synchronize()
    work = torch.cuda.Stream()
    with torch.cuda.stream(work):
        mx.begin_workspace_planning()
        for a in acts.values():
            mx.gemm(a, w, out_dtype=torch.bfloat16)
        stats = mx.finalize_workspace_planning()
        assert stats["frozen"] == 1 and stats["lanes"] == 1 and stats["max_barrier_bytes"] > 0
        with pytest.raises(RuntimeError, match="frozen"):
            mx.begin_workspace_planning()
        for m, a in acts.items():
            assert torch.equal(mx.gemm(a, w, out_dtype=torch.bfloat16), eager[m])
        assert mx.workspace_stats()["persistent_launches"] >= 3
        assert mx.workspace_barriers_zero()
        # capture on the stream that owns the lane and replay 100 times
        out = torch.empty_like(eager[16])
        a_q = mx.quantize_mxfp8(acts[16])
        work.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=work):
            mx.gemm_w6a8(a_q, w, out_dtype=torch.bfloat16, out=out)
        for _ in range(100):
            graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, eager[16])
        assert mx.workspace_barriers_zero()
    # a capture on a stream without a lane must be refused
    side = torch.cuda.Stream()
    refused = False
    g2 = torch.cuda.CUDAGraph()
    try:
        with torch.cuda.graph(g2, stream=side):
            mx.gemm_w6a8(a_q, w, out_dtype=torch.bfloat16, out=out)
    except RuntimeError as error:
        refused = "no lane" in str(error)
    assert refused


def test_cluster_split_k_matches_scratch_split_and_single_pass(mx):
    """The three ways of covering K agree within the GEMM tolerance and each is
    deterministic run to run."""
    gen = _cpu_gen(14)
    a = torch.randn((24, 6144), generator=gen).to(torch.bfloat16)
    w = (torch.randn((5120, 6144), generator=gen) * 0.02).to(torch.bfloat16)
    act, wgt, (a_q, a_s, w_q, w_s) = _packed_operands(mx, a, w)
    want = o.gemm_w6a8(a_q, a_s, w_q, w_s, out_dtype=torch.bfloat16)
    outs = {}
    for mode in ("cluster", "workspace", "off"):
        mx.set_split_k_mode(mode)
        try:
            plan = mx.gemm_w6a8_plan(24, 5120, 6144)
            outs[mode] = mx.gemm_w6a8(act, wgt, out_dtype=torch.bfloat16)
            for _ in range(3):
                assert torch.equal(mx.gemm_w6a8(act, wgt, out_dtype=torch.bfloat16), outs[mode])
        finally:
            mx.set_split_k_mode("cluster")
        assert _rel_fro(outs[mode], want) <= GEMM_REL_FRO, (mode, plan)
    assert mx.gemm_w6a8_plan(24, 5120, 6144)["cluster_k"] == 6


@pytest.mark.parametrize("m,n,k,tile", [(129, 256, 128, 0), (200, 1024, 2048, 128), (700, 1024, 2048, 256),
                                        (1500, 5120, 1024, 0), (1500, 5120, 1024, 192),
                                        (300, 384, 512, 0), (520, 896, 1024, 256)])
def test_cta_pair_kernel_equals_single_cta_kernel(mx, m, n, k, tile):
    """The two-CTA kernel (256 weight rows per tile) and the single-CTA kernel add the
    same products in the same K order: outputs are bit-identical, and both meet the
    GEMM tolerance against the oracle."""
    gen = _cpu_gen(m + n + k + tile)
    a = torch.randn((m, k), generator=gen).to(torch.bfloat16)
    w = (torch.randn((n, k), generator=gen) * 0.02).to(torch.bfloat16)
    act, wgt, (a_q, a_s, w_q, w_s) = _packed_operands(mx, a, w)
    assert mx.is_cta_pair_enabled()
    plan = mx.gemm_w6a8_plan(m, n, k, tile)
    assert plan["cta_pair"] == 1 and plan["tile_tokens"] in (128, 192, 256)
    paired = mx.gemm_w6a8_config(act, wgt, out_dtype=torch.bfloat16, tile_tokens=tile)
    half = mx.gemm_w6a8_config(act, wgt, 0.25, out_dtype=torch.float16, tile_tokens=tile)
    mx.set_cta_pair_mode(False)
    try:
        assert mx.gemm_w6a8_plan(m, n, k, tile)["cta_pair"] == 0
        single = mx.gemm_w6a8_config(act, wgt, out_dtype=torch.bfloat16, tile_tokens=tile)
        single_half = mx.gemm_w6a8_config(act, wgt, 0.25, out_dtype=torch.float16, tile_tokens=tile)
    finally:
        mx.set_cta_pair_mode(True)
    assert torch.equal(paired, single) and torch.equal(half, single_half)
    want = o.gemm_w6a8(a_q, a_s, w_q, w_s, out_dtype=torch.bfloat16)
    assert _rel_fro(paired, want) <= GEMM_REL_FRO
    assert mx.device_status() == 0


def test_cta_pair_kernel_is_not_planned_outside_its_shapes(mx):
    assert mx.gemm_w6a8_plan(128, 1024, 2048)["cta_pair"] == 0      # one tile of tokens
    assert mx.gemm_w6a8_plan(512, 1000, 1024)["cta_pair"] == 0      # n not a multiple of 128
    assert mx.gemm_w6a8_plan(512, 128, 1024)["cta_pair"] == 0       # a single weight tile
    assert mx.gemm_w6a8_plan(512, 896, 1024)["cta_pair"] == 1       # last pair half empty
    assert mx.gemm_w6a8_plan(512, 1024, 2048, 64)["cta_pair"] == 0  # tile the pair kernel lacks
    assert mx.gemm_w6a8_plan(512, 1024, 2048)["cta_pair"] == 1
