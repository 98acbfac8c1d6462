"""CPU tests that pin the oracle to the reference's golden vectors and helpers."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import mx_oracle as o


@pytest.fixture(scope="module")
def cvt(golden_dir):
    return np.load(golden_dir / "cvt_tables.npz")


@pytest.fixture(scope="module")
def ref(golden_dir):
    return np.load(golden_dir / "reference_helpers.npz")


def _all_bf16():
    return (np.arange(65536, dtype=np.uint32) << 16).view(np.float32)


def test_e4m3_conversion_matches_cuda_host_table(cvt):
    x = _all_bf16()
    finite = np.isfinite(x)
    assert np.array_equal(o.encode_e4m3(x[finite]), cvt["e4m3"][finite])


def test_e3m2_conversion_matches_cuda_host_table(cvt):
    x = _all_bf16()
    finite = np.isfinite(x)
    assert np.array_equal(o.encode_e3m2(x[finite]), cvt["e3m2"][finite])


def test_torch_float8_cast_matches_table_inside_range(cvt):
    # The reference test's cross-check formula uses torch's cast; it differs from
    # the saturating conversion only beyond +-448, which the scale rule excludes.
    x = _all_bf16()
    inside = np.isfinite(x) & (np.abs(x) <= 448.0)
    cast = torch.from_numpy(x[inside]).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(cast, cvt["e4m3"][inside])


def test_e3m2_and_ue8m0_tables_match_reference_decoders(ref):
    assert np.array_equal(o.decode_e3m2(torch.arange(64, dtype=torch.uint8)).numpy(), ref["e3m2_table"])
    mine = o.decode_ue8m0(torch.arange(256, dtype=torch.uint8)).view(torch.int32).numpy()
    assert np.array_equal(mine, ref["ue8m0_table_bits"])
    assert o.decode_ue8m0(torch.tensor([0x7F], dtype=torch.uint8)).item() == 1.0


def test_e3m2_table_known_values():
    table = o.decode_e3m2(torch.arange(64, dtype=torch.uint8))
    assert table[0] == 0.0 and table[1] == 0.0625 and table[3] == 0.1875
    assert table[4] == 0.25 and table[31] == 28.0 and table[63] == -28.0
    assert table[32] == 0.0 and torch.signbit(table[32])


def test_pack_matches_reference_bitstream(ref):
    assert np.array_equal(o.pack_fp6(ref["pack_codes"]), ref["pack_bytes"])
    assert o.pack_fp6([1, 2, 3, 4]).tolist() == [129, 48, 16]
    assert ref["pack_1234"].tolist() == [129, 48, 16]
    rows, k = ref["pack_codes"].shape
    assert np.array_equal(o.unpack_fp6(ref["pack_bytes"], rows, k), ref["pack_codes"] & 0x3F)


def test_w6a6_decoded_gemm_matches_reference_gemm(ref):
    a = o.dequant_mxfp6(ref["w6a6_a_codes"], ref["w6a6_sfa"])
    b = o.dequant_mxfp6(ref["w6a6_b_codes"], ref["w6a6_sfb"])
    out = (a @ b.t()).to(torch.float16).view(torch.int16).numpy()
    assert np.array_equal(out, ref["w6a6_out_f16_bits"])


def _c1_inputs():
    gen = torch.Generator(device="cpu").manual_seed(0)
    a = torch.randn((16, 2048), generator=gen, dtype=torch.float32).to(torch.bfloat16)
    w = (torch.randn((1024, 2048), generator=gen, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    return a, w


def test_correctness_gemm_matches_reference_decode_path(ref):
    a, w = _c1_inputs()
    a_q, a_s = o.quantize_mxfp8(a)
    w_q, w_s = o.quantize_mxfp6(w)
    assert np.array_equal(a_q, ref["c1_a_codes_by_reference_formula"])
    assert np.array_equal(a_s, ref["c1_a_scales"])
    out = o.gemm_w6a8(a_q, a_s, w_q, w_s, out_dtype=torch.bfloat16)
    assert np.array_equal(out.view(torch.int16).numpy(), ref["c1_out_bf16_bits"])


def test_quantizer_variants_agree():
    gen = torch.Generator(device="cpu").manual_seed(3)
    for dtype in (torch.bfloat16, torch.float16):
        x = (torch.randn((9, 256), generator=gen) * 6.0).to(dtype)
        c_np, s_np = o.quantize_mxfp8(x)
        c_t, s_t = o.quantize_mxfp8_torch(x)
        assert np.array_equal(c_np, c_t) and np.array_equal(s_np, s_t)


def test_quantizer_corner_cases():
    x = torch.zeros((1, 128), dtype=torch.bfloat16)
    x[0, 32] = -0.0
    x[0, 33] = -1e-38
    x[0, 64:96] = 448.0          # exact power-of-two ratio: scale stays 1.0
    x[0, 96] = 449.0             # just above: scale doubles (bf16(449) = 448 -> stays)
    x[0, 97] = 452.0
    codes, scales = o.quantize_mxfp8(x)
    assert scales[0, 0] == 28 and not codes[0, :32].any()      # all-zero group: 2^-99
    assert codes[0, 32] == 0x80                                  # -0.0 keeps its sign
    assert codes[0, 33] & 0x80
    assert scales[0, 2] == 127 and codes[0, 64] == 0x7E          # 448 -> max finite code
    assert scales[0, 3] == 128                                   # 452/448 > 1 -> 2.0
    # scaled group maximum always lands in (T/2, T]
    gen = torch.Generator(device="cpu").manual_seed(5)
    y = (torch.randn((64, 512), generator=gen) * torch.logspace(-6, 6, 64)[:, None]).to(torch.bfloat16)
    for bits, target in ((8, 448.0), (6, 28.0)):
        _, s = o.quantize_mx(y, bits)
        amax = y.float().view(64, 16, 32).abs().amax(dim=2)
        scaled = amax / o.decode_ue8m0(torch.from_numpy(s))
        assert bool(((scaled > target / 2) & (scaled <= target)).all())


def test_all_e3m2_values_round_trip_with_unit_scale():
    # Every group holds +-28, so the scale is exactly 1.0 and codes come back unchanged
    # (the reference's round-trip check, tests/test_ops.py:1544-1555).
    values = o.decode_e3m2(torch.arange(64, dtype=torch.uint8)).repeat(4, 2)
    codes, scales = o.quantize_mxfp6(values.to(torch.bfloat16))
    assert (scales == 0x7F).all()
    back = o.decode_e3m2(torch.from_numpy(codes))
    assert torch.equal(back, values)


def test_expand_fp6_to_fp8_is_lossless():
    codes = np.arange(64, dtype=np.uint8).repeat(4).reshape(2, 128)
    expanded = o.expand_fp6_to_fp8(o.pack_fp6(codes), 2, 128)
    assert torch.equal(o.decode_e4m3(torch.from_numpy(expanded)), o.decode_e3m2(torch.from_numpy(codes)))
    # the four E3M2 subnormals map to E4M3 0x00, 0x18, 0x20, 0x24
    assert o.encode_e4m3(o.decode_e3m2(torch.arange(4)).numpy()).tolist() == [0x00, 0x18, 0x20, 0x24]


@pytest.mark.parametrize("rows,k", [(1, 64), (1, 128), (16, 128), (32, 256), (128, 128), (129, 256), (2048, 128)])
def test_scale_layout_round_trip_and_padding(rows, k):
    gen = np.random.default_rng(rows * 1000 + k)
    logical = gen.integers(120, 135, size=(rows, k // 32), dtype=np.uint8)
    packed = o.pack_scales(logical)
    groups = (k // 32 + 3) // 4 * 4
    assert packed.size == (rows + 127) // 128 * 128 * groups
    assert np.array_equal(o.unpack_scales(packed, rows, k), logical)
    # every byte that is not a logical scale is 0x7f
    mask = np.ones(packed.size, dtype=bool)
    r, g = np.meshgrid(np.arange(rows), np.arange(k // 32), indexing="ij")
    mask[o.packed_scale_offset(r, g, k // 32)] = False
    assert (packed[mask] == 0x7F).all()


def test_scale_offset_formula_examples():
    # 128 rows x 4 groups form one 512-byte atom ordered (row % 32, row / 32, group).
    assert o.packed_scale_offset(0, 0, 8) == 0
    assert o.packed_scale_offset(1, 0, 8) == 16
    assert o.packed_scale_offset(32, 0, 8) == 4
    assert o.packed_scale_offset(0, 3, 8) == 3
    assert o.packed_scale_offset(0, 4, 8) == 512
    assert o.packed_scale_offset(128, 0, 8) == 1024


def test_grouped_scale_offsets_known_answer():
    counts = (1, 0, 3, 129, 2)
    offsets = np.concatenate([[0], np.cumsum(counts)])
    assert o.grouped_scale_offsets(offsets).tolist() == [0, 128, 128, 256, 512, 640]
    gen = np.random.default_rng(0)
    logical = gen.integers(120, 135, size=(sum(counts), 4), dtype=np.uint8)
    packed, soff = o.pack_grouped_scales(logical, offsets)
    for e, rows in enumerate(counts):
        if rows == 0:
            continue
        first = int(soff[e])
        padded = (rows + 127) // 128 * 128
        piece = packed[first * 4 : (first + padded) * 4]
        assert np.array_equal(o.unpack_scales(piece, rows, 128), logical[offsets[e] : offsets[e] + rows])


def test_silu_path_roundings():
    gen = torch.Generator(device="cpu").manual_seed(9)
    x = torch.randn((5, 128), generator=gen) * 3
    v = o.silu_and_mul_bf16(x)
    g = x[:, :64].bfloat16().float()
    u = x[:, 64:].bfloat16().float()
    s = (g / (1 + torch.exp(-g))).bfloat16().float()
    assert torch.equal(v, (s * u).bfloat16().float())
    codes, scales = o.silu_and_mul_mxfp8(x)
    assert codes.shape == (5, 64) and scales.shape == (5, 2)


def test_topk_ties_pick_smaller_expert_and_renormalise():
    logits = torch.zeros((2, 256), dtype=torch.bfloat16)
    logits[1, 200] = 3.0
    logits[1, 7] = 3.0
    w, ids = o.softmax_topk(logits, 8, True)
    assert ids[0].tolist() == list(range(8))
    assert ids[1].tolist()[:2] == [7, 200]
    assert torch.allclose(w.sum(dim=1), torch.ones(2))


def test_reduce_sigmoid_gate_identity():
    # gate logit 20 passes the shared row, gate 0 halves it (tests/test_ops.py:1178-1209).
    routed = torch.zeros((8, 64), dtype=torch.bfloat16)
    shared = torch.ones((1, 64), dtype=torch.bfloat16)
    w = torch.zeros((1, 8))
    inv = torch.arange(8, dtype=torch.int32)
    full = o.moe_reduce(routed, w, inv, shared, torch.tensor([20.0]))
    half = o.moe_reduce(routed, w, inv, shared, torch.tensor([0.0]))
    assert torch.equal(full.float(), torch.ones((1, 64)))
    assert torch.equal(half.float(), torch.full((1, 64), 0.5))


def test_division_free_scale_rule_equals_the_division_for_every_half_precision_magnitude():
    """The kernels pick the UE8M0 scale from the exponent and mantissa fields of the block
    maximum, code = max(28, exponent - shift + (mantissa > 0x600000)) with shift 8 for the
    E4M3 target 448 and 4 for the E3M2 target 28, instead of dividing as the reference does
    (csrc/quantization.cu:118-127).  Both agree for every non-negative finite BF16 and FP16
    value a block maximum can take."""
    bf16 = (np.arange(0, 0x7F80, dtype=np.uint32) << 16).view(np.float32)
    fp16 = np.arange(0, 0x7C00, dtype=np.uint16).view(np.float16).astype(np.float32)
    for values in (bf16, fp16):
        bits = values.view(np.uint32)
        exponent = (bits >> 23).astype(np.int64)
        bump = ((bits & 0x7FFFFF) > 0x600000).astype(np.int64)
        for target, shift in ((448.0, 8), (28.0, 4)):
            fast = np.maximum(28, exponent - shift + bump)
            with np.errstate(over="ignore"):
                want = (o._scale_bits(values, target) >> 23).astype(np.int64)
            assert np.array_equal(fast, want), (target, np.flatnonzero(fast != want)[:5])
