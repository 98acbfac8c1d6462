"""Parity of the dense W6A8 GEMM on the shapes and plans the benchmark times.

The five projections of the 27B-class decoder at decode and prefill batch sizes, each
through the DEFAULT plan (the one ``bench.py`` gets: the weight-streaming kernel with its
cluster split up to 64 rows, the persistent kernel up to 96 rows, CTA pairs above), compared
with the CPU oracle (decoded FP32 matmul on the same codes, the reference's
``reference_gemm``, tests/test_ops.py:1426-1435) on sampled output columns: the first and
last 130 features (tile edges on both sides) and a few inside.  Tolerance: rel-Frobenius
<= 1e-3 against the oracle's output in the same dtype (the reference's own check uses
rtol 2e-3, tests/test_ops.py:1881-1885).  The activation codes and scales that the GPU
quantizer produced are compared bit for bit with the oracle's on the way.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import mx_oracle as o

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
GEMM_REL_FRO = 1.0e-3
NK = [(7168, 5120), (5120, 6144), (34816, 5120), (5120, 17408), (2048, 5120)]
M_VALUES = [1, 8, 32, 64, 96, 128, 512]


def _expected_plan(m: int, n: int, k: int) -> dict:
    n_tiles = n // 128
    split = 2 * n_tiles <= 240
    if m <= 32 or (m <= 64 and split):
        ck = min(8, 240 // n_tiles, k // 128) if split else 1
        return {"kernel": "stream", "tile_tokens": 16 if m <= 16 else 32 if m <= 32 else 64,
                "cluster_k": max(ck, 1), "cta_pair": 0, "splits": 1}
    if m <= 128:
        # 65..128 rows: two 64-row tiles while the weights fit the L2, else one 96- or 128-row
        # tile (the 128-row tile has no cluster split)
        tile = 64 if (m <= 64 or n * k * 3 // 4 <= 32 << 20) else 96 if m <= 96 else 128
        tiles = n_tiles * -(-m // tile)
        ck = min(8, (148 - 16) // tiles, k // 128) if (2 * tiles <= 148 and tile <= 96) else 1
        return {"kernel": "persistent", "tile_tokens": tile,
                "cluster_k": ck if ck >= 2 else 1, "cta_pair": 0, "splits": 1}
    return {"kernel": "cta_pair", "cluster_k": 1, "cta_pair": 1, "splits": 1}


@pytest.fixture(scope="module")
def weights(mx):
    """Packed weights as the benchmark builds them: every 6-bit pattern is a valid code."""
    made = {}
    for index, (n, k) in enumerate(NK):
        gen = torch.Generator(device=DEV).manual_seed(1000 + index)
        values = torch.randint(0, 256, (n * k * 3 // 4,), generator=gen, dtype=torch.uint8, device=DEV)
        scales = torch.randint(118, 124, (mx.packed_scale_numel(n, k),), generator=gen,
                               dtype=torch.uint8, device=DEV)
        made[(n, k)] = mx.PackedMXFP6Tensor(values, scales, n, k)
    yield made
    made.clear()
    torch.cuda.empty_cache()


@pytest.mark.parametrize("n,k", NK)
@pytest.mark.parametrize("m", M_VALUES)
def test_default_plan_matches_oracle_on_sampled_columns(mx, weights, m, n, k):
    plan = mx.gemm_w6a8_plan(m, n, k)
    for key, want in _expected_plan(m, n, k).items():
        assert plan[key] == want, (key, plan)
    wgt = weights[(n, k)]
    a = torch.randn((m, k), generator=torch.Generator(device="cpu").manual_seed(2000 + m)).to(torch.bfloat16)
    a_dev = a.to(DEV)

    act = mx.quantize_mxfp8(a_dev)
    a_codes, a_scales = o.quantize_mxfp8_torch(a)
    assert np.array_equal(act.values.cpu().numpy().reshape(m, k), a_codes)
    assert np.array_equal(mx.unpack_scales(act.scales, m, k).cpu().numpy(), a_scales)

    out = mx.gemm_w6a8(act, wgt, out_dtype=torch.bfloat16)
    fused = mx.gemm_from_float(a_dev, wgt, out_dtype=torch.bfloat16)  # the call the benchmark makes
    assert torch.equal(out, fused)
    again = mx.gemm_w6a8(act, wgt, out_dtype=torch.bfloat16)
    assert torch.equal(out, again)  # split-K sums in a fixed order

    inner = torch.randint(130, n - 130, (6,), generator=torch.Generator().manual_seed(n + m))
    cols = torch.cat([torch.arange(0, 130), inner, torch.arange(n - 130, n)]).to(DEV)
    rows = torch.arange(m) if m <= 128 else torch.tensor([0, 1, 127, 128, 191, 192, 255, 256, m - 1])
    w_codes = mx.unpack_fp6(wgt.values, n, k)[cols].cpu().numpy()
    w_scales = mx.unpack_scales(wgt.scales, n, k)[cols].cpu().numpy()
    want = o.gemm_w6a8(a_codes[rows.numpy()], a_scales[rows.numpy()], w_codes, w_scales,
                       out_dtype=torch.bfloat16)
    got = out[rows.to(DEV)][:, cols].float().cpu()
    rel = float((got - want.float()).norm() / want.float().norm().clamp_min(1e-30))
    assert rel <= GEMM_REL_FRO, (m, n, k, rel)
    assert mx.device_status() == 0


@pytest.mark.parametrize("config_id,m", [(3, 16), (7, 1), (10, 24), (21, 24), (35, 300), (40, 16), (53, 50)])
def test_explicit_configuration_and_override_registry(mx, weights, config_id, m):
    """``gemm_w6a8_config(config_id=...)`` runs the named configuration; ``set_w6a8_config``
    makes the plain call take it for exactly that shape and output dtype
    (the reference's contract, csrc/torch_extension.cu:1139-1167,1192-1199)."""
    n, k = 2048, 5120
    wgt = weights[(n, k)]
    a = torch.randn((m, k), generator=torch.Generator(device="cpu").manual_seed(77 + m)).to(torch.bfloat16).to(DEV)
    act = mx.quantize_mxfp8(a)
    default = mx.gemm_w6a8(act, wgt, out_dtype=torch.bfloat16)
    explicit = mx.gemm_w6a8_config(act, wgt, out_dtype=torch.bfloat16, config_id=config_id)
    rel = float((explicit.float() - default.float()).norm() / default.float().norm())
    assert rel <= GEMM_REL_FRO
    described = mx.w6a8_configs()[config_id]
    try:
        assert mx.set_w6a8_config(a, m, n, k, config_id, output_dtype=torch.bfloat16)
        plan = mx.gemm_w6a8_plan(m, n, k)
        assert plan["kernel"] == described["kernel"] and plan["tile_tokens"] == described["tile_tokens"]
        if described["cluster_k"] > 1:
            assert plan["cluster_k"] == described["cluster_k"]
        if described["splits"] > 1:
            assert plan["splits"] == described["splits"]
        pinned = mx.gemm_w6a8(act, wgt, out_dtype=torch.bfloat16)
        assert torch.equal(pinned, explicit)
        # another batch size is not affected
        assert mx.gemm_w6a8_plan(m + 1, n, k)["kernel"] == mx.gemm_w6a8_plan(m + 1, n, k)["kernel"]
    finally:
        mx.set_w6a8_config(a, m, n, k, -1, output_dtype=torch.bfloat16)
    back = mx.gemm_w6a8_plan(m, n, k)
    assert back == mx.gemm_w6a8_plan(m, n, k) and torch.equal(mx.gemm_w6a8(act, wgt, out_dtype=torch.bfloat16), default)
    with pytest.raises(ValueError):
        mx.set_w6a8_config(a, m, n, k, 58, output_dtype=torch.bfloat16)       # no such id
    with pytest.raises(ValueError):
        mx.set_w6a8_config(a, 64, n, k, 3, output_dtype=torch.bfloat16)       # 16-row tile, 64 rows
    with pytest.raises(ValueError):
        mx.set_w6a8_config(a, m, n, k, 3, swizzle=3, output_dtype=torch.bfloat16)
    assert mx.device_status() == 0
