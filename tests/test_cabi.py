"""CPU tests of the C ABI boundary: the library loads, exports what the header
declares, and its host-only entry points behave (no GPU work is launched)."""

from __future__ import annotations

import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "mxfp6_b200.h"


def _declared_functions() -> list[str]:
    text = HEADER.read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mxfp6_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    names = _declared_functions()
    assert "mxfp6_gemm_w6a8" in names and "mxfp6_quantize_mxfp8" in names
    assert len(names) >= 20


def test_library_exports_every_declared_symbol():
    from mxfp6_sm120_b200 import _loader

    path = _loader.load_library()
    raw = ctypes.CDLL(str(path))
    for name in _declared_functions():
        assert hasattr(raw, name), f"{name} is declared in the header but not exported"
    # the ctypes signature table covers the whole header
    assert set(_declared_functions()) == set(_loader.SIGNATURES)


def test_abi_version_matches_header():
    from mxfp6_sm120_b200._loader import library

    version = int(re.search(r"#define MXFP6_B200_ABI_VERSION (\d+)", HEADER.read_text()).group(1))
    assert library().mxfp6_b200_abi_version() == version


def test_packed_scale_bytes():
    from mxfp6_sm120_b200._loader import library

    lib = library()
    assert lib.mxfp6_packed_scale_bytes(1, 64) == 128 * 4
    assert lib.mxfp6_packed_scale_bytes(129, 256) == 256 * 8
    assert lib.mxfp6_packed_scale_bytes(16, 2048) == 128 * 64


def test_plan_is_host_arithmetic_and_validates():
    import mxfp6_sm120_b200 as mx

    small = mx.gemm_w6a8_plan(16, 1024, 2048)
    assert small["tile_tokens"] == 16 and small["splits"] >= 1 and small["stages"] >= 2
    big = mx.gemm_w6a8_plan(8192, 34816, 5120)
    assert big["tile_tokens"] in (192, 256) and big["splits"] == 1 and big["grid"] <= 148
    clustered = mx.gemm_w6a8_plan(32, 2048, 5120)
    assert clustered["cluster_k"] == 8 and clustered["splits"] == 1 and clustered["partial_bytes"] == 0
    assert clustered["grid"] % clustered["cluster_k"] == 0
    mx.set_split_k_mode("workspace")
    try:
        assert mx.is_stream_k_enabled()
        split = mx.gemm_w6a8_plan(32, 2048, 5120)
        assert split["splits"] > 1 and split["partial_bytes"] > 0 and split["counter_bytes"] > 0
        assert split["cluster_k"] == 1
    finally:
        mx.set_split_k_mode("cluster")
    mx.set_split_k_mode("off")
    try:
        off = mx.gemm_w6a8_plan(32, 2048, 5120)
        assert off["splits"] == 1 and off["cluster_k"] == 1
    finally:
        mx.set_split_k_mode("cluster")
    with pytest.raises(ValueError):
        mx.set_split_k_mode("bogus")
    with pytest.raises(ValueError, match="multiple of 128"):
        mx.gemm_w6a8_plan(16, 1024, 2000)
    with pytest.raises(ValueError, match="multiple of 8"):
        mx.gemm_w6a8_plan(16, 1003, 2048)
    with pytest.raises(ValueError, match="positive"):
        mx.gemm_w6a8_plan(0, 1024, 2048)
    with pytest.raises(ValueError, match="tile_tokens"):
        mx.gemm_w6a8_plan(64, 1024, 2048, tile_tokens=16)


def test_null_pointer_arguments_are_rejected_before_any_launch():
    from mxfp6_sm120_b200._loader import library

    lib = library()
    assert lib.mxfp6_pack_fp6(None, 16, None, None) == 1
    assert b"null" in lib.mxfp6_b200_last_error()
    assert lib.mxfp6_quantize_mxfp8(None, 1, 4, 128, None, None, None, None) == 1
    assert lib.mxfp6_unpack_scales(None, 0, 128, None, None) == 1


def test_missing_library_is_an_import_error(monkeypatch, tmp_path):
    import importlib

    from mxfp6_sm120_b200 import _loader

    fresh = importlib.reload(_loader)
    monkeypatch.setenv("MXFP6_LIBRARY_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(ImportError, match="libmxfp6_b200.so"):
        fresh.load_library()
    monkeypatch.delenv("MXFP6_LIBRARY_PATH")
    importlib.reload(_loader)


def test_python_validation_mirrors_reference_errors():
    import torch

    import mxfp6_sm120_b200 as mx

    cpu = torch.zeros((4, 128), dtype=torch.uint8)
    with pytest.raises(ValueError, match="CUDA tensor"):
        mx.pack_fp6(cpu)
    with pytest.raises(ValueError, match="CUDA tensor"):
        mx.quantize_mxfp8(torch.zeros((4, 128), dtype=torch.bfloat16))
    with pytest.raises(TypeError, match="out_dtype"):
        mx.gemm(torch.zeros(1), None, out_dtype=torch.float32)
    assert mx.is_available() in (True, False)
    assert mx.is_tuned_shape(32, 34816, 5120) and not mx.is_tuned_shape(33, 34816, 5120)
    assert mx.packed_scale_numel(129, 256) == 2048


def test_decoder_side_entry_points_validate_before_any_launch():
    """Argument checks of the fused norm and the peer-memory collectives run on the host."""
    import ctypes as c

    from mxfp6_sm120_b200._loader import library

    lib = library()
    # fused (residual +) RMSNorm + MXFP8: null input, then a residual without its output
    assert lib.mxfp6_rmsnorm_quantize_mxfp8(None, None, None, 1, None, 1e-6, 4, 128, None, None,
                                            None, None) == 1
    blocks = (c.c_void_p * 2)(None, None)
    # world outside [1, 8], a rank outside the world, a buffer index that does not exist
    assert lib.mxfp6_tp_allreduce_bf16(blocks, 9, 0, 0, 4096, None, 4, 128, None) == 1
    assert lib.mxfp6_tp_allreduce_bf16(blocks, 2, 2, 0, 4096, None, 4, 128, None) == 1
    assert lib.mxfp6_tp_allreduce_bf16(blocks, 2, 0, 2, 4096, None, 4, 128, None) == 1
    assert b"buffer" in lib.mxfp6_b200_last_error()
    assert lib.mxfp6_tp_allreduce_rmsnorm_quantize_mxfp8(blocks, 2, 0, 0, 4096, None, None, 1e-6,
                                                         4, 128, None, None, None) == 1
    handle = (c.c_ubyte * 64)()
    out = c.c_void_p()
    assert lib.mxfp6_tp_block_alloc(100, c.byref(out), handle) == 1   # not a multiple of 256
    assert b"256" in lib.mxfp6_b200_last_error()
