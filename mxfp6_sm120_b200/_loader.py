"""Locates and loads ``libmxfp6_b200.so`` and declares its C ABI for ctypes.

Mirrors the reference loader's contract (python/mxfp6/_loader.py:14-50):
``MXFP6_LIBRARY_PATH`` overrides discovery, a missing library is an
``ImportError`` and there is no fallback implementation.
"""

from __future__ import annotations

import ctypes
import os
import threading
from ctypes import POINTER, c_char_p, c_float, c_int, c_int64, c_size_t, c_void_p
from pathlib import Path

_LOAD_LOCK = threading.Lock()
_LIBRARY: ctypes.CDLL | None = None
_LIBRARY_PATH: Path | None = None

_I64P = POINTER(c_int64)
_IP = POINTER(c_int)

# name -> (restype, argtypes); every symbol declared in include/mxfp6_b200.h.
SIGNATURES: dict[str, tuple] = {
    "mxfp6_b200_abi_version": (c_int, []),
    "mxfp6_b200_last_error": (c_char_p, []),
    "mxfp6_b200_device_status": (c_int, [_IP, c_int]),
    "mxfp6_pack_fp6": (c_int, [c_void_p, c_int64, c_void_p, c_void_p]),
    "mxfp6_unpack_fp6": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p]),
    "mxfp6_pad_fp6": (c_int, [c_void_p, c_int64, c_void_p, c_void_p]),
    "mxfp6_expand_fp6_to_fp8": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p]),
    "mxfp6_pack_scales": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p]),
    "mxfp6_unpack_scales": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p]),
    "mxfp6_packed_scale_bytes": (c_int64, [c_int64, c_int64]),
    "mxfp6_grouped_scale_offsets": (c_int, [c_void_p, c_int, c_void_p, c_void_p]),
    "mxfp6_pack_grouped_scales": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_void_p, c_void_p],
    ),
    "mxfp6_tp_block_alloc": (c_int, [c_size_t, POINTER(c_void_p), c_void_p]),
    "mxfp6_tp_block_open": (c_int, [c_void_p, POINTER(c_void_p)]),
    "mxfp6_tp_block_close": (c_int, [c_void_p]),
    "mxfp6_tp_block_free": (c_int, [c_void_p]),
    "mxfp6_tp_set_wait_limit": (c_int, [c_int64]),
    "mxfp6_tp_get_wait_limit": (c_int64, []),
    "mxfp6_tp_allreduce_bf16": (
        c_int,
        [POINTER(c_void_p), c_int, c_int, c_int, c_size_t, c_void_p, c_int64, c_int64, c_void_p],
    ),
    "mxfp6_tp_allreduce_two_phase_bf16": (
        c_int,
        [POINTER(c_void_p), c_int, c_int, c_int, c_size_t, c_void_p, c_int64, c_int64, c_void_p],
    ),
    "mxfp6_tp_reduce_scatter_bf16": (
        c_int,
        [POINTER(c_void_p), c_int, c_int, c_int, c_size_t, c_void_p, c_int64, c_int64, c_void_p],
    ),
    "mxfp6_tp_allgather": (
        c_int,
        [POINTER(c_void_p), c_int, c_int, c_int, c_size_t, c_int, _I64P, _I64P, POINTER(c_void_p),
         c_void_p],
    ),
    "mxfp6_tp_allreduce_rmsnorm_quantize_mxfp8": (
        c_int,
        [POINTER(c_void_p), c_int, c_int, c_int, c_size_t, c_void_p, c_void_p, c_float, c_int64,
         c_int64, c_void_p, c_void_p, c_void_p],
    ),
    "mxfp6_rmsnorm_quantize_mxfp8": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_float, c_int64, c_int64, c_void_p,
         c_void_p, c_void_p, c_void_p],
    ),
    "mxfp6_quantize_mxfp8": (
        c_int,
        [c_void_p, c_int, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p],
    ),
    "mxfp6_quantize_mxfp6": (
        c_int,
        [c_void_p, c_int, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p],
    ),
    "mxfp6_gemm_w6a8": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_float, c_void_p,
         c_int, c_void_p],
    ),
    "mxfp6_gemm_w6a8_static_scratch": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_float, c_void_p,
         c_int, c_void_p],
    ),
    "mxfp6_gemm_w6a8_ex": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_float, c_void_p,
         c_int, c_int, c_int, c_void_p, c_size_t, c_void_p],
    ),
    "mxfp6_gemm_w6a8_plan": (c_int, [c_int64, c_int64, c_int64, c_int, c_int, _I64P]),
    "mxfp6_set_stream_kernel_mode": (c_int, [c_int]),
    "mxfp6_get_stream_kernel_mode": (c_int, []),
    "mxfp6_w6a8_config_abi": (c_char_p, []),
    "mxfp6_w6a8_config_count": (c_int, []),
    "mxfp6_w6a8_config_describe": (c_int, [c_int, _IP]),
    "mxfp6_set_w6a8_config": (c_int, [c_int64, c_int64, c_int64, c_int, c_int]),
    "mxfp6_gemm_w6a8_config": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_float, c_void_p,
         c_int, c_int, c_void_p],
    ),
    "mxfp6_set_split_k_mode": (c_int, [c_int]),
    "mxfp6_get_split_k_mode": (c_int, []),
    "mxfp6_set_cta_pair_mode": (c_int, [c_int]),
    "mxfp6_get_cta_pair_mode": (c_int, []),
    "mxfp6_gemm_from_float": (
        c_int,
        [c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_float, c_void_p, c_int,
         c_void_p, c_void_p, c_void_p],
    ),
    "mxfp6_array_gemm_w6a8": (
        c_int,
        [c_void_p, c_int, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_int,
         c_int64, c_int, c_int, c_int64, c_int64, c_void_p],
    ),
    "mxfp6_array_gemm_w6a8_silu_mxfp8": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p,
         c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_int64, c_int64, c_void_p],
    ),
    "mxfp6_array_gemm_w6a8_reduce": (
        c_int,
        [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
         c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int64, c_int,
         c_int64, c_int64, c_int, c_void_p],
    ),
    "mxfp6_moe_decode_layer_supported": (c_int, [c_int64, c_int, c_int, c_int64, c_int64]),
    "mxfp6_moe_decode_layer_preferred": (c_int, [c_int64, c_int, c_int, c_int64, c_int64]),
    "mxfp6_moe_decode_layer": (
        c_int,
        [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
         c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
         c_void_p, c_int64, c_int, c_int, c_int, c_int64, c_int64, c_int, c_void_p],
    ),
    "mxfp6_moe_reduce_tp_pointers": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int,
         c_int, c_int64, c_void_p, c_void_p, c_int, c_int, c_void_p],
    ),
    "mxfp6_moe_reduce_array": (
        c_int,
        [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int64, c_int, c_int64,
         c_void_p],
    ),
    "mxfp6_moe_router_logits": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_void_p],
    ),
    "mxfp6_moe_topk_quant": (
        c_int,
        [c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
         c_void_p, c_void_p, c_void_p],
    ),
    "mxfp6_moe_topk_quant_route": (
        c_int,
        [c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
         c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
         c_void_p, c_void_p, c_void_p, c_void_p],
    ),
    "mxfp6_moe_route": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_void_p, c_int, c_int,
         c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    ),
    "mxfp6_moe_route_shared": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_void_p, c_int, c_int, c_int,
         c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    ),
    "mxfp6_grouped_gemm_w6a8": (
        c_int,
        [c_void_p, c_int, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
         c_int, c_int64, c_int64, c_int64, c_int, c_void_p],
    ),
    "mxfp6_w1_swiglu_mxfp8": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p,
         c_void_p, c_int, c_int64, c_int64, c_int64, c_int, c_void_p],
    ),
    "mxfp6_silu_and_mul_mxfp8": (
        c_int,
        [c_void_p, c_int, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
         c_int, c_void_p],
    ),
    "mxfp6_moe_reduce": (
        c_int,
        [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64,
         c_int, c_int, c_int64, c_void_p],
    ),
    "mxfp6_workspace_begin_planning": (c_int, []),
    "mxfp6_workspace_finalize_planning": (c_int, [c_void_p, _I64P]),
    "mxfp6_workspace_stats": (c_int, [_I64P]),
    "mxfp6_workspace_barriers_zero": (c_int, [_IP]),
    "mxfp6_workspace_reset": (c_int, []),
}


def _library_candidates() -> list[Path]:
    override = os.environ.get("MXFP6_LIBRARY_PATH")
    if override:
        return [Path(override)]
    package_dir = Path(__file__).resolve().parent
    return [package_dir / "lib" / "libmxfp6_b200.so"]


def load_library() -> Path:
    """Load the native library once and return its path."""
    global _LIBRARY, _LIBRARY_PATH
    with _LOAD_LOCK:
        if _LIBRARY is not None:
            assert _LIBRARY_PATH is not None
            return _LIBRARY_PATH
        candidates = _library_candidates()
        for path in candidates:
            if path.is_file():
                library = ctypes.CDLL(str(path))
                for name, (restype, argtypes) in SIGNATURES.items():
                    function = getattr(library, name)  # AttributeError -> broken build
                    function.restype = restype
                    function.argtypes = argtypes
                _LIBRARY = library
                _LIBRARY_PATH = path
                return path
        searched = ", ".join(str(path) for path in candidates)
        raise ImportError(
            "Could not find libmxfp6_b200.so; build it with "
            "`python -m mxfp6_sm120_b200.build` or set MXFP6_LIBRARY_PATH. "
            f"Searched: {searched}"
        )


def library() -> ctypes.CDLL:
    """Return the loaded ``ctypes.CDLL`` (loading it on first use)."""
    load_library()
    assert _LIBRARY is not None
    return _LIBRARY


def check(status: int) -> None:
    """Raise the exception that corresponds to a non-zero C ABI status."""
    if status == 0:
        return
    message = library().mxfp6_b200_last_error().decode("utf-8", "replace")
    if status == 1:
        raise ValueError(message)
    raise RuntimeError(message)
