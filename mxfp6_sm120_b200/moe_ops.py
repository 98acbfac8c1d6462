"""Routed-MoE operators (top-k routing, permutation, grouped W6A8 GEMMs, fused
SwiGLU requantization, reduce) with the names and argument meaning of the
reference's ``python/mxfp6/ops.py``.  All ``*_out`` functions write into
caller-owned tensors and allocate nothing, so a whole layer captures into one
CUDA graph.  Shapes are generic (hidden size, intermediate size, expert count
and k are read from the tensors) instead of the reference's hard-coded
2048 / 256 / 256 / 8.
"""

from __future__ import annotations

import ctypes

import torch

from ._loader import check, library, load_library
from .ops import (
    SCALE_VECTOR_SIZE,
    _DTYPE_CODE,
    _ptr,
    _require_cuda_uint8_contiguous,
    _require_sm100,
    _stream,
    _validate_output_dtype,
    packed_scale_numel,
)

_GATE_CODE = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}


def _as_u8(tensor: torch.Tensor) -> torch.Tensor:
    return tensor.view(torch.uint8) if tensor.dtype == torch.float8_e4m3fn else tensor


def _check_offsets(tensor: torch.Tensor, device: torch.device, name: str) -> None:
    if (
        tensor.device != device
        or tensor.dtype != torch.int64
        or tensor.ndim != 1
        or tensor.numel() < 2
        or not tensor.is_contiguous()
    ):
        raise ValueError(f"{name} must be a contiguous CUDA int64 tensor with E+1 entries")


def grouped_scale_rows(rows: int, experts: int) -> int:
    """Row capacity of a grouped packed scale buffer: every active expert may add
    up to 127 rows of padding (the reference's sizing, python/mxfp6/ops.py:1494)."""
    return rows + min(rows, experts) * 127


# ------------------------------------------------------------------- SiLU * mul + MXFP8


def _check_silu_input(input: torch.Tensor) -> tuple[int, int]:
    if (
        input.device.type != "cuda"
        or input.dtype not in (torch.float16, torch.bfloat16)
        or input.ndim != 2
        or not input.is_contiguous()
        or input.shape[1] % 64
    ):
        raise ValueError(
            "input must be contiguous CUDA float16/bfloat16 [M,2K] with K divisible by 32"
        )
    return int(input.shape[0]), int(input.shape[1]) // 2


def _silu_raw(input, output, logical, packed, expert_offsets, scale_offsets) -> None:
    rows, inter = _check_silu_input(input)
    experts = 0 if expert_offsets is None else expert_offsets.numel() - 1
    with torch.cuda.device(input.device):
        check(
            library().mxfp6_silu_and_mul_mxfp8(
                input.data_ptr(), _DTYPE_CODE[input.dtype], rows, inter, output.data_ptr(),
                _ptr(logical), _ptr(packed), _ptr(expert_offsets), _ptr(scale_offsets), experts,
                _stream(input.device),
            )
        )


def silu_and_mul_mxfp8_logical(input: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Fuse SiLU-and-mul with row-major logical MXFP8 quantization."""
    rows, inter = _check_silu_input(input)
    _require_sm100(input.device)
    load_library()
    values = torch.empty((rows, inter), dtype=torch.uint8, device=input.device)
    scales = torch.empty((rows, inter // SCALE_VECTOR_SIZE), dtype=torch.uint8, device=input.device)
    _silu_raw(input, values, scales, None, None, None)
    return values.view(torch.float8_e4m3fn), scales


def silu_and_mul_mxfp8_packed_out(
    output: torch.Tensor, packed_scales: torch.Tensor, input: torch.Tensor
) -> None:
    """Fuse SiLU-and-mul with MXFP8 quantization into dense packed scales."""
    rows, inter = _check_silu_input(input)
    if _as_u8(output).shape != (rows, inter) or not output.is_contiguous():
        raise ValueError(f"output must be contiguous CUDA MXFP8 {(rows, inter)}")
    _require_cuda_uint8_contiguous(packed_scales, "packed_scales")
    if packed_scales.numel() < packed_scale_numel(rows, inter):
        raise ValueError("packed_scales is too small")
    _require_sm100(input.device)
    load_library()
    _silu_raw(input, _as_u8(output), None, packed_scales, None, None)


def silu_and_mul_mxfp8_grouped(
    input: torch.Tensor,
    expert_offsets: torch.Tensor,
    scale_offsets: torch.Tensor | None = None,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Fuse SiLU-and-mul with routed MXFP8 quantization and scale packing."""
    rows, inter = _check_silu_input(input)
    _check_offsets(expert_offsets, input.device, "expert_offsets")
    if scale_offsets is not None:
        _check_offsets(scale_offsets, input.device, "scale_offsets")
        if scale_offsets.shape != expert_offsets.shape:
            raise ValueError("scale_offsets must have E+1 entries")
    _require_sm100(input.device)
    load_library()
    experts = expert_offsets.numel() - 1
    if scale_offsets is None:
        scale_offsets = torch.empty_like(expert_offsets)
        with torch.cuda.device(input.device):
            check(
                library().mxfp6_grouped_scale_offsets(
                    expert_offsets.data_ptr(), experts, scale_offsets.data_ptr(),
                    _stream(input.device),
                )
            )
    values = torch.empty((rows, inter), dtype=torch.uint8, device=input.device)
    groups = (inter // SCALE_VECTOR_SIZE + 3) // 4 * 4
    scales = torch.full(
        (grouped_scale_rows(rows, experts) * groups,), 0x7F, dtype=torch.uint8, device=input.device
    )
    _silu_raw(input, values, None, scales, expert_offsets, scale_offsets)
    return values.view(torch.float8_e4m3fn), scales, scale_offsets


def silu_and_mul_mxfp8_grouped_out(
    output: torch.Tensor,
    scales: torch.Tensor,
    input: torch.Tensor,
    expert_offsets: torch.Tensor,
    scale_offsets: torch.Tensor,
    use_pdl: bool = False,
    grouped_output: torch.Tensor | None = None,
    weight: torch.Tensor | None = None,
    weight_scales: torch.Tensor | None = None,
) -> None:
    """Write grouped activation, optionally launching its W2 GEMM."""
    rows, inter = _check_silu_input(input)
    _check_offsets(expert_offsets, input.device, "expert_offsets")
    _check_offsets(scale_offsets, input.device, "scale_offsets")
    if _as_u8(output).shape != (rows, inter) or not output.is_contiguous():
        raise ValueError(f"output must be contiguous CUDA MXFP8 {(rows, inter)}")
    _require_cuda_uint8_contiguous(scales, "scales")
    fused = grouped_output is not None
    if fused != (weight is not None) or fused != (weight_scales is not None):
        raise ValueError("grouped_output, weight, and weight_scales must be provided together")
    _require_sm100(input.device)
    load_library()
    _silu_raw(input, _as_u8(output), None, scales, expert_offsets, scale_offsets)
    if fused:
        grouped_gemm_w6a8_out(
            grouped_output, output, scales, weight, weight_scales, expert_offsets, scale_offsets
        )


# ------------------------------------------------------------------------------ routing


def _route_raw(activation, logical_scales, topk_ids, expert_map, local_experts, permuted,
               grouped_scales, cursors, expert_offsets, scale_offsets, inverse, source_tokens,
               include_shared=False):
    tokens, hidden = (int(v) for v in activation.shape)
    with torch.cuda.device(activation.device):
        check(
            library().mxfp6_moe_route_shared(
                _as_u8(activation).data_ptr(), logical_scales.data_ptr(), topk_ids.data_ptr(),
                int(topk_ids.dtype == torch.int64), tokens, int(topk_ids.shape[1]), hidden,
                _ptr(expert_map), 0 if expert_map is None else expert_map.numel(), local_experts,
                int(bool(include_shared)), expert_offsets.data_ptr(), scale_offsets.data_ptr(), cursors.data_ptr(),
                None if permuted is None else _as_u8(permuted).data_ptr(),
                grouped_scales.data_ptr(), inverse.data_ptr(), _ptr(source_tokens),
                _stream(activation.device),
            )
        )


def _check_route_inputs(activation, logical_scales, topk_ids) -> None:
    if (
        activation.device.type != "cuda"
        or activation.dtype not in (torch.float8_e4m3fn, torch.uint8)
        or activation.ndim != 2
        or not activation.is_contiguous()
        or activation.shape[1] % SCALE_VECTOR_SIZE
    ):
        raise ValueError(
            "activation must be contiguous CUDA float8_e4m3fn/uint8 [M,K] with K divisible by 32"
        )
    expected = (activation.shape[0], activation.shape[1] // SCALE_VECTOR_SIZE)
    if (
        logical_scales.device != activation.device
        or logical_scales.dtype != torch.uint8
        or tuple(logical_scales.shape) != expected
        or not logical_scales.is_contiguous()
    ):
        raise ValueError(f"logical_scales must be contiguous CUDA uint8 {expected}")
    if (
        topk_ids.device != activation.device
        or topk_ids.dtype not in (torch.int32, torch.int64)
        or topk_ids.ndim != 2
        or topk_ids.shape[0] != activation.shape[0]
        or not topk_ids.is_contiguous()
    ):
        raise ValueError("topk_ids must be contiguous CUDA int32/int64 [M,topk]")


def route_mxfp8_out(
    activation: torch.Tensor,
    logical_scales: torch.Tensor,
    topk_ids: torch.Tensor,
    expert_map: torch.Tensor | None,
    local_experts: int,
    permuted_activation: torch.Tensor,
    include_shared: bool = False,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Route MXFP8 rows into ``permuted_activation``.

    Returns ``(grouped_scales, expert_offsets, scale_offsets, inverse_permutation)``.
    ``expert_map`` (global id -> local id or -1) drops routes of experts that live
    on other ranks; their ``inverse_permutation`` entries are -1.  With ``include_shared``
    ``local_experts`` counts one trailing shared expert: its group holds every token once, in
    token order, after the routed rows (``permuted_activation`` then has ``M*topk + M`` rows;
    ``inverse_permutation`` keeps ``M*topk`` entries), as in the reference
    (python/mxfp6/ops.py:694-774, csrc/moe.cu:4449-4631).
    """
    _check_route_inputs(activation, logical_scales, topk_ids)
    include_shared = bool(include_shared)
    routes = activation.shape[0] * topk_ids.shape[1]
    total_rows = routes + (activation.shape[0] if include_shared else 0)
    if (
        permuted_activation.device != activation.device
        or permuted_activation.dtype != activation.dtype
        or tuple(permuted_activation.shape) != (total_rows, activation.shape[1])
        or not permuted_activation.is_contiguous()
    ):
        raise ValueError(
            f"permuted_activation must be contiguous {(total_rows, activation.shape[1])} "
            "with the activation dtype and device"
        )
    minimum_experts = 2 if include_shared else 1
    if not minimum_experts <= local_experts <= 1024:
        raise ValueError(
            f"local_experts must be in [{minimum_experts}, 1024] and include one trailing "
            "shared expert when include_shared is true"
        )
    if expert_map is not None and (
        expert_map.device != activation.device
        or expert_map.dtype != torch.int32
        or expert_map.ndim != 1
        or not expert_map.is_contiguous()
    ):
        raise ValueError("expert_map must be a contiguous CUDA int32 vector")
    _require_sm100(activation.device)
    load_library()
    device = activation.device
    groups = (activation.shape[1] // SCALE_VECTOR_SIZE + 3) // 4 * 4
    grouped_scales = torch.full(
        (grouped_scale_rows(total_rows, local_experts) * groups,), 0x7F, dtype=torch.uint8,
        device=device,
    )
    expert_offsets = torch.empty(local_experts + 1, dtype=torch.int64, device=device)
    scale_offsets = torch.empty(local_experts + 1, dtype=torch.int64, device=device)
    cursors = torch.empty(local_experts, dtype=torch.int32, device=device)
    inverse = torch.empty(routes, dtype=torch.int32, device=device)
    _route_raw(activation, logical_scales, topk_ids, expert_map, local_experts,
               permuted_activation, grouped_scales, cursors, expert_offsets, scale_offsets,
               inverse, None, include_shared)
    return grouped_scales, expert_offsets, scale_offsets, inverse


def qwen35_route_mxfp8_out(
    activation: torch.Tensor,
    logical_scales: torch.Tensor,
    topk_ids: torch.Tensor,
    permuted_activation: torch.Tensor,
    packed_scales: torch.Tensor,
    expert_cursors: torch.Tensor,
    expert_offsets: torch.Tensor,
    scale_offsets: torch.Tensor,
    inverse_permutation: torch.Tensor,
    include_shared: bool = False,
    source_tokens: torch.Tensor | None = None,
    expert_map: torch.Tensor | None = None,
) -> None:
    """Route MXFP8 rows into preallocated grouped buffers (allocation-free).

    ``expert_offsets`` / ``scale_offsets`` have one entry per local expert plus one; with
    ``include_shared`` the last expert is the shared one (python/mxfp6/ops.py:776-870), so the
    buffers are sized for ``M*topk + M`` rows and one more padded scale group.
    """
    _check_route_inputs(activation, logical_scales, topk_ids)
    include_shared = bool(include_shared)
    local_experts = expert_offsets.numel() - 1
    tokens, hidden = (int(v) for v in activation.shape)
    routes = tokens * int(topk_ids.shape[1])
    total_rows = routes + (tokens if include_shared else 0)
    if local_experts < (2 if include_shared else 1):
        raise ValueError("expert_offsets must hold one entry per local expert plus one, the "
                         "trailing shared expert included when include_shared is true")
    # capacities, not exact shapes: a workspace may hold larger buffers than one call needs
    groups = (hidden // SCALE_VECTOR_SIZE + 3) // 4 * 4
    active_experts = min(routes, local_experts - int(include_shared)) + int(include_shared)
    for tensor, dtype, need, name in (
        (expert_cursors, torch.int32, local_experts, "expert_cursors"),
        (scale_offsets, torch.int64, local_experts + 1, "scale_offsets"),
        (inverse_permutation, torch.int32, routes, "inverse_permutation"),
        (packed_scales, torch.uint8, (total_rows + active_experts * 127) * groups, "packed_scales"),
    ) + (() if source_tokens is None else ((source_tokens, torch.int32, total_rows, "source_tokens"),)) + (
        () if permuted_activation is None
        else ((permuted_activation, activation.dtype, total_rows * hidden, "permuted_activation"),)
    ):
        same_type = tensor.dtype == dtype or (
            name == "permuted_activation" and tensor.dtype in (torch.uint8, torch.float8_e4m3fn))
        if (tensor.device != activation.device or not same_type
                or tensor.numel() < need or not tensor.is_contiguous()):
            raise ValueError(f"{name} must be contiguous CUDA {dtype} with at least {need} values")
    _require_sm100(activation.device)
    load_library()
    _route_raw(activation, logical_scales, topk_ids, expert_map, local_experts,
               permuted_activation, packed_scales, expert_cursors, expert_offsets, scale_offsets,
               inverse_permutation, source_tokens, include_shared)


def qwen35_topk_quant_out(
    quantized: torch.Tensor,
    logical_scales: torch.Tensor,
    packed_scales: torch.Tensor | None,
    topk_weights: torch.Tensor,
    topk_ids: torch.Tensor,
    hidden: torch.Tensor,
    routed_logits: torch.Tensor,
    renormalize: bool = False,
) -> None:
    """Fuse softmax top-k routing with dual-layout MXFP8 quantization of ``hidden``
    (``packed_scales`` may be ``None`` when only the logical layout is wanted)."""
    if (
        hidden.device.type != "cuda"
        or hidden.dtype != torch.bfloat16
        or hidden.ndim != 2
        or hidden.shape[0] < 1
        or hidden.shape[1] % SCALE_VECTOR_SIZE
        or not hidden.is_contiguous()
    ):
        raise ValueError("hidden must be contiguous CUDA bfloat16 [B,H] with H divisible by 32")
    batch, width = (int(v) for v in hidden.shape)
    if (
        routed_logits.device != hidden.device
        or routed_logits.dtype != torch.bfloat16
        or routed_logits.ndim != 2
        or routed_logits.shape[0] != batch
        or not routed_logits.is_contiguous()
    ):
        raise ValueError("routed_logits must be contiguous CUDA bfloat16 [B,E]")
    experts = int(routed_logits.shape[1])
    topk = int(topk_ids.shape[1]) if topk_ids.ndim == 2 else 0
    expected = (
        (quantized, torch.uint8, (batch, width), "quantized"),
        (logical_scales, torch.uint8, (batch, width // SCALE_VECTOR_SIZE), "logical_scales"),
        (topk_weights, torch.float32, (batch, topk), "topk_weights"),
        (topk_ids, torch.int32, (batch, topk), "topk_ids"),
    )
    for tensor, dtype, shape, name in expected:
        if (
            tensor.device != hidden.device
            or _as_u8(tensor).dtype != dtype
            or tuple(tensor.shape) != shape
            or not tensor.is_contiguous()
        ):
            raise ValueError(f"{name} must be contiguous CUDA {dtype} {tuple(shape)}")
    if packed_scales is not None and (
        packed_scales.device != hidden.device
        or packed_scales.dtype != torch.uint8
        or packed_scales.numel() < packed_scale_numel(batch, width)
        or not packed_scales.is_contiguous()
    ):
        raise ValueError("packed_scales must be contiguous CUDA uint8 of the dense packed size")
    if not isinstance(renormalize, bool):
        raise TypeError("renormalize must be a bool")
    if not 1 <= topk <= 16 or not topk <= experts <= 1024:
        raise ValueError("need 1 <= topk <= 16 and topk <= experts <= 1024")
    _require_sm100(hidden.device)
    load_library()
    with torch.cuda.device(hidden.device):
        check(
            library().mxfp6_moe_topk_quant(
                hidden.data_ptr(), routed_logits.data_ptr(), batch, width, experts, topk,
                int(renormalize), _as_u8(quantized).data_ptr(), logical_scales.data_ptr(),
                _ptr(packed_scales), topk_weights.data_ptr(), topk_ids.data_ptr(),
                _stream(hidden.device),
            )
        )


def qwen35_topk_quant_route_out(
    quantized: torch.Tensor,
    logical_scales: torch.Tensor,
    dense_scales: torch.Tensor,
    topk_weights: torch.Tensor,
    topk_ids: torch.Tensor,
    permuted_activation: torch.Tensor,
    grouped_scales: torch.Tensor,
    expert_cursors: torch.Tensor,
    expert_offsets: torch.Tensor,
    scale_offsets: torch.Tensor,
    inverse_permutation: torch.Tensor,
    hidden: torch.Tensor,
    routed_logits: torch.Tensor,
    grouped_output: torch.Tensor | None = None,
    weight: torch.Tensor | None = None,
    weight_scales: torch.Tensor | None = None,
    source_tokens: torch.Tensor | None = None,
    renormalize: bool = False,
    expert_map: torch.Tensor | None = None,
) -> None:
    """Top-k routing + quantization + row permutation, optionally followed by the
    grouped W1 GEMM (``grouped_output``/``weight``/``weight_scales`` together).

    Rows are always materialised in ``permuted_activation``; ``source_tokens``,
    when given, additionally receives the token index of every routed row.
    """
    fused = grouped_output is not None
    if fused != (weight is not None) or fused != (weight_scales is not None):
        raise ValueError("grouped_output, weight, and weight_scales must be provided together")
    if (
        hidden.device.type != "cuda"
        or hidden.dtype != torch.bfloat16
        or hidden.ndim != 2
        or hidden.shape[1] % SCALE_VECTOR_SIZE
        or not hidden.is_contiguous()
    ):
        raise ValueError("hidden must be contiguous CUDA bfloat16 [B,H] with H divisible by 32")
    batch, width = (int(v) for v in hidden.shape)
    experts = int(routed_logits.shape[1])
    topk = int(topk_ids.shape[1])
    routes = batch * topk
    local_experts = expert_offsets.numel() - 1
    expected = (
        (quantized, (batch, width), "quantized"),
        (logical_scales, (batch, width // SCALE_VECTOR_SIZE), "logical_scales"),
        (topk_weights, (batch, topk), "topk_weights"),
        (topk_ids, (batch, topk), "topk_ids"),
        (routed_logits, (batch, experts), "routed_logits"),
        (permuted_activation, (routes, width), "permuted_activation"),
        (inverse_permutation, (routes,), "inverse_permutation"),
    )
    for tensor, shape, name in expected:
        if tensor.device != hidden.device or tuple(tensor.shape) != shape or not tensor.is_contiguous():
            raise ValueError(f"{name} must be contiguous CUDA {tuple(shape)}")
    if topk_ids.dtype != torch.int32 or topk_weights.dtype != torch.float32:
        raise ValueError("topk_ids must be int32 and topk_weights float32")
    if not isinstance(renormalize, bool):
        raise TypeError("renormalize must be a bool")
    _require_sm100(hidden.device)
    load_library()
    with torch.cuda.device(hidden.device):
        check(
            library().mxfp6_moe_topk_quant_route(
                hidden.data_ptr(), routed_logits.data_ptr(), batch, width, experts, topk,
                int(renormalize), _as_u8(quantized).data_ptr(), logical_scales.data_ptr(),
                dense_scales.data_ptr(), topk_weights.data_ptr(), topk_ids.data_ptr(),
                _ptr(expert_map), 0 if expert_map is None else expert_map.numel(), local_experts,
                expert_offsets.data_ptr(), scale_offsets.data_ptr(), expert_cursors.data_ptr(),
                _as_u8(permuted_activation).data_ptr(), grouped_scales.data_ptr(),
                inverse_permutation.data_ptr(), _ptr(source_tokens), _stream(hidden.device),
            )
        )
    if fused:
        grouped_gemm_w6a8_out(grouped_output, permuted_activation, grouped_scales, weight,
                              weight_scales, expert_offsets, scale_offsets)


# ------------------------------------------------------------------------ grouped GEMMs


def _check_grouped_operands(activation, activation_scales, weight, weight_scales, expert_offsets,
                            scale_offsets) -> tuple[int, int, int, int]:
    if (
        activation.device.type != "cuda"
        or activation.dtype not in (torch.float8_e4m3fn, torch.uint8)
        or activation.ndim != 2
        or not activation.is_contiguous()
    ):
        raise ValueError("activation must be contiguous CUDA float8_e4m3fn/uint8 [M,K]")
    _require_sm100(activation.device)
    for tensor, name in (
        (activation_scales, "activation_scales"),
        (weight, "weight"),
        (weight_scales, "weight_scales"),
    ):
        _require_cuda_uint8_contiguous(tensor, name)
        if tensor.device != activation.device:
            raise ValueError(f"{name} must be on {activation.device}")
    if weight.ndim != 3:
        raise ValueError("weight must have shape [E,N,packed_K]")
    for tensor, name in ((expert_offsets, "expert_offsets"), (scale_offsets, "scale_offsets")):
        if (
            tensor.device != activation.device
            or tensor.dtype != torch.int64
            or tensor.ndim != 1
            or not tensor.is_contiguous()
        ):
            raise ValueError(f"{name} must be a contiguous CUDA int64 tensor")
    experts, rows_per_expert, packed_k = (int(v) for v in weight.shape)
    k = packed_k * 4 // 3
    if int(activation.shape[1]) != k:
        raise ValueError(f"activation K {activation.shape[1]} does not match weight K {k}")
    if expert_offsets.numel() != experts + 1 or scale_offsets.numel() != experts + 1:
        raise ValueError("expert_offsets and scale_offsets must have E+1 entries")
    groups = (k // SCALE_VECTOR_SIZE + 3) // 4 * 4
    scale_rows = activation_scales.numel() // groups // 128 * 128
    return experts, rows_per_expert, k, scale_rows


def grouped_gemm_w6a8_out(
    output: torch.Tensor,
    activation: torch.Tensor,
    activation_scales: torch.Tensor,
    weight: torch.Tensor,
    weight_scales: torch.Tensor,
    expert_offsets: torch.Tensor,
    scale_offsets: torch.Tensor,
    tile_n: int = 0,
    use_pdl: bool = False,
) -> None:
    """Run native grouped ``A8 @ W6.T`` into a preallocated output.

    ``tile_n`` (the reference's tile selector) is accepted and ignored unless it is
    one of the token-tile sizes 64, 128, 192, 256 of the tcgen05 kernel.
    """
    experts, n, k, scale_rows = _check_grouped_operands(
        activation, activation_scales, weight, weight_scales, expert_offsets, scale_offsets
    )
    if (
        output.device != activation.device
        or output.dtype not in (torch.float16, torch.bfloat16)
        or output.ndim != 2
        or tuple(output.shape) != (activation.shape[0], n)
        or not output.is_contiguous()
    ):
        raise ValueError("output must be contiguous CUDA float16/bfloat16 [M,N]")
    load_library()
    tile = tile_n if tile_n in (64, 128, 192, 256) else 0
    with torch.cuda.device(activation.device):
        check(
            library().mxfp6_grouped_gemm_w6a8(
                output.data_ptr(), _DTYPE_CODE[output.dtype], _as_u8(activation).data_ptr(),
                activation_scales.data_ptr(), scale_rows, weight.data_ptr(),
                weight_scales.data_ptr(), expert_offsets.data_ptr(), scale_offsets.data_ptr(),
                experts, int(activation.shape[0]), n, k, tile, _stream(activation.device),
            )
        )


def grouped_gemm_w6a8(
    activation: torch.Tensor,
    activation_scales: torch.Tensor,
    weight: torch.Tensor,
    weight_scales: torch.Tensor,
    expert_offsets: torch.Tensor,
    scale_offsets: torch.Tensor,
    *,
    out_dtype: torch.dtype = torch.bfloat16,
) -> torch.Tensor:
    """Return native grouped ``A8 @ W6.T`` for routed MoE rows."""
    out_dtype = _validate_output_dtype(out_dtype)
    if weight.ndim != 3:
        raise ValueError("weight must have shape [E,N,packed_K]")
    output = torch.empty(
        (activation.shape[0], weight.shape[1]), device=activation.device, dtype=out_dtype
    )
    grouped_gemm_w6a8_out(
        output, activation, activation_scales, weight, weight_scales, expert_offsets, scale_offsets
    )
    return output


def qwen35_grouped_w1_silu_mxfp8_out(
    output: torch.Tensor,
    output_scales: torch.Tensor,
    activation: torch.Tensor,
    activation_scales: torch.Tensor,
    weight: torch.Tensor,
    weight_scales: torch.Tensor,
    expert_offsets: torch.Tensor,
    scale_offsets: torch.Tensor,
    use_pdl: bool = False,
    source_tokens: torch.Tensor | None = None,
    tile_tokens: int = 0,
) -> None:
    """Grouped W1 (gate rows, then up rows) with the fused SiLU*mul + MXFP8 epilogue.

    ``activation`` holds the permuted rows and ``activation_scales`` their grouped
    packed scales; ``output`` is E4M3 ``[rows, I]`` and ``output_scales`` the grouped
    packed scales of the result (same ``scale_offsets``).
    """
    if source_tokens is not None and activation.shape[0] != output.shape[0]:
        raise ValueError(
            "indirect rows are not supported: pass the permuted activation rows "
            "(qwen35_route_mxfp8_out writes them)"
        )
    experts, two_inter, k, scale_rows = _check_grouped_operands(
        activation, activation_scales, weight, weight_scales, expert_offsets, scale_offsets
    )
    inter = two_inter // 2
    if _as_u8(output).shape != (activation.shape[0], inter) or not output.is_contiguous():
        raise ValueError(f"output must be contiguous CUDA MXFP8 {(activation.shape[0], inter)}")
    _require_cuda_uint8_contiguous(output_scales, "output_scales")
    load_library()
    with torch.cuda.device(activation.device):
        check(
            library().mxfp6_w1_swiglu_mxfp8(
                _as_u8(output).data_ptr(), output_scales.data_ptr(), None,
                _as_u8(activation).data_ptr(), activation_scales.data_ptr(), scale_rows,
                weight.data_ptr(), weight_scales.data_ptr(), expert_offsets.data_ptr(),
                scale_offsets.data_ptr(), experts, int(activation.shape[0]), inter, k, tile_tokens,
                _stream(activation.device),
            )
        )


def dense_w1_silu_mxfp8_out(
    output: torch.Tensor,
    output_scales: torch.Tensor,
    activation: torch.Tensor,
    activation_scales: torch.Tensor,
    weight: torch.Tensor,
    weight_scales: torch.Tensor,
) -> None:
    """Dense W1 + fused SiLU*mul + MXFP8 (the shared expert's first projection).

    ``weight`` is packed ``[2I, K*3/4]`` (gate rows, then up rows); activation and
    output scales use the dense packed layout.
    """
    rows, k = (int(v) for v in activation.shape)
    inter = int(weight.numel()) // (k * 3 // 4) // 2
    _require_sm100(activation.device)
    load_library()
    groups = (k // SCALE_VECTOR_SIZE + 3) // 4 * 4
    with torch.cuda.device(activation.device):
        check(
            library().mxfp6_w1_swiglu_mxfp8(
                _as_u8(output).data_ptr(), output_scales.data_ptr(), None,
                _as_u8(activation).data_ptr(), activation_scales.data_ptr(),
                activation_scales.numel() // groups // 128 * 128, weight.data_ptr(),
                weight_scales.data_ptr(), None, None, 1, rows, inter, k, 0,
                _stream(activation.device),
            )
        )


# ------------------------------------------------------------------------------- reduce


def _check_reduce_operands(output, routed_output, topk_weights, inverse_permutation,
                           shared_output, shared_gate) -> int:
    """Argument checks of the reducers; returns the row length of the gate tensor."""
    if (
        routed_output.device.type != "cuda"
        or routed_output.dtype not in (torch.float16, torch.bfloat16)
        or routed_output.ndim != 2
        or not routed_output.is_contiguous()
    ):
        raise ValueError("routed_output must be contiguous CUDA float16/bfloat16 [routes,H]")
    if (
        output.device != routed_output.device
        or output.dtype != routed_output.dtype
        or output.ndim != 2
        or not output.is_contiguous()
    ):
        raise ValueError("output must be contiguous CUDA [tokens,H] with routed_output's dtype")
    if (
        topk_weights.device != routed_output.device
        or topk_weights.dtype != torch.float32
        or topk_weights.ndim != 2
        or not topk_weights.is_contiguous()
    ):
        raise ValueError("topk_weights must be contiguous CUDA float32 [tokens,topk]")
    if (
        inverse_permutation.device != routed_output.device
        or inverse_permutation.dtype != torch.int32
        or inverse_permutation.ndim != 1
        or not inverse_permutation.is_contiguous()
    ):
        raise ValueError("inverse_permutation must be a contiguous CUDA int32 vector")
    if shared_output is not None and (
        shared_output.device != routed_output.device
        or shared_output.dtype != routed_output.dtype
        or shared_output.shape != output.shape
        or not shared_output.is_contiguous()
    ):
        raise ValueError(
            "shared_output must be contiguous and match output's device, dtype, and shape"
        )
    gate_stride = 1
    if shared_gate is not None:
        if (
            shared_output is None
            or shared_gate.device != routed_output.device
            or shared_gate.dtype not in _GATE_CODE
            or not shared_gate.is_contiguous()
            or (
                shared_gate.numel() != output.shape[0]
                and (shared_gate.ndim != 2 or shared_gate.shape[0] != output.shape[0])
            )
        ):
            raise ValueError(
                "shared_gate requires shared_output and one contiguous floating "
                "value or row per token"
            )
        gate_stride = shared_gate.numel() // output.shape[0]
    return gate_stride


def moe_reduce_out(
    output: torch.Tensor,
    routed_output: torch.Tensor,
    topk_weights: torch.Tensor,
    inverse_permutation: torch.Tensor,
    shared_output: torch.Tensor | None = None,
    shared_gate: torch.Tensor | None = None,
    use_pdl: bool = False,
) -> None:
    """Reduce routed rows and optionally gate/add a shared-expert output."""
    gate_stride = _check_reduce_operands(output, routed_output, topk_weights, inverse_permutation,
                                         shared_output, shared_gate)
    load_library()
    tokens, hidden = (int(v) for v in output.shape)
    with torch.cuda.device(output.device):
        check(
            library().mxfp6_moe_reduce(
                output.data_ptr(), routed_output.data_ptr(), _DTYPE_CODE[output.dtype],
                topk_weights.data_ptr(), inverse_permutation.data_ptr(), _ptr(shared_output),
                _ptr(shared_gate), 0 if shared_gate is None else _GATE_CODE[shared_gate.dtype],
                gate_stride, tokens, hidden, int(topk_weights.shape[1]),
                int(routed_output.shape[0]), _stream(output.device),
            )
        )


def moe_reduce_tp2_out(
    output: torch.Tensor,
    routed_output: torch.Tensor,
    topk_weights: torch.Tensor,
    inverse_permutation: torch.Tensor,
    shared_output: torch.Tensor | None = None,
    shared_gate: torch.Tensor | None = None,
    signal_ptrs: list[int] | None = None,
    buffer_ptrs: list[int] | None = None,
    rank: int | None = None,
    *,
    group=None,
    peer=None,
) -> None:
    """Reduce, then sum the result over the tensor-parallel ranks.

    With ``signal_ptrs`` / ``buffer_ptrs`` / ``rank`` this is the reference's call
    (python/mxfp6/ops.py:950-1025, kernel csrc/moe.cu:7698-7925): the pointers of every
    rank's signal area (64 zero-initialised bytes at least) and data buffer, as a
    custom all-reduce hands them out, for 2 ranks as in the reference or up to 8.  The
    partial goes into this rank's buffer, one kernel sums all ranks' partials over peer
    memory in rank order with bounded waits (the reference spins without a limit), and a
    closing handshake makes the buffer safe to rewrite.  BF16 only, like the reference.

    Without the pointer lists: with ``peer`` (a ``tp_fused.SymmetricBlocks``) the partial goes
    into this rank's symmetric block and the same kernel sums over the blocks; without it an
    NCCL all-reduce follows the reduce kernel.
    """
    import torch.distributed as dist

    if signal_ptrs is not None or buffer_ptrs is not None or rank is not None:
        if signal_ptrs is None or buffer_ptrs is None or rank is None:
            raise ValueError("signal_ptrs, buffer_ptrs and rank go together")
        world = len(signal_ptrs)
        if world != len(buffer_ptrs) or not 1 <= world <= 8 or not 0 <= int(rank) < world:
            raise ValueError("the fused reduce requires one signal and one buffer pointer per rank "
                             "(at most 8) and a rank among them")
        if output.dtype != torch.bfloat16 or routed_output.dtype != torch.bfloat16:
            raise ValueError("routed_output and output must be contiguous CUDA bfloat16")
        if shared_output is None or shared_gate is None:
            raise ValueError("shared_output and shared_gate are required")
        # the argument checks of the plain reduce, without launching it
        _check_reduce_operands(output, routed_output, topk_weights, inverse_permutation,
                               shared_output, shared_gate)
        _require_sm100(output.device)
        load_library()
        tokens, hidden = (int(v) for v in output.shape)
        signals = (ctypes.c_uint64 * world)(*[int(v) for v in signal_ptrs])
        buffers = (ctypes.c_uint64 * world)(*[int(v) for v in buffer_ptrs])
        with torch.cuda.device(output.device):
            check(
                library().mxfp6_moe_reduce_tp_pointers(
                    output.data_ptr(), routed_output.data_ptr(), topk_weights.data_ptr(),
                    inverse_permutation.data_ptr(), shared_output.data_ptr(), shared_gate.data_ptr(),
                    _GATE_CODE[shared_gate.dtype], shared_gate.numel() // tokens, tokens, hidden,
                    int(topk_weights.shape[1]), int(routed_output.shape[0]), signals, buffers, world,
                    int(rank), _stream(output.device),
                )
            )
        return
    if peer is not None and peer.world > 1:
        rows, hidden = (int(v) for v in output.shape)
        partial = peer.next_partial(rows, hidden)
        moe_reduce_out(partial, routed_output, topk_weights, inverse_permutation, shared_output,
                       shared_gate)
        peer.allreduce(output)
        return
    moe_reduce_out(output, routed_output, topk_weights, inverse_permutation, shared_output,
                   shared_gate)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(output, group=group)


# ------------------------------------------------- decode batches: one GEMM per route
#
# Route r = token * lanes + lane with lanes = topk + include_shared; the expert of a
# routed lane is ``topk_ids[token, lane]``, the lane after the last routed one is the
# always-on shared expert (the LAST matrix of the weight stack, or a separate one).
# These are the reference's "array" and split-K operators (python/mxfp6/ops.py:1143-1241,
# 1553-1950); here they are generic in hidden size, intermediate size and expert count.


def _check_route_operands(activation, logical_scales, weight, weight_scales, topk_ids):
    if (
        activation.device.type != "cuda"
        or activation.dtype not in (torch.float8_e4m3fn, torch.uint8)
        or activation.ndim != 2
        or not activation.is_contiguous()
    ):
        raise ValueError("activation must be contiguous CUDA float8_e4m3fn/uint8 [M,K]")
    _require_sm100(activation.device)
    for tensor, name in ((logical_scales, "logical_scales"), (weight, "weight"),
                         (weight_scales, "weight_scales")):
        _require_cuda_uint8_contiguous(tensor, name)
        if tensor.device != activation.device:
            raise ValueError(f"{name} must be on {activation.device}")
    if (
        topk_ids.device != activation.device
        or topk_ids.dtype not in (torch.int32, torch.int64)
        or topk_ids.ndim != 2
        or not topk_ids.is_contiguous()
    ):
        raise ValueError("topk_ids must be contiguous CUDA int32/int64 [tokens,topk]")
    if weight.ndim != 3:
        raise ValueError("weight must have shape [E,N,packed_K]")
    k = int(activation.shape[1])
    if int(weight.shape[2]) * 4 != k * 3:
        raise ValueError("activation K does not match packed weight K")
    if tuple(logical_scales.shape) != (int(activation.shape[0]), k // SCALE_VECTOR_SIZE):
        raise ValueError("logical_scales must have shape [activation_rows,K/32]")
    return k


def _check_separate_shared(shared_weight, shared_weight_scales, weight, device):
    if (shared_weight is None) != (shared_weight_scales is None):
        raise ValueError("shared_weight and shared_weight_scales must be provided together")
    if shared_weight is None:
        return
    for tensor, name in ((shared_weight, "shared_weight"), (shared_weight_scales, "shared_weight_scales")):
        _require_cuda_uint8_contiguous(tensor, name)
        if tensor.device != device:
            raise ValueError(f"{name} must be on {device}")
    if shared_weight.ndim != 3 or tuple(shared_weight.shape) != (1, *weight.shape[1:]):
        raise ValueError("shared_weight must be contiguous CUDA uint8 [1,N,packed_K]")


def array_gemm_w6a8_out(
    output: torch.Tensor,
    activation: torch.Tensor,
    logical_scales: torch.Tensor,
    weight: torch.Tensor,
    weight_scales: torch.Tensor,
    topk_ids: torch.Tensor,
    include_shared: bool = False,
) -> None:
    """Run equal-shape route GEMMs, optionally appending a shared route."""
    k = _check_route_operands(activation, logical_scales, weight, weight_scales, topk_ids)
    tokens, topk = (int(v) for v in topk_ids.shape)
    routes = tokens * (topk + int(include_shared))
    n = int(weight.shape[1])
    if (
        output.device != activation.device
        or output.dtype not in (torch.float16, torch.bfloat16)
        or output.ndim != 2
        or not output.is_contiguous()
    ):
        raise ValueError("output must be contiguous CUDA float16/bfloat16 [routes,N]")
    if tuple(output.shape) != (routes, n):
        raise ValueError("output must contain all routed/shared rows")
    if int(activation.shape[0]) not in (tokens, routes):
        raise ValueError("activation rows must equal tokens or all routed/shared rows")
    load_library()
    with torch.cuda.device(activation.device):
        check(
            library().mxfp6_array_gemm_w6a8(
                output.data_ptr(), _DTYPE_CODE[output.dtype], _as_u8(activation).data_ptr(),
                logical_scales.data_ptr(), int(activation.shape[0]), weight.data_ptr(),
                weight_scales.data_ptr(), int(weight.shape[0]), topk_ids.data_ptr(),
                int(topk_ids.dtype == torch.int64), tokens, topk, int(include_shared), n, k,
                _stream(activation.device),
            )
        )


def array_gemm_w6a8_silu_mxfp8_out(
    output: torch.Tensor,
    output_scales: torch.Tensor,
    activation: torch.Tensor,
    logical_scales: torch.Tensor,
    weight: torch.Tensor,
    weight_scales: torch.Tensor,
    topk_ids: torch.Tensor,
    include_shared: bool = False,
    shared_weight: torch.Tensor | None = None,
    shared_weight_scales: torch.Tensor | None = None,
) -> None:
    """Fuse route W6A8 gate/up GEMM, SiLU multiply, and MXFP8 quantization.

    ``weight`` is ``[E, 2I, packed_K]`` (gate rows, then up rows); ``output`` is E4M3
    ``[routes, I]`` and ``output_scales`` logical UE8M0 ``[routes, I/32]``.
    """
    k = _check_route_operands(activation, logical_scales, weight, weight_scales, topk_ids)
    _check_separate_shared(shared_weight, shared_weight_scales, weight, activation.device)
    tokens, topk = (int(v) for v in topk_ids.shape)
    routes = tokens * (topk + int(include_shared))
    inter = int(weight.shape[1]) // 2
    for tensor, name in ((output, "output"), (output_scales, "output_scales")):
        _require_cuda_uint8_contiguous(_as_u8(tensor), name)
        if tensor.device != activation.device:
            raise ValueError(f"{name} must be on {activation.device}")
    if tuple(output.shape) != (routes, inter) or tuple(output_scales.shape) != (routes, inter // 32):
        raise ValueError("output must be [routes,I] and output_scales [routes,I/32]")
    if int(activation.shape[0]) not in (tokens, routes):
        raise ValueError("activation rows must equal tokens or all routed/shared rows")
    load_library()
    with torch.cuda.device(activation.device):
        check(
            library().mxfp6_array_gemm_w6a8_silu_mxfp8(
                _as_u8(output).data_ptr(), output_scales.data_ptr(), _as_u8(activation).data_ptr(),
                logical_scales.data_ptr(), int(activation.shape[0]), weight.data_ptr(),
                weight_scales.data_ptr(), int(weight.shape[0]), _ptr(shared_weight),
                _ptr(shared_weight_scales), topk_ids.data_ptr(),
                int(topk_ids.dtype == torch.int64), tokens, topk, int(include_shared), inter, k,
                _stream(activation.device),
            )
        )


def qwen35_w1_splitk_silu_mxfp8_out(
    output: torch.Tensor,
    output_scales: torch.Tensor,
    partial: torch.Tensor | None,
    activation: torch.Tensor,
    logical_scales: torch.Tensor,
    weight: torch.Tensor,
    weight_scales: torch.Tensor,
    topk_ids: torch.Tensor,
    include_shared: bool = True,
    shared_weight: torch.Tensor | None = None,
    shared_weight_scales: torch.Tensor | None = None,
) -> None:
    """Small-batch split-K W1 with the fused SiLU / MXFP8 epilogue.

    One activation row per token (``activation`` is ``[B, K]``); K is split over the CTAs
    of a thread-block cluster and reduced through distributed shared memory, so
    ``partial`` (the reference's global split-K scratch) is accepted and not used.
    """
    if not isinstance(include_shared, bool):
        raise TypeError("include_shared must be a bool")
    if int(activation.shape[0]) != int(topk_ids.shape[0]):
        raise ValueError("activation must hold one row per token")
    array_gemm_w6a8_silu_mxfp8_out(output, output_scales, activation, logical_scales, weight,
                                   weight_scales, topk_ids, include_shared, shared_weight,
                                   shared_weight_scales)


def _gate_stride(shared_gate: torch.Tensor, tokens: int, device) -> int:
    if (
        shared_gate.device != device
        or shared_gate.dtype not in _GATE_CODE
        or not shared_gate.is_contiguous()
        or (shared_gate.numel() != tokens and (shared_gate.ndim != 2 or shared_gate.shape[0] != tokens))
    ):
        raise ValueError("shared_gate must contain one contiguous floating value or row per token")
    return shared_gate.numel() // tokens


def array_gemm_w6a8_reduce_out(
    output: torch.Tensor,
    activation: torch.Tensor,
    logical_scales: torch.Tensor,
    weight: torch.Tensor,
    weight_scales: torch.Tensor,
    topk_ids: torch.Tensor,
    topk_weights: torch.Tensor,
    shared_gate: torch.Tensor,
    shared_output: torch.Tensor | None = None,
    shared_weight: torch.Tensor | None = None,
    shared_weight_scales: torch.Tensor | None = None,
    use_packed_vector_loads: bool = False,
    routing_ready: bool = False,
) -> None:
    """Route W2 GEMMs fused with the weighted reduce and the gated shared expert.

    ``activation`` is ``[tokens * 9, K]`` (eight routed rows and the shared row per token)
    or ``[tokens * 8, K]`` when ``shared_output`` brings the shared expert's rows.
    ``use_packed_vector_loads`` selects a load path of the reference's kernel and has no
    counterpart here.  ``routing_ready=True`` (not in the reference) vouches that ``topk_ids``
    were complete before the kernel preceding this one let its dependents start, as they are
    behind ``array_gemm_w6a8_silu_mxfp8_out``; the weights are then fetched ahead of the
    dependency wait.
    """
    k = _check_route_operands(activation, logical_scales, weight, weight_scales, topk_ids)
    _check_separate_shared(shared_weight, shared_weight_scales, weight, activation.device)
    tokens, topk = (int(v) for v in topk_ids.shape)
    if (
        topk_weights.device != activation.device
        or topk_weights.dtype != torch.float32
        or not topk_weights.is_contiguous()
        or topk_weights.shape != topk_ids.shape
    ):
        raise ValueError("topk_weights must be contiguous CUDA float32 [tokens,topk]")
    if (
        output.device != activation.device
        or output.dtype not in (torch.float16, torch.bfloat16)
        or output.ndim != 2
        or not output.is_contiguous()
        or tuple(output.shape) != (tokens, int(weight.shape[1]))
    ):
        raise ValueError("output must be contiguous CUDA float16/bfloat16 [tokens,N]")
    external = shared_output is not None
    if external and shared_weight is not None:
        raise ValueError("separate shared weights cannot be combined with shared_output")
    if external and (
        shared_output.device != activation.device
        or shared_output.dtype != output.dtype
        or shared_output.shape != output.shape
        or not shared_output.is_contiguous()
    ):
        raise ValueError(
            "shared_output must be contiguous and match output's shape, dtype, and CUDA device")
    lanes = topk + (0 if external else 1)
    if int(activation.shape[0]) != tokens * lanes:
        raise ValueError(f"activation must have shape [tokens*({topk} or {topk + 1}),K]")
    stride = _gate_stride(shared_gate, tokens, activation.device)
    load_library()
    with torch.cuda.device(activation.device):
        check(
            library().mxfp6_array_gemm_w6a8_reduce(
                output.data_ptr(), _DTYPE_CODE[output.dtype], _as_u8(activation).data_ptr(),
                logical_scales.data_ptr(), weight.data_ptr(), weight_scales.data_ptr(),
                int(weight.shape[0]), _ptr(shared_weight), _ptr(shared_weight_scales),
                topk_ids.data_ptr(), int(topk_ids.dtype == torch.int64), topk_weights.data_ptr(),
                shared_gate.data_ptr(), _GATE_CODE[shared_gate.dtype], stride, _ptr(shared_output),
                0 if external else 1, tokens, topk, int(weight.shape[1]), k, int(routing_ready),
                _stream(activation.device),
            )
        )


def qwen35_w2_splitk_reduce_out(
    output: torch.Tensor,
    partial: torch.Tensor | None,
    activation: torch.Tensor,
    logical_scales: torch.Tensor,
    weight: torch.Tensor,
    weight_scales: torch.Tensor,
    topk_ids: torch.Tensor,
    topk_weights: torch.Tensor,
    shared_gate: torch.Tensor,
    shared_weight: torch.Tensor | None = None,
    shared_weight_scales: torch.Tensor | None = None,
    routing_ready: bool = False,
) -> None:
    """Small-batch W2 with the weighted reduce and the gated shared row in its epilogue.

    The lanes of a token are split over the CTAs of a cluster and every lane accumulates
    in tensor memory, so ``partial`` (the reference's split-K scratch) is accepted and not
    used.
    """
    array_gemm_w6a8_reduce_out(output, activation, logical_scales, weight, weight_scales, topk_ids,
                               topk_weights, shared_gate, None, shared_weight, shared_weight_scales,
                               routing_ready=routing_ready)


def moe_reduce_array_out(
    output: torch.Tensor,
    combined_output: torch.Tensor,
    topk_weights: torch.Tensor,
    shared_gate: torch.Tensor,
) -> None:
    """Reduce interleaved routed/shared rows emitted by the array path."""
    if (
        combined_output.device.type != "cuda"
        or combined_output.dtype not in (torch.float16, torch.bfloat16)
        or combined_output.ndim != 2
        or not combined_output.is_contiguous()
    ):
        raise ValueError(
            "combined_output must be contiguous CUDA float16/bfloat16 [tokens*(topk+1),H]")
    if (
        output.device != combined_output.device
        or output.dtype != combined_output.dtype
        or output.ndim != 2
        or not output.is_contiguous()
    ):
        raise ValueError("output must be contiguous CUDA [tokens,H] with combined_output's dtype")
    if (
        topk_weights.device != combined_output.device
        or topk_weights.dtype != torch.float32
        or topk_weights.ndim != 2
        or not topk_weights.is_contiguous()
    ):
        raise ValueError("topk_weights must be contiguous CUDA float32 [tokens,topk]")
    tokens, hidden = (int(v) for v in output.shape)
    topk = int(topk_weights.shape[1])
    if tuple(combined_output.shape) != (tokens * (topk + 1), hidden) or int(topk_weights.shape[0]) != tokens:
        raise ValueError("combined_output must have shape [tokens*(topk+1),H]")
    _require_sm100(output.device)
    stride = _gate_stride(shared_gate, tokens, output.device)
    load_library()
    with torch.cuda.device(output.device):
        check(
            library().mxfp6_moe_reduce_array(
                output.data_ptr(), combined_output.data_ptr(), _DTYPE_CODE[output.dtype],
                topk_weights.data_ptr(), shared_gate.data_ptr(), _GATE_CODE[shared_gate.dtype],
                stride, tokens, topk, hidden, _stream(output.device),
            )
        )


def router_logits_out(
    routed_logits: torch.Tensor,
    shared_gate: torch.Tensor,
    hidden: torch.Tensor,
    gate_weight: torch.Tensor,
    shared_gate_weight: torch.Tensor | None = None,
) -> None:
    """The router GEMV alone: ``routed_logits[b, e] = bf16(hidden[b] . gate_weight[e])`` in FP32
    and the shared expert's gate logit into ``shared_gate[b]`` (the first half of
    ``qwen35_router_quant_out``)."""
    if (
        hidden.device.type != "cuda"
        or hidden.dtype != torch.bfloat16
        or hidden.ndim != 2
        or not hidden.is_contiguous()
        or hidden.shape[1] % 32
    ):
        raise ValueError("hidden must be contiguous CUDA bfloat16 [B,H] with H divisible by 32")
    _require_sm100(hidden.device)
    batch, width = (int(v) for v in hidden.shape)
    experts = int(routed_logits.shape[1])
    gate_rows = experts if shared_gate_weight is not None else experts + 1
    if (
        gate_weight.device != hidden.device
        or gate_weight.dtype != torch.bfloat16
        or tuple(gate_weight.shape) != (gate_rows, width)
        or not gate_weight.is_contiguous()
    ):
        raise ValueError(f"gate_weight must be contiguous CUDA bfloat16 [{gate_rows},{width}]")
    if shared_gate_weight is not None and (
        shared_gate_weight.device != hidden.device
        or shared_gate_weight.dtype != torch.bfloat16
        or tuple(shared_gate_weight.shape) != (1, width)
        or not shared_gate_weight.is_contiguous()
    ):
        raise ValueError(f"shared_gate_weight must be contiguous CUDA bfloat16 [1,{width}]")
    if (
        routed_logits.device != hidden.device
        or routed_logits.dtype != torch.bfloat16
        or tuple(routed_logits.shape) != (batch, experts)
        or not routed_logits.is_contiguous()
    ):
        raise ValueError("routed_logits must be contiguous CUDA bfloat16 [B,E]")
    if (
        shared_gate.device != hidden.device
        or shared_gate.dtype != torch.bfloat16
        or shared_gate.numel() != batch
        or not shared_gate.is_contiguous()
    ):
        raise ValueError("shared_gate must be contiguous CUDA bfloat16 with B values")
    load_library()
    with torch.cuda.device(hidden.device):
        check(
            library().mxfp6_moe_router_logits(
                hidden.data_ptr(), gate_weight.data_ptr(), _ptr(shared_gate_weight),
                routed_logits.data_ptr(), shared_gate.data_ptr(), batch, width, experts, gate_rows,
                _stream(hidden.device),
            )
        )


def qwen35_router_quant_out(
    quantized: torch.Tensor,
    logical_scales: torch.Tensor,
    routed_logits: torch.Tensor,
    topk_weights: torch.Tensor,
    topk_ids: torch.Tensor,
    shared_gate: torch.Tensor,
    hidden: torch.Tensor,
    gate_weight: torch.Tensor,
    renormalize: bool = False,
    shared_gate_weight: torch.Tensor | None = None,
) -> None:
    """Router GEMV, softmax top-k and MXFP8 quantization of the hidden rows.

    ``gate_weight`` holds the routed gate rows ``[E, H]`` followed by the shared expert's
    gate row (``[E + 1, H]``) unless ``shared_gate_weight`` ``[1, H]`` brings that row.
    Two launches here (the logits, then top-k + quantization) where the reference has one
    cooperative kernel.
    """
    if not isinstance(renormalize, bool):
        raise TypeError("renormalize must be a bool")
    router_logits_out(routed_logits, shared_gate, hidden, gate_weight, shared_gate_weight)
    qwen35_topk_quant_out(quantized, logical_scales, None, topk_weights, topk_ids, hidden,
                          routed_logits, renormalize=renormalize)


def moe_decode_layer_supported(tokens: int, topk: int, experts: int, hidden_size: int,
                               intermediate: int) -> bool:
    """Whether :func:`moe_decode_layer_out` takes the problem (host arithmetic, no GPU)."""
    load_library()
    return bool(library().mxfp6_moe_decode_layer_supported(int(tokens), int(topk), int(experts),
                                                           int(hidden_size), int(intermediate)))


def moe_decode_layer_preferred(tokens: int, topk: int, experts: int, hidden_size: int,
                               intermediate: int) -> bool:
    """Whether the two-launch form is supported AND expected to be the faster one."""
    load_library()
    return bool(library().mxfp6_moe_decode_layer_preferred(int(tokens), int(topk), int(experts),
                                                           int(hidden_size), int(intermediate)))


def moe_decode_layer_out(
    output: torch.Tensor,
    activation: torch.Tensor,
    activation_scales: torch.Tensor,
    topk_weights: torch.Tensor,
    topk_ids: torch.Tensor,
    hidden: torch.Tensor,
    router_logits: torch.Tensor,
    shared_gate: torch.Tensor,
    w1: torch.Tensor,
    w1_scales: torch.Tensor,
    w2: torch.Tensor,
    w2_scales: torch.Tensor,
    shared_w1: torch.Tensor | None = None,
    shared_w1_scales: torch.Tensor | None = None,
    shared_w2: torch.Tensor | None = None,
    shared_w2_scales: torch.Tensor | None = None,
    renormalize: bool = True,
    w2_own_routing: bool = False,
) -> None:
    """The decode schedule in two launches: top-k selection and MXFP8 quantization of the hidden
    rows happen inside the W1 kernel's CTAs, so no front-end kernel runs and W1 depends on
    nothing but ``hidden`` and ``router_logits``.

    Same results as ``qwen35_topk_quant_out`` -> ``qwen35_w1_splitk_silu_mxfp8_out`` ->
    ``qwen35_w2_splitk_reduce_out`` (the reference's schedule, python/mxfp6/qwen35.py:384-432).
    ``w1`` ``[E(+1), 2I, 3H/4]``, ``w2`` ``[E(+1), H, 3I/4]``; the shared expert is the last
    matrix of both unless the four ``shared_*`` tensors bring it.  ``activation``
    ``[tokens * (topk + 1), I]`` and ``activation_scales`` are scratch.  W2 reads the ids and
    weights W1 wrote; ``w2_own_routing=True`` makes it select again for itself before its
    dependency wait and fetch weights meanwhile (same bytes; it pays only while W2's CTAs fit
    on the GPU beside W1's).
    """
    if (
        hidden.device.type != "cuda"
        or hidden.dtype != torch.bfloat16
        or hidden.ndim != 2
        or not hidden.is_contiguous()
    ):
        raise ValueError("hidden must be contiguous CUDA bfloat16 [tokens,H]")
    _require_sm100(hidden.device)
    tokens, width = (int(v) for v in hidden.shape)
    if (
        router_logits.device != hidden.device
        or router_logits.dtype != torch.bfloat16
        or router_logits.ndim != 2
        or int(router_logits.shape[0]) != tokens
        or not router_logits.is_contiguous()
    ):
        raise ValueError("router_logits must be contiguous CUDA bfloat16 [tokens,E]")
    experts = int(router_logits.shape[1])
    topk = int(topk_ids.shape[1])
    for tensor, name in ((w1, "w1"), (w1_scales, "w1_scales"), (w2, "w2"), (w2_scales, "w2_scales")):
        _require_cuda_uint8_contiguous(tensor, name)
        if tensor.device != hidden.device:
            raise ValueError(f"{name} must be on {hidden.device}")
    if w1.ndim != 3 or w2.ndim != 3 or int(w1.shape[2]) * 4 != width * 3 or int(w2.shape[1]) != width:
        raise ValueError("w1 must be [E,2I,3H/4] and w2 [E,H,3I/4]")
    inter = int(w1.shape[1]) // 2
    if int(w2.shape[2]) * 4 != inter * 3 or w1.shape[0] != w2.shape[0]:
        raise ValueError("w1 and w2 disagree on the intermediate size or the expert count")
    shared = (shared_w1, shared_w1_scales, shared_w2, shared_w2_scales)
    if any(t is None for t in shared) != all(t is None for t in shared):
        raise ValueError("the separate shared expert comes as four tensors or none")
    if shared_w1 is not None:
        _check_separate_shared(shared_w1, shared_w1_scales, w1, hidden.device)
        _check_separate_shared(shared_w2, shared_w2_scales, w2, hidden.device)
    lanes = tokens * (topk + 1)
    if (
        topk_ids.dtype != torch.int32
        or topk_weights.dtype != torch.float32
        or tuple(topk_weights.shape) != (tokens, topk)
        or tuple(topk_ids.shape) != (tokens, topk)
        or not topk_ids.is_contiguous()
        or not topk_weights.is_contiguous()
    ):
        raise ValueError("topk_ids int32 and topk_weights float32 must be contiguous [tokens,topk]")
    if tuple(activation.shape) != (lanes, inter) or tuple(activation_scales.shape) != (lanes, inter // 32):
        raise ValueError("activation must be [tokens*(topk+1),I] and activation_scales [..,I/32]")
    if (
        output.device != hidden.device
        or output.dtype not in (torch.float16, torch.bfloat16)
        or tuple(output.shape) != (tokens, width)
        or not output.is_contiguous()
    ):
        raise ValueError("output must be contiguous CUDA float16/bfloat16 [tokens,H]")
    stride = _gate_stride(shared_gate, tokens, hidden.device)
    if not isinstance(renormalize, bool):
        raise TypeError("renormalize must be a bool")
    load_library()
    with torch.cuda.device(hidden.device):
        check(
            library().mxfp6_moe_decode_layer(
                output.data_ptr(), _DTYPE_CODE[output.dtype], hidden.data_ptr(),
                router_logits.data_ptr(), shared_gate.data_ptr(), _GATE_CODE[shared_gate.dtype], stride,
                w1.data_ptr(), w1_scales.data_ptr(), w2.data_ptr(), w2_scales.data_ptr(),
                int(w1.shape[0]), _ptr(shared_w1), _ptr(shared_w1_scales), _ptr(shared_w2),
                _ptr(shared_w2_scales), _as_u8(activation).data_ptr(), activation_scales.data_ptr(),
                topk_ids.data_ptr(), topk_weights.data_ptr(), tokens, topk, experts, int(renormalize),
                width, inter, int(bool(w2_own_routing)), _stream(hidden.device),
            )
        )
