"""Allocation-free routed-MoE schedules and their scratch workspaces.

Follows the reference's ``python/mxfp6/qwen35.py`` (workspace carved out of
caller-owned storage, one call per layer, capturable in one CUDA graph) with two
differences: the sizes (hidden, intermediate, experts, k) are parameters with the
reference model's values as defaults instead of module constants, and the
decode schedule (one single-row GEMM per route) takes any small batch, not one token.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .moe_ops import (
    dense_w1_silu_mxfp8_out,
    grouped_gemm_w6a8_out,
    grouped_scale_rows,
    moe_decode_layer_out,
    moe_decode_layer_preferred,
    moe_reduce_out,
    qwen35_grouped_w1_silu_mxfp8_out,
    qwen35_route_mxfp8_out,
    qwen35_topk_quant_out,
    qwen35_topk_quant_route_out,
    qwen35_router_quant_out,
    router_logits_out,
    qwen35_w1_splitk_silu_mxfp8_out,
    qwen35_w2_splitk_reduce_out,
    silu_and_mul_mxfp8_grouped_out,
)
from .ops import MXFP8Tensor, PackedMXFP6Tensor, gemm_w6a8, packed_scale_numel, quantize_mxfp8_logical

_HIDDEN_SIZE = 2048
_INTERMEDIATE_SIZE = 512
_NUM_EXPERTS = 256
_TOPK = 8
_SCALE_ROWS_PER_ATOM = 128


def _align_up(value: int, alignment: int) -> int:
    return (value + alignment - 1) // alignment * alignment


def _groups4(width: int) -> int:
    return (width // 32 + 3) // 4 * 4


@dataclass(frozen=True)
class MoeShape:
    """Sizes of one routed-MoE layer."""

    hidden: int = _HIDDEN_SIZE
    intermediate: int = _INTERMEDIATE_SIZE
    experts: int = _NUM_EXPERTS
    topk: int = _TOPK


def _layout(batch_size: int, shape: MoeShape) -> list[tuple[str, tuple[int, ...], torch.dtype, int]]:
    routes = batch_size * shape.topk
    padded_rows = grouped_scale_rows(routes, shape.experts)
    return [
        ("quantized", (batch_size, shape.hidden), torch.uint8, 16),
        ("input_scales", (batch_size, shape.hidden // 32), torch.uint8, 16),
        ("packed_input_scales", (packed_scale_numel(batch_size, shape.hidden),), torch.uint8, 16),
        ("topk_weights", (batch_size, shape.topk), torch.float32, 16),
        ("topk_ids", (batch_size, shape.topk), torch.int32, 16),
        ("source_tokens", (routes,), torch.int32, 16),
        ("permuted", (routes, shape.hidden), torch.uint8, 128),
        ("grouped_input_scales", (padded_rows * _groups4(shape.hidden),), torch.uint8, 128),
        ("activated", (routes, shape.intermediate), torch.uint8, 128),
        ("activated_scales", (padded_rows * _groups4(shape.intermediate),), torch.uint8, 128),
        ("expert_cursors", (shape.experts,), torch.int32, 16),
        ("expert_offsets", (shape.experts + 1,), torch.int64, 16),
        ("scale_offsets", (shape.experts + 1,), torch.int64, 16),
        ("inverse_permutation", (routes,), torch.int32, 16),
        ("routed_output", (routes, shape.hidden), torch.bfloat16, 128),
    ]


def qwen35_grouped_workspace_bytes(batch_size: int, shape: MoeShape = MoeShape()) -> int:
    """Bytes of scratch one layer call needs for ``batch_size`` tokens."""
    if batch_size < 1:
        raise ValueError("batch_size must be positive")
    offset = 0
    for _, dims, dtype, alignment in _layout(batch_size, shape):
        elements = 1
        for d in dims:
            elements *= d
        offset = _align_up(offset, alignment) + elements * torch.empty((), dtype=dtype).element_size()
    return _align_up(offset, 256)


def qwen35_grouped_workspace_shapes(
    batch_size: int, shape: MoeShape = MoeShape()
) -> tuple[tuple[int, int], tuple[int, int]]:
    """Return two BF16 workspace shapes that together hold the grouped schedule's
    scratch (the reference splits its scratch over two tensors the same way)."""
    total = qwen35_grouped_workspace_bytes(batch_size, shape)
    routes = batch_size * shape.topk
    half = _align_up((total + 1) // 2, 256)
    width = (half // 2 + routes - 1) // routes
    return (routes, width), (routes, width)


class _ByteArena:
    """Carves typed, aligned views out of one caller-owned allocation, front to back."""

    def __init__(self, storage: torch.Tensor, offset: int = 0) -> None:
        if not storage.is_contiguous():
            raise ValueError("workspace storage must be contiguous")
        self.storage = storage.view(torch.uint8).flatten()
        self.offset = offset

    def take(self, shape: tuple[int, ...], dtype: torch.dtype, alignment: int) -> torch.Tensor:
        nbytes = math.prod(shape) * dtype.itemsize
        # alignment is a property of the ADDRESS, not of the offset into the allocation
        address = self.storage.data_ptr() + self.offset
        begin = self.offset + (-address) % alignment
        if begin + nbytes > self.storage.numel():
            raise ValueError("grouped MoE workspace is too small")
        self.offset = begin + nbytes
        return self.storage[begin : self.offset].view(dtype).view(shape)


@dataclass(frozen=True)
class Qwen35GroupedWorkspace:
    """Views over graph-stable scratch storage for the grouped schedule."""

    quantized: torch.Tensor
    input_scales: torch.Tensor
    packed_input_scales: torch.Tensor
    topk_weights: torch.Tensor
    topk_ids: torch.Tensor
    source_tokens: torch.Tensor
    permuted: torch.Tensor
    grouped_input_scales: torch.Tensor
    activated: torch.Tensor
    activated_scales: torch.Tensor
    expert_cursors: torch.Tensor
    expert_offsets: torch.Tensor
    scale_offsets: torch.Tensor
    inverse_permutation: torch.Tensor
    routed_output: torch.Tensor
    shape: MoeShape = MoeShape()

    @classmethod
    def from_storage(
        cls,
        output: torch.Tensor,
        first: torch.Tensor,
        second: torch.Tensor | None = None,
        shape: MoeShape = MoeShape(),
    ) -> "Qwen35GroupedWorkspace":
        """Partition caller-owned scratch tensors without allocating CUDA memory.

        ``first`` (and ``second`` when the scratch is split in two, as the reference
        does) must together hold :func:`qwen35_grouped_workspace_bytes` bytes.
        """
        if (
            output.dtype != torch.bfloat16
            or output.ndim != 2
            or output.shape[1] != shape.hidden
            or not output.is_contiguous()
        ):
            raise ValueError(f"output must be contiguous BF16 [B,{shape.hidden}]")
        batch_size = int(output.shape[0])
        arenas = [_ByteArena(first)] + ([] if second is None else [_ByteArena(second)])
        views = {}
        index = 0
        for name, dims, dtype, alignment in _layout(batch_size, shape):
            while True:
                try:
                    views[name] = arenas[index].take(dims, dtype, alignment)
                    break
                except ValueError:
                    index += 1
                    if index >= len(arenas):
                        raise ValueError("grouped MoE workspace is too small") from None
        return cls(shape=shape, **views)

    @classmethod
    def allocate(cls, batch_size: int, device, shape: MoeShape = MoeShape()):
        """Convenience constructor that owns its storage."""
        storage = torch.empty(
            qwen35_grouped_workspace_bytes(batch_size, shape) + 256, dtype=torch.uint8, device=device
        )
        output = torch.empty((batch_size, shape.hidden), dtype=torch.bfloat16, device=device)
        return cls.from_storage(output, storage, None, shape)


def qwen35_grouped_gemm_out(
    workspace: Qwen35GroupedWorkspace,
    hidden: torch.Tensor,
    router_logits: torch.Tensor,
    w1: torch.Tensor,
    w1_scales: torch.Tensor,
    w2: torch.Tensor,
    w2_scales: torch.Tensor,
    renormalize: bool = True,
    expert_map: torch.Tensor | None = None,
) -> None:
    """Queue routing and the two grouped GEMMs into ``workspace``.

    top-k + MXFP8 quantization + row permutation, then the grouped W1 with the
    fused SiLU*mul + MXFP8 epilogue, then the grouped W2 into
    ``workspace.routed_output``.
    """
    qwen35_topk_quant_route_out(
        workspace.quantized,
        workspace.input_scales,
        workspace.packed_input_scales,
        workspace.topk_weights,
        workspace.topk_ids,
        workspace.permuted,
        workspace.grouped_input_scales,
        workspace.expert_cursors,
        workspace.expert_offsets,
        workspace.scale_offsets,
        workspace.inverse_permutation,
        hidden,
        router_logits,
        source_tokens=workspace.source_tokens,
        renormalize=renormalize,
        expert_map=expert_map,
    )
    _grouped_experts_out(workspace, w1, w1_scales, w2, w2_scales)


# From this many routed rows on, W1 runs as a plain grouped GEMM followed by the
# SiLU*mul/MXFP8 kernel: in the fused kernel four epilogue warps per SM do all the
# activation math, which a prefill batch makes the bottleneck (4096 tokens, top-8:
# 119 + 25 us unfused against 169 us fused).  Both forms give identical bytes.
UNFUSED_W1_MIN_ROUTES = 16384


def _grouped_experts_out(workspace, w1, w1_scales, w2, w2_scales) -> None:
    routes, hidden = (int(v) for v in workspace.routed_output.shape)
    two_inter = int(w1.shape[1])
    if routes >= UNFUSED_W1_MIN_ROUTES and two_inter <= hidden:
        # The BF16 gate/up rows live in the front of routed_output, which W2 overwrites
        # only after the activation kernel has consumed them.
        gate_up = workspace.routed_output.view(-1)[: routes * two_inter].view(routes, two_inter)
        grouped_gemm_w6a8_out(
            gate_up,
            workspace.permuted,
            workspace.grouped_input_scales,
            w1,
            w1_scales,
            workspace.expert_offsets,
            workspace.scale_offsets,
        )
        silu_and_mul_mxfp8_grouped_out(
            workspace.activated,
            workspace.activated_scales,
            gate_up,
            workspace.expert_offsets,
            workspace.scale_offsets,
            grouped_output=workspace.routed_output,
            weight=w2,
            weight_scales=w2_scales,
        )
        return
    qwen35_grouped_w1_silu_mxfp8_out(
        workspace.activated,
        workspace.activated_scales,
        workspace.permuted,
        workspace.grouped_input_scales,
        w1,
        w1_scales,
        workspace.expert_offsets,
        workspace.scale_offsets,
    )
    grouped_gemm_w6a8_out(
        workspace.routed_output,
        workspace.activated,
        workspace.activated_scales,
        w2,
        w2_scales,
        workspace.expert_offsets,
        workspace.scale_offsets,
    )


def qwen35_grouped_reduce_out(
    workspace: Qwen35GroupedWorkspace,
    output: torch.Tensor,
    shared_output: torch.Tensor | None = None,
    shared_gate: torch.Tensor | None = None,
) -> torch.Tensor:
    """Reduce routed rows and optionally add the (gated) shared expert."""
    moe_reduce_out(
        output,
        workspace.routed_output,
        workspace.topk_weights,
        workspace.inverse_permutation,
        shared_output=shared_output,
        shared_gate=shared_gate,
    )
    return output


def qwen35_grouped_moe_logits_out(
    workspace: Qwen35GroupedWorkspace,
    output: torch.Tensor,
    hidden: torch.Tensor,
    router_logits: torch.Tensor,
    w1: torch.Tensor,
    w1_scales: torch.Tensor,
    w2: torch.Tensor,
    w2_scales: torch.Tensor,
    shared_output: torch.Tensor | None = None,
    renormalize: bool = True,
    shared_gate: torch.Tensor | None = None,
) -> torch.Tensor:
    """Run the allocation-free fused-router grouped schedule."""
    qwen35_grouped_gemm_out(
        workspace, hidden, router_logits, w1, w1_scales, w2, w2_scales, renormalize=renormalize
    )
    return qwen35_grouped_reduce_out(workspace, output, shared_output, shared_gate)


def qwen35_grouped_moe_out(
    workspace: Qwen35GroupedWorkspace,
    output: torch.Tensor,
    hidden: torch.Tensor,
    w1: torch.Tensor,
    w1_scales: torch.Tensor,
    w2: torch.Tensor,
    w2_scales: torch.Tensor,
    topk_weights: torch.Tensor,
    topk_ids: torch.Tensor,
) -> torch.Tensor:
    """Run the routed schedule with caller-provided top-k weights and ids."""
    qwen35_topk_quant_out_rows(workspace, hidden)
    qwen35_route_mxfp8_out(
        workspace.quantized,
        workspace.input_scales,
        topk_ids,
        workspace.permuted,
        workspace.grouped_input_scales,
        workspace.expert_cursors,
        workspace.expert_offsets,
        workspace.scale_offsets,
        workspace.inverse_permutation,
        source_tokens=workspace.source_tokens,
    )
    _grouped_experts_out(workspace, w1, w1_scales, w2, w2_scales)
    moe_reduce_out(output, workspace.routed_output, topk_weights, workspace.inverse_permutation)
    return output


def qwen35_topk_quant_out_rows(workspace: Qwen35GroupedWorkspace, hidden: torch.Tensor) -> None:
    """Quantize ``hidden`` into the workspace (values, logical and dense packed scales)."""
    from ._loader import check, library
    from .ops import _stream

    batch, width = (int(v) for v in hidden.shape)
    with torch.cuda.device(hidden.device):
        check(
            library().mxfp6_moe_topk_quant(
                hidden.data_ptr(), None, batch, width, 0, 0, 0, workspace.quantized.data_ptr(),
                workspace.input_scales.data_ptr(), workspace.packed_input_scales.data_ptr(), None,
                None, _stream(hidden.device),
            )
        )


@dataclass(frozen=True)
class SharedExpertWorkspace:
    """Scratch of the always-on shared expert: its MXFP8 intermediate and output."""

    activated: torch.Tensor
    activated_scales: torch.Tensor
    output: torch.Tensor

    @classmethod
    def allocate(cls, batch_size: int, device, shape: MoeShape = MoeShape()):
        return cls(
            torch.empty((batch_size, shape.intermediate), dtype=torch.uint8, device=device),
            torch.full((packed_scale_numel(batch_size, shape.intermediate),), 0x7F,
                       dtype=torch.uint8, device=device),
            torch.empty((batch_size, shape.hidden), dtype=torch.bfloat16, device=device),
        )


def shared_expert_out(
    shared: SharedExpertWorkspace,
    workspace: Qwen35GroupedWorkspace,
    w1: PackedMXFP6Tensor,
    w2: PackedMXFP6Tensor,
) -> torch.Tensor:
    """Shared expert on the rows already quantized in ``workspace``: dense W1 with the
    fused SiLU*mul + MXFP8 epilogue, then the dense W2 GEMM (BF16 out).

    The reference's callers compute the same thing with two dense GEMMs and
    ``silu_and_mul_mxfp8_packed_out`` (benchmarks/benchmark_qwen35_moe_layer.py:1102-1127).
    """
    batch, hidden = (int(v) for v in workspace.quantized.shape)
    dense_w1_silu_mxfp8_out(shared.activated, shared.activated_scales, workspace.quantized,
                            workspace.packed_input_scales, w1.values, w1.scales)
    act = MXFP8Tensor(shared.activated.view(-1), shared.activated_scales, batch,
                      int(shared.activated.shape[1]))
    return gemm_w6a8(act, w2, out_dtype=torch.bfloat16, out=shared.output)


# ---- decode schedule: one single-row GEMM per route, three launches after the router ----


@dataclass(frozen=True)
class Qwen35MoeB1Workspace:
    """Scratch of the decode schedule (the reference's B=1 workspace,
    python/mxfp6/qwen35.py:73-83,247-298, for ``batch`` tokens of any layer shape).

    ``activation`` holds ``topk + 1`` rows per token: the routed experts' activated rows,
    then the shared expert's.  ``w1_partial`` / ``w2_partial`` are the reference's split-K
    scratch; the kernels here reduce inside a thread-block cluster, so both are empty.
    """

    quantized: torch.Tensor          # [B, H] e4m3
    input_scales: torch.Tensor       # [B, H/32] logical UE8M0
    routed_logits: torch.Tensor      # [B, E] bf16
    topk_weights: torch.Tensor       # [B, topk] f32
    topk_ids: torch.Tensor           # [B, topk] i32
    shared_gate: torch.Tensor        # [B] bf16 (logit; the reduce applies the sigmoid)
    w1_partial: torch.Tensor
    activation: torch.Tensor         # [B * (topk + 1), I] e4m3
    activation_scales: torch.Tensor  # [B * (topk + 1), I/32]
    w2_partial: torch.Tensor
    output: torch.Tensor             # [B, H] bf16

    @classmethod
    def allocate(cls, device, shape: MoeShape = MoeShape(), batch: int = 1):
        if batch < 1:
            raise ValueError("batch must be positive")
        h, i, e, k = shape.hidden, shape.intermediate, shape.experts, shape.topk
        lanes = batch * (k + 1)
        u8 = dict(dtype=torch.uint8, device=device)
        return cls(
            torch.empty((batch, h), dtype=torch.float8_e4m3fn, device=device),
            torch.empty((batch, h // 32), **u8),
            torch.empty((batch, e), dtype=torch.bfloat16, device=device),
            torch.empty((batch, k), dtype=torch.float32, device=device),
            torch.empty((batch, k), dtype=torch.int32, device=device),
            torch.empty((batch,), dtype=torch.bfloat16, device=device),
            torch.empty((0,), dtype=torch.float32, device=device),
            torch.empty((lanes, i), dtype=torch.float8_e4m3fn, device=device),
            torch.empty((lanes, i // 32), **u8),
            torch.empty((0,), dtype=torch.float32, device=device),
            torch.empty((batch, h), dtype=torch.bfloat16, device=device),
        )


def qwen35_moe_b1_out(
    workspace: Qwen35MoeB1Workspace,
    hidden: torch.Tensor,
    combined_gate: torch.Tensor,
    w1: torch.Tensor,
    w1_scales: torch.Tensor,
    w2: torch.Tensor,
    w2_scales: torch.Tensor,
    renormalize: bool = False,
) -> torch.Tensor:
    """Decode schedule from the hidden rows: router, W1 routes, W2 routes + reduce
    (python/mxfp6/qwen35.py:384-432).

    ``combined_gate`` is the routed gate rows followed by the shared expert's gate row;
    ``w1`` ``[E + 1, 2I, 3H/4]`` and ``w2`` ``[E + 1, H, 3I/4]`` end with the shared expert.
    """
    tokens, hidden_size = (int(v) for v in hidden.shape)
    if moe_decode_layer_preferred(tokens, int(workspace.topk_ids.shape[1]),
                                  int(workspace.routed_logits.shape[1]), hidden_size,
                                  int(w1.shape[1]) // 2):
        # router, then W1 with top-k and quantization inside, then W2: three launches
        router_logits_out(workspace.routed_logits, workspace.shared_gate, hidden, combined_gate)
        moe_decode_layer_out(workspace.output, workspace.activation, workspace.activation_scales,
                             workspace.topk_weights, workspace.topk_ids, hidden,
                             workspace.routed_logits, workspace.shared_gate, w1, w1_scales, w2,
                             w2_scales, renormalize=renormalize)
        return workspace.output
    qwen35_router_quant_out(
        workspace.quantized, workspace.input_scales, workspace.routed_logits,
        workspace.topk_weights, workspace.topk_ids, workspace.shared_gate, hidden,
        combined_gate, renormalize=renormalize)
    return _decode_routes_out(workspace, w1, w1_scales, w2, w2_scales, None, None)


def qwen35_moe_decode_logits_out(
    workspace: Qwen35MoeB1Workspace,
    hidden: torch.Tensor,
    router_logits: torch.Tensor,
    shared_gate: torch.Tensor,
    w1: torch.Tensor,
    w1_scales: torch.Tensor,
    w2: torch.Tensor,
    w2_scales: torch.Tensor,
    shared_w1: PackedMXFP6Tensor | None = None,
    shared_w2: PackedMXFP6Tensor | None = None,
    renormalize: bool = True,
    two_launches: bool | None = None,
) -> torch.Tensor:
    """Decode schedule from given router logits.  Two launches where that is expected to be
    faster (top-k and quantization inside the W1 kernel, ``moe_decode_layer_out``), else three:
    top-k + quantization, W1 routes, W2 routes + reduce; ``two_launches`` forces either.
    Both give the same bytes.  The shared expert is the last matrix of ``w1`` / ``w2`` or,
    when ``shared_w1`` / ``shared_w2`` are given, a separate pair."""
    tokens, hidden_size = (int(v) for v in hidden.shape)
    topk = int(workspace.topk_ids.shape[1])
    if two_launches is None:
        two_launches = moe_decode_layer_preferred(tokens, topk, int(router_logits.shape[1]),
                                                  hidden_size, int(w1.shape[1]) // 2)
    if two_launches:
        sw = (None,) * 4
        if shared_w1 is not None:
            sw = (shared_w1.values.view(1, *w1.shape[1:]), shared_w1.scales,
                  shared_w2.values.view(1, *w2.shape[1:]), shared_w2.scales)
        moe_decode_layer_out(workspace.output, workspace.activation, workspace.activation_scales,
                             workspace.topk_weights, workspace.topk_ids, hidden, router_logits,
                             shared_gate, w1, w1_scales, w2, w2_scales, *sw, renormalize=renormalize)
        return workspace.output
    qwen35_topk_quant_out(workspace.quantized, workspace.input_scales, None,
                          workspace.topk_weights, workspace.topk_ids, hidden, router_logits,
                          renormalize=renormalize)
    return _decode_routes_out(workspace, w1, w1_scales, w2, w2_scales, shared_w1, shared_w2,
                              shared_gate)


def _decode_routes_out(workspace, w1, w1_scales, w2, w2_scales, shared_w1, shared_w2,
                       shared_gate=None):
    sw1 = sw1s = sw2 = sw2s = None
    if shared_w1 is not None:
        sw1, sw1s = shared_w1.values.view(1, *w1.shape[1:]), shared_w1.scales
        sw2, sw2s = shared_w2.values.view(1, *w2.shape[1:]), shared_w2.scales
    qwen35_w1_splitk_silu_mxfp8_out(
        workspace.activation, workspace.activation_scales, workspace.w1_partial,
        workspace.quantized, workspace.input_scales, w1, w1_scales, workspace.topk_ids,
        True, sw1, sw1s)
    qwen35_w2_splitk_reduce_out(
        workspace.output, workspace.w2_partial, workspace.activation,
        workspace.activation_scales, w2, w2_scales, workspace.topk_ids, workspace.topk_weights,
        workspace.shared_gate if shared_gate is None else shared_gate, sw2, sw2s,
        routing_ready=True)  # the ids were written before W1, which waits before it lets W2 start
    return workspace.output
