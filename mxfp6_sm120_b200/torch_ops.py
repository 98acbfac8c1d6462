"""``torch.ops.mxfp6.*``: the reference's operator namespace over this library.

External callers of the reference reach its kernels through the dispatcher, not through
the Python package: the vLLM integration calls
``torch.ops.mxfp6.gemm_w6a8(x_u8, weight, input_scale, weight_scale, rows, N, K, 1.0, dtype)``
(examples/vllm/patches/vllm-v0.25.1-mxfp6.patch:277-300).  This module defines the same
operator names with the same schemas (csrc/torch_extension.cu:2120-2157 for the dense and
format operators, csrc/moe.cu:10012-10132 for the routed-MoE fragment) and implements each
for the CUDA dispatch key with the wrappers of this package, which call the C ABI.

Importing the package registers the namespace once per process.  If another library has
defined ``mxfp6`` already (the reference's own extension loaded beside this one),
registration is skipped and :data:`REGISTERED` stays ``False``.
"""

from __future__ import annotations

import torch

from . import moe_ops, ops

REGISTERED = False
_LIBRARY = None  # keeps the registrations alive

# name -> schema after the name, in the reference's order
_SCHEMAS = {
    # dense GEMMs, explicit configurations, workspace arena, formats
    "gemm": "(Tensor a, Tensor b, Tensor sfa, Tensor sfb, int m, int n, int k, float alpha=1.0, "
            "ScalarType? out_dtype=None) -> Tensor",
    "gemm_w6a8": "(Tensor a, Tensor b, Tensor sfa, Tensor sfb, int m, int n, int k, float alpha=1.0, "
                 "ScalarType? out_dtype=None) -> Tensor",
    "gemm_w6a8_config": "(Tensor a, Tensor b, Tensor sfa, Tensor sfb, int m, int n, int k, float alpha, "
                        "int config_id, int swizzle, int raster_order, ScalarType? out_dtype=None) -> Tensor",
    "gemm_from_float": "(Tensor input, Tensor b, Tensor sfb, int n, float alpha=1.0, "
                       "ScalarType? out_dtype=None) -> Tensor",
    "gemm_from_float_config": "(Tensor input, Tensor b, Tensor sfb, int n, float alpha, int config_id, "
                              "int swizzle, int raster_order, ScalarType? out_dtype=None) -> Tensor",
    "set_w6a8_config": "(Tensor anchor, int m, int n, int k, int config_id, int swizzle, int raster_order, "
                       "ScalarType? out_dtype=None) -> bool",
    "w6a8_config_abi": "(Tensor anchor) -> str",
    "begin_workspace_planning": "(Tensor anchor) -> ()",
    "finalize_workspace_planning": "(Tensor anchor) -> Dict(str, int)",
    "workspace_stats": "(Tensor anchor) -> Dict(str, int)",
    "workspace_barriers_zero": "(Tensor anchor) -> bool",
    "_set_workspace_collection": "(Tensor anchor, bool enabled) -> bool",
    "pack_fp6": "(Tensor codes) -> Tensor",
    "unpack_fp6": "(Tensor packed, int rows, int k) -> Tensor",
    "pad_fp6": "(Tensor packed) -> Tensor",
    "expand_fp6_to_fp8": "(Tensor packed, int rows, int k) -> Tensor",
    "quantize_mxfp8": "(Tensor input) -> (Tensor values, Tensor scales)",
    "quantize_mxfp8_dual": "(Tensor input) -> (Tensor values, Tensor logical_scales, Tensor packed_scales)",
    "quantize_mxfp8_dual_out": "(Tensor(a!) output, Tensor(b!) logical_scales, Tensor(c!) packed_scales, "
                               "Tensor input) -> ()",
    "quantize_mxfp6": "(Tensor input) -> (Tensor values, Tensor scales)",
    "pack_scales": "(Tensor logical, int rows, int k) -> Tensor",
    "unpack_scales": "(Tensor packed, int rows, int k) -> Tensor",
    # routed MoE
    "quantize_mxfp8_logical": "(Tensor input) -> (Tensor values, Tensor scales)",
    "route_mxfp8_out": "(Tensor activation, Tensor logical_scales, Tensor topk_ids, Tensor? expert_map, "
                       "int local_experts, Tensor(a!) permuted_activation, bool include_shared=False) -> "
                       "(Tensor packed_scales, Tensor expert_offsets, Tensor scale_offsets, "
                       "Tensor inverse_permutation)",
    "qwen35_route_mxfp8_out": "(Tensor activation, Tensor logical_scales, Tensor topk_ids, "
                              "Tensor(a!) permuted_activation, Tensor(b!) packed_scales, "
                              "Tensor(c!) expert_cursors, Tensor(d!) expert_offsets, "
                              "Tensor(e!) scale_offsets, Tensor(f!) inverse_permutation, "
                              "bool include_shared=False) -> ()",
    "pack_grouped_scales": "(Tensor logical, Tensor expert_offsets) -> (Tensor packed, Tensor scale_offsets)",
    "silu_and_mul_mxfp8_grouped": "(Tensor input, Tensor expert_offsets, Tensor? scale_offsets=None) -> "
                                  "(Tensor values, Tensor scales, Tensor scale_offsets)",
    "silu_and_mul_mxfp8_grouped_out": "(Tensor(a!) output, Tensor(b!) scales, Tensor input, "
                                      "Tensor expert_offsets, Tensor scale_offsets, bool use_pdl=False, "
                                      "Tensor(c!)? grouped_output=None, Tensor? weight=None, "
                                      "Tensor? weight_scales=None) -> ()",
    "silu_and_mul_mxfp8_logical": "(Tensor input) -> (Tensor values, Tensor scales)",
    "silu_and_mul_mxfp8_packed_out": "(Tensor(a!) output, Tensor(b!) packed_scales, Tensor input) -> ()",
    "array_gemm_w6a8_out": "(Tensor(a!) output, Tensor activation, Tensor logical_scales, Tensor weight, "
                           "Tensor weight_scales, Tensor topk_ids, bool include_shared=False) -> ()",
    "array_gemm_w6a8_silu_mxfp8_out": "(Tensor(a!) output, Tensor(b!) output_scales, Tensor activation, "
                                      "Tensor logical_scales, Tensor weight, Tensor weight_scales, "
                                      "Tensor topk_ids, bool include_shared=False) -> ()",
    "array_gemm_w6a8_reduce_out": "(Tensor(a!) output, Tensor activation, Tensor logical_scales, "
                                  "Tensor weight, Tensor weight_scales, Tensor topk_ids, "
                                  "Tensor topk_weights, Tensor shared_gate, Tensor? shared_output=None, "
                                  "Tensor? shared_weight=None, Tensor? shared_weight_scales=None, "
                                  "bool use_packed_vector_loads=False) -> ()",
    "qwen35_router_quant_out": "(Tensor(a!) quantized, Tensor(b!) logical_scales, Tensor(c!) routed_logits, "
                               "Tensor(d!) topk_weights, Tensor(e!) topk_ids, Tensor(f!) shared_gate, "
                               "Tensor hidden, Tensor gate_weight, bool renormalize=False, "
                               "Tensor? shared_gate_weight=None) -> ()",
    "qwen35_topk_quant_out": "(Tensor(a!) quantized, Tensor(b!) logical_scales, Tensor(c!) packed_scales, "
                             "Tensor(d!) topk_weights, Tensor(e!) topk_ids, Tensor hidden, "
                             "Tensor routed_logits, bool renormalize=False) -> ()",
    "qwen35_topk_quant_route_out": "(Tensor(a!) quantized, Tensor(b!) logical_scales, Tensor(c!) dense_scales, "
                                   "Tensor(d!) topk_weights, Tensor(e!) topk_ids, "
                                   "Tensor(f!) permuted_activation, Tensor(g!) grouped_scales, "
                                   "Tensor(h!) expert_cursors, Tensor(i!) expert_offsets, "
                                   "Tensor(j!) scale_offsets, Tensor(k!) inverse_permutation, Tensor hidden, "
                                   "Tensor routed_logits, Tensor(l!)? grouped_output=None, "
                                   "Tensor? weight=None, Tensor? weight_scales=None, "
                                   "Tensor(m!)? source_tokens=None, bool renormalize=False) -> ()",
    "qwen35_w1_splitk_silu_mxfp8_out": "(Tensor(a!) output, Tensor(b!) output_scales, Tensor(c!) partial, "
                                       "Tensor activation, Tensor logical_scales, Tensor weight, "
                                       "Tensor weight_scales, Tensor topk_ids, bool include_shared=True, "
                                       "Tensor? shared_weight=None, Tensor? shared_weight_scales=None) -> ()",
    "qwen35_w2_splitk_reduce_out": "(Tensor(a!) output, Tensor(b!) partial, Tensor activation, "
                                   "Tensor logical_scales, Tensor weight, Tensor weight_scales, "
                                   "Tensor topk_ids, Tensor topk_weights, Tensor shared_gate, "
                                   "Tensor? shared_weight=None, Tensor? shared_weight_scales=None) -> ()",
    "grouped_gemm_w6a8_out": "(Tensor(a!) output, Tensor activation, Tensor activation_scales, Tensor weight, "
                             "Tensor weight_scales, Tensor expert_offsets, Tensor scale_offsets, int tile_n=0, "
                             "bool use_pdl=False) -> ()",
    "qwen35_grouped_w1_silu_mxfp8_out": "(Tensor(a!) output, Tensor(b!) output_scales, Tensor activation, "
                                        "Tensor activation_scales, Tensor weight, Tensor weight_scales, "
                                        "Tensor expert_offsets, Tensor scale_offsets, bool use_pdl=False, "
                                        "Tensor? source_tokens=None) -> ()",
    "moe_reduce_out": "(Tensor(a!) output, Tensor routed_output, Tensor topk_weights, "
                      "Tensor inverse_permutation, Tensor? shared_output=None, Tensor? shared_gate=None, "
                      "bool use_pdl=False) -> ()",
    "moe_reduce_tp2_out": "(Tensor(a!) output, Tensor routed_output, Tensor topk_weights, "
                          "Tensor inverse_permutation, Tensor shared_output, Tensor shared_gate, "
                          "int[] signal_ptrs, int[] buffer_ptrs, int rank) -> ()",
    "moe_reduce_array_out": "(Tensor(a!) output, Tensor combined_output, Tensor topk_weights, "
                            "Tensor shared_gate) -> ()",
}


def _dtype(out_dtype):
    return torch.float16 if out_dtype is None else out_dtype


def _act(a, sfa, m, k):
    return ops.MXFP8Tensor(a.view(torch.uint8).reshape(-1), sfa, int(m), int(k))


def _wgt(b, sfb, n, k):
    return ops.PackedMXFP6Tensor(b.reshape(-1), sfb, int(n), int(k))


def _check_launch_hints(swizzle, raster_order):
    # Tile-order hints of the reference's CUTLASS kernels; validated, then unused.
    if swizzle not in (1, 2, 4, 8) or raster_order not in (0, 1, 2):
        raise ValueError("swizzle must be 1, 2, 4 or 8 and raster_order 0, 1 or 2")


def _gemm(a, b, sfa, sfb, m, n, k, alpha=1.0, out_dtype=None):
    return ops.gemm_packed(a, b, sfa, sfb, m, n, k, alpha, out_dtype=_dtype(out_dtype))


def _gemm_w6a8(a, b, sfa, sfb, m, n, k, alpha=1.0, out_dtype=None):
    return ops.gemm_w6a8(_act(a, sfa, m, k), _wgt(b, sfb, n, k), alpha, out_dtype=_dtype(out_dtype))


def _gemm_w6a8_config(a, b, sfa, sfb, m, n, k, alpha, config_id, swizzle, raster_order, out_dtype=None):
    _check_launch_hints(swizzle, raster_order)
    return ops.gemm_w6a8_config(_act(a, sfa, m, k), _wgt(b, sfb, n, k), alpha,
                                out_dtype=_dtype(out_dtype), config_id=int(config_id))


def _gemm_from_float(input, b, sfb, n, alpha=1.0, out_dtype=None):
    return ops.gemm_from_float(input, _wgt(b, sfb, n, input.shape[1]), alpha, out_dtype=_dtype(out_dtype))


def _gemm_from_float_config(input, b, sfb, n, alpha, config_id, swizzle, raster_order, out_dtype=None):
    _check_launch_hints(swizzle, raster_order)
    return ops.gemm_w6a8_config(ops.quantize_mxfp8(input), _wgt(b, sfb, n, input.shape[1]), alpha,
                                out_dtype=_dtype(out_dtype), config_id=int(config_id))


def _set_w6a8_config(anchor, m, n, k, config_id, swizzle, raster_order, out_dtype=None):
    return ops.set_w6a8_config(anchor, m, n, k, config_id, swizzle, raster_order, out_dtype)


def _set_workspace_collection(anchor, enabled):
    # The reference's switch only starts or stops recording layouts; here recording is the
    # planning phase of the arena, so switching it off freezes what was recorded.
    previous = bool(ops.workspace_stats(anchor.device)["planning"])
    if enabled and not previous:
        ops.begin_workspace_planning(anchor.device)
    elif previous and not enabled:
        ops.finalize_workspace_planning(anchor.device)
    return previous


def _quantize_mxfp8(input):
    q = ops.quantize_mxfp8(input)
    return q.values.view(q.rows, q.k).view(torch.float8_e4m3fn), q.scales


def _quantize_mxfp6(input):
    q = ops.quantize_mxfp6(input)
    return q.values, q.scales


def _pack_scales(logical, rows, k):
    if tuple(logical.shape) != (int(rows), int(k) // ops.SCALE_VECTOR_SIZE):
        raise ValueError("logical must have shape [rows, k / 32]")
    return ops.pack_scales(logical)


def _array_silu(output, output_scales, activation, logical_scales, weight, weight_scales, topk_ids,
                include_shared=False):
    moe_ops.array_gemm_w6a8_silu_mxfp8_out(output, output_scales, activation, logical_scales, weight,
                                           weight_scales, topk_ids, bool(include_shared))


def _topk_quant_route(quantized, logical_scales, dense_scales, topk_weights, topk_ids, permuted_activation,
                      grouped_scales, expert_cursors, expert_offsets, scale_offsets, inverse_permutation,
                      hidden, routed_logits, grouped_output=None, weight=None, weight_scales=None,
                      source_tokens=None, renormalize=False):
    moe_ops.qwen35_topk_quant_route_out(
        quantized, logical_scales, dense_scales, topk_weights, topk_ids, permuted_activation,
        grouped_scales, expert_cursors, expert_offsets, scale_offsets, inverse_permutation, hidden,
        routed_logits, grouped_output, weight, weight_scales, source_tokens, bool(renormalize))


def _grouped_w1(output, output_scales, activation, activation_scales, weight, weight_scales, expert_offsets,
                scale_offsets, use_pdl=False, source_tokens=None):
    moe_ops.qwen35_grouped_w1_silu_mxfp8_out(output, output_scales, activation, activation_scales, weight,
                                             weight_scales, expert_offsets, scale_offsets, bool(use_pdl),
                                             source_tokens)


def _reduce_tp2(output, routed_output, topk_weights, inverse_permutation, shared_output, shared_gate,
                signal_ptrs, buffer_ptrs, rank):
    moe_ops.moe_reduce_tp2_out(output, routed_output, topk_weights, inverse_permutation, shared_output,
                               shared_gate, list(signal_ptrs), list(buffer_ptrs), int(rank))


def _returns_none(function):
    def call(*args, **kwargs):
        function(*args, **kwargs)

    return call


_IMPLEMENTATIONS = {
    "gemm": _gemm,
    "gemm_w6a8": _gemm_w6a8,
    "gemm_w6a8_config": _gemm_w6a8_config,
    "gemm_from_float": _gemm_from_float,
    "gemm_from_float_config": _gemm_from_float_config,
    "set_w6a8_config": _set_w6a8_config,
    "w6a8_config_abi": lambda anchor: ops.w6a8_config_abi(anchor),
    "begin_workspace_planning": lambda anchor: ops.begin_workspace_planning(anchor.device),
    "finalize_workspace_planning": lambda anchor: ops.finalize_workspace_planning(anchor.device),
    "workspace_stats": lambda anchor: ops.workspace_stats(anchor.device),
    "workspace_barriers_zero": lambda anchor: ops.workspace_barriers_zero(anchor.device),
    "_set_workspace_collection": _set_workspace_collection,
    "pack_fp6": ops.pack_fp6,
    "unpack_fp6": ops.unpack_fp6,
    "pad_fp6": ops.pad_fp6,
    "expand_fp6_to_fp8": ops.expand_fp6_to_fp8,
    "quantize_mxfp8": _quantize_mxfp8,
    "quantize_mxfp8_dual": ops.quantize_mxfp8_dual,
    "quantize_mxfp8_dual_out": _returns_none(ops.quantize_mxfp8_dual_out),
    "quantize_mxfp6": _quantize_mxfp6,
    "pack_scales": _pack_scales,
    "unpack_scales": ops.unpack_scales,
    "quantize_mxfp8_logical": ops.quantize_mxfp8_logical,
    "route_mxfp8_out": moe_ops.route_mxfp8_out,
    "qwen35_route_mxfp8_out": _returns_none(moe_ops.qwen35_route_mxfp8_out),
    "pack_grouped_scales": ops.pack_grouped_scales,
    "silu_and_mul_mxfp8_grouped": moe_ops.silu_and_mul_mxfp8_grouped,
    "silu_and_mul_mxfp8_grouped_out": _returns_none(moe_ops.silu_and_mul_mxfp8_grouped_out),
    "silu_and_mul_mxfp8_logical": moe_ops.silu_and_mul_mxfp8_logical,
    "silu_and_mul_mxfp8_packed_out": _returns_none(moe_ops.silu_and_mul_mxfp8_packed_out),
    "array_gemm_w6a8_out": _returns_none(moe_ops.array_gemm_w6a8_out),
    "array_gemm_w6a8_silu_mxfp8_out": _array_silu,
    "array_gemm_w6a8_reduce_out": _returns_none(moe_ops.array_gemm_w6a8_reduce_out),
    "qwen35_router_quant_out": _returns_none(moe_ops.qwen35_router_quant_out),
    "qwen35_topk_quant_out": _returns_none(moe_ops.qwen35_topk_quant_out),
    "qwen35_topk_quant_route_out": _topk_quant_route,
    "qwen35_w1_splitk_silu_mxfp8_out": _returns_none(moe_ops.qwen35_w1_splitk_silu_mxfp8_out),
    "qwen35_w2_splitk_reduce_out": _returns_none(moe_ops.qwen35_w2_splitk_reduce_out),
    "grouped_gemm_w6a8_out": _returns_none(moe_ops.grouped_gemm_w6a8_out),
    "qwen35_grouped_w1_silu_mxfp8_out": _grouped_w1,
    "moe_reduce_out": _returns_none(moe_ops.moe_reduce_out),
    "moe_reduce_tp2_out": _reduce_tp2,
    "moe_reduce_array_out": _returns_none(moe_ops.moe_reduce_array_out),
}


def operator_names() -> list[str]:
    """The operator names this module defines under ``torch.ops.mxfp6``."""
    return list(_SCHEMAS)


def register() -> bool:
    """Define and implement the namespace (idempotent); ``False`` if it is taken already."""
    global REGISTERED, _LIBRARY
    if REGISTERED:
        return True
    assert _SCHEMAS.keys() == _IMPLEMENTATIONS.keys()
    try:
        library = torch.library.Library("mxfp6", "DEF")
    except RuntimeError:
        return False
    for name, schema in _SCHEMAS.items():
        library.define(name + schema)
        library.impl(name, _IMPLEMENTATIONS[name], "CUDA")
    _LIBRARY = library
    REGISTERED = True
    return True


register()
