"""B200-native (sm_100a) W6A8 GEMM and MoE kernels with packed MXFP6 weights.

Drop-in for the operator surface of Nekofish-L/mxfp6_sm120's ``mxfp6`` package:
``import mxfp6_sm120_b200 as mxfp6``.
"""

from ._loader import load_library
from .autotune import (
    W6A8Config,
    cache_directory as autotune_cache_directory,
    is_autotune_cache_only,
    is_autotune_enabled,
)
from .ops import (
    MXFP8Tensor,
    PackedMXFP6Tensor,
    SCALE_VECTOR_SIZE,
    TUNED_M,
    TUNED_NK,
    autotune_w6a8,
    begin_workspace_planning,
    device_status,
    expand_fp6_to_fp8,
    finalize_workspace_planning,
    gemm,
    gemm_from_codes,
    gemm_from_float,
    gemm_packed,
    gemm_w6a8,
    gemm_w6a8_config,
    gemm_w6a8_plan,
    is_available,
    is_stream_k_enabled,
    rmsnorm_quantize_mxfp8,
    set_cta_pair_mode,
    is_cta_pair_enabled,
    set_stream_kernel_mode,
    is_stream_kernel_enabled,
    set_w6a8_config,
    w6a8_config_abi,
    w6a8_configs,
    set_split_k_mode,
    is_tuned_shape,
    pack_fp6,
    pack_grouped_scales,
    pack_operand,
    pack_scales,
    packed_scale_numel,
    pad_fp6,
    quantize_activation,
    quantize_mxfp6,
    quantize_mxfp8,
    quantize_mxfp8_dual,
    quantize_mxfp8_dual_out,
    quantize_mxfp8_logical,
    to_mma_k64_weight,
    unpack_fp6,
    unpack_operand,
    unpack_scales,
    warmup_w6a8,
    workspace_barriers_zero,
    workspace_stats,
)

from .moe_ops import (
    array_gemm_w6a8_out,
    array_gemm_w6a8_reduce_out,
    array_gemm_w6a8_silu_mxfp8_out,
    dense_w1_silu_mxfp8_out,
    grouped_gemm_w6a8,
    grouped_gemm_w6a8_out,
    grouped_scale_rows,
    moe_decode_layer_out,
    moe_decode_layer_preferred,
    moe_decode_layer_supported,
    moe_reduce_array_out,
    moe_reduce_out,
    moe_reduce_tp2_out,
    qwen35_grouped_w1_silu_mxfp8_out,
    qwen35_router_quant_out,
    qwen35_w1_splitk_silu_mxfp8_out,
    qwen35_w2_splitk_reduce_out,
    qwen35_route_mxfp8_out,
    qwen35_topk_quant_out,
    qwen35_topk_quant_route_out,
    route_mxfp8_out,
    silu_and_mul_mxfp8_grouped,
    silu_and_mul_mxfp8_grouped_out,
    silu_and_mul_mxfp8_logical,
    silu_and_mul_mxfp8_packed_out,
)
from .qwen35 import (
    MoeShape,
    Qwen35GroupedWorkspace,
    Qwen35MoeB1Workspace,
    SharedExpertWorkspace,
    qwen35_grouped_gemm_out,
    qwen35_grouped_moe_logits_out,
    qwen35_grouped_moe_out,
    qwen35_grouped_reduce_out,
    qwen35_grouped_workspace_bytes,
    qwen35_grouped_workspace_shapes,
    qwen35_moe_b1_out,
    qwen35_moe_decode_logits_out,
    shared_expert_out,
)

from .checkpoint import MoeLayerCheckpoint, TensorSource, load_linear, load_moe_layer
from .adapter import MxFp6LinearKernel, MxFp6MoERunner
from . import torch_ops  # registers torch.ops.mxfp6.* (the reference's dispatcher names)

from .decoder import (
    DecoderConfig,
    DecoderLayer,
    DecoderWorkspace,
    DenseDecoder,
    random_layer,
    shard_layer,
)

__version__ = "0.1.0"
