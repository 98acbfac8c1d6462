"""Serving-framework adapter surface: a linear kernel and a routed-experts runner.

The reference ships its vLLM integration as a patch and an adapter module: a quantization
scheme whose ``process_weights_after_loading`` packs the logical scales and whose
``apply_weights`` quantizes the activation and calls ``torch.ops.mxfp6.gemm_w6a8``
(examples/vllm/patches/vllm-v0.25.1-mxfp6.patch:120-170,255-300,326-470), and a MoE runner
that owns per-batch workspaces and picks the single-token schedule or the grouped one
(examples/vllm/adapter/mxfp6_tp2_vllm.py:114-565).  The classes here have the same duties and
method names but take plain ``torch.nn.Module`` / tensors, so a framework glues them in with
a few lines and the tests run without one.  All GEMM calls go through the dispatcher names
(``torch.ops.mxfp6.*``), as an external caller's would.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from . import torch_ops  # noqa: F401  (registers torch.ops.mxfp6)
from .checkpoint import MoeLayerCheckpoint, pack_scales_host
from .moe_layer import DECODE_MAX_TOKENS, MoeLayer, MoeLayerState
from .ops import SCALE_VECTOR_SIZE, is_available

OCP_MX_BLOCK_SIZE = SCALE_VECTOR_SIZE


def is_mxfp6_b200_available() -> bool:
    """Whether the native library loads and the current device is an sm_100 GPU."""
    return is_available()


def is_problem_supported(output_features: int, input_features: int) -> bool:
    """The reference's rule for a linear partition (patch :136-140): N % 8, K % 128."""
    return output_features % 8 == 0 and input_features % 128 == 0


def pack_mxfp6_scales(logical_scales: torch.Tensor) -> torch.Tensor:
    """Logical UE8M0 ``[N, K/32]`` -> the kernels' 128 x 4 atoms, on the tensor's device."""
    return pack_scales_host(logical_scales.contiguous())


class MxFp6LinearKernel:
    """W6A8 linear layer over checkpoint tensors.

    ``layer.weight`` holds the packed E3M2 codes ``[N, 3K/4]`` (uint8) and
    ``layer.weight_scale`` the logical UE8M0 scales ``[N, K/32]`` as loaded;
    :meth:`process_weights_after_loading` replaces the latter with the packed layout once.
    """

    def __init__(self, output_size_per_partition: int, input_size_per_partition: int,
                 out_dtype: torch.dtype = torch.bfloat16):
        if not is_problem_supported(output_size_per_partition, input_size_per_partition):
            raise ValueError("the W6A8 kernels need N divisible by 8 and K by 128; got "
                             f"N={output_size_per_partition}, K={input_size_per_partition}")
        self.n = int(output_size_per_partition)
        self.k = int(input_size_per_partition)
        self.out_dtype = out_dtype

    def process_weights_after_loading(self, layer: torch.nn.Module) -> None:
        weight = layer.weight.data
        scale = layer.weight_scale.data
        if tuple(weight.shape) != (self.n, self.k * 3 // 4) or weight.dtype != torch.uint8:
            raise ValueError(f"weight must be uint8 [{self.n}, {self.k * 3 // 4}]")
        if tuple(scale.shape) != (self.n, self.k // OCP_MX_BLOCK_SIZE) or scale.dtype != torch.uint8:
            raise ValueError(f"weight_scale must be uint8 [{self.n}, {self.k // OCP_MX_BLOCK_SIZE}]")
        layer.weight = torch.nn.Parameter(weight.contiguous(), requires_grad=False)
        layer.weight_scale = torch.nn.Parameter(pack_mxfp6_scales(scale), requires_grad=False)

    def apply_weights(self, layer: torch.nn.Module, x: torch.Tensor,
                      bias: torch.Tensor | None = None) -> torch.Tensor:
        output_shape = (*x.shape[:-1], self.n)
        x_2d = x.reshape(-1, x.shape[-1]).contiguous()
        quantized_x, input_scale = torch.ops.mxfp6.quantize_mxfp8(x_2d)
        y = torch.ops.mxfp6.gemm_w6a8(quantized_x.view(torch.uint8), layer.weight, input_scale,
                                      layer.weight_scale, x_2d.shape[0], self.n, self.k, 1.0,
                                      self.out_dtype)
        if bias is not None:
            y = y + bias
        return y.reshape(output_shape)


@dataclass
class MxFp6MoERunner:
    """Routed experts + gated shared expert of one layer, with per-batch workspaces.

    Built from a :class:`~.checkpoint.MoeLayerCheckpoint` (this rank's slice).  ``forward``
    takes the hidden rows and computes the router itself (``combined_gate``), like the
    reference's runner; batches up to :data:`~.moe_layer.DECODE_MAX_TOKENS` take the decode
    schedule, larger ones the grouped schedule.  Workspaces are created on first use per batch
    size and reused, so a captured graph replays without allocating; larger inputs are
    processed in chunks of ``max_tokens``.
    """

    weights: MoeLayerCheckpoint
    topk: int = 8
    renormalize: bool = True
    max_tokens: int = 4096
    layer: MoeLayer = field(init=False)
    _states: dict[int, MoeLayerState] = field(init=False, default_factory=dict)
    _logits: dict[int, tuple[torch.Tensor, torch.Tensor]] = field(init=False, default_factory=dict)

    def __post_init__(self):
        self.layer = self.weights.moe_layer(self.topk)

    def _workspace(self, tokens: int) -> MoeLayerState:
        if tokens > self.max_tokens:
            raise RuntimeError(f"internal chunk exceeds {self.max_tokens} tokens: got {tokens}")
        if tokens not in self._states:
            device = self.weights.combined_gate.device
            self._states[tokens] = self.layer.workspace(tokens)
            self._logits[tokens] = (
                torch.empty((tokens, self.weights.experts), dtype=torch.bfloat16, device=device),
                torch.empty((tokens,), dtype=torch.bfloat16, device=device))
        return self._states[tokens]

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        """``[tokens, H]`` BF16 in, ``[tokens, H]`` BF16 out (this rank's partial under tensor
        parallelism: the caller sums the ranks, e.g. with ``moe_reduce_tp2_out``'s collective)."""
        total = int(hidden_states.shape[0])
        if total > self.max_tokens:
            # chunks of one size share a workspace: each result is copied out before the next runs
            out = torch.empty_like(hidden_states)
            for lo in range(0, total, self.max_tokens):
                out[lo: lo + self.max_tokens].copy_(self.forward(hidden_states[lo: lo + self.max_tokens]))
            return out
        state = self._workspace(total)
        logits, shared_gate = self._logits[total]
        hidden_states = hidden_states.contiguous()
        if state.decode is not None and total <= DECODE_MAX_TOKENS:
            # the router GEMV, then the decode schedule on its logits (two or three launches)
            from .moe_ops import router_logits_out
            from .qwen35 import qwen35_moe_decode_logits_out

            ws = state.decode
            router_logits_out(ws.routed_logits, ws.shared_gate, hidden_states, self.weights.combined_gate)
            e, i, h = self.weights.experts, self.weights.intermediate, self.weights.hidden
            lay = self.layer
            return qwen35_moe_decode_logits_out(
                ws, hidden_states, ws.routed_logits, ws.shared_gate,
                lay.w1.values.view(e, 2 * i, h * 3 // 4), lay.w1.scales,
                lay.w2.values.view(e, h, i * 3 // 4), lay.w2.scales, lay.shared_w1, lay.shared_w2,
                renormalize=self.renormalize)
        from ._loader import check, library
        from .ops import _stream

        with torch.cuda.device(hidden_states.device):
            check(library().mxfp6_moe_router_logits(
                hidden_states.data_ptr(), self.weights.combined_gate.data_ptr(), None, logits.data_ptr(),
                shared_gate.data_ptr(), total, self.weights.hidden, self.weights.experts,
                self.weights.experts + 1, _stream(hidden_states.device)))
        return self.layer.forward_grouped(state, hidden_states, logits, shared_gate,
                                          renormalize=self.renormalize)
