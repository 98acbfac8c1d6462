"""One routed-MoE layer (routed experts + always-on shared expert) as a single object.

The caller side of the grouped schedule: weights, workspaces and one ``forward`` that
queues the whole layer on the current stream without allocating, so it captures into
one CUDA graph.  The reference leaves this composition to its benchmark
(benchmarks/benchmark_qwen35_moe_layer.py:1102-1127,1401-1403,1524-1549).
"""

from __future__ import annotations

from dataclasses import dataclass, replace

import torch

from .ops import PackedMXFP6Tensor, quantize_mxfp6
from .moe_ops import qwen35_topk_quant_route_out
from .qwen35 import (
    MoeShape,
    Qwen35GroupedWorkspace,
    Qwen35MoeB1Workspace,
    SharedExpertWorkspace,
    _grouped_experts_out,
    qwen35_grouped_reduce_out,
    qwen35_moe_decode_logits_out,
    shared_expert_out,
)

# Batches of at most this many tokens take the decode schedule (one single-row GEMM per
# route, three launches); larger ones the grouped schedule.  Measured on a B200 with the
# named configuration (hidden 2048, 256 experts, top-8, intermediate 512), warm, decode
# against grouped: 16.5 / 35 us at 1 token, 36.9 / 66 at 8, 59 / 82 at 16, 111 / 115 at 32;
# beyond that the grouped schedule reads every expert once and wins.
DECODE_MAX_TOKENS = 32


@dataclass
class MoeLayerState:
    workspace: Qwen35GroupedWorkspace
    shared: SharedExpertWorkspace
    output: torch.Tensor
    side_stream: torch.cuda.Stream | None = None
    fork: torch.cuda.Event | None = None
    join: torch.cuda.Event | None = None
    decode: Qwen35MoeB1Workspace | None = None   # batches of up to DECODE_MAX_TOKENS tokens


@dataclass
class MoeLayer:
    shape: MoeShape
    w1: PackedMXFP6Tensor          # [E * 2I, H]: per expert gate rows then up rows
    w2: PackedMXFP6Tensor          # [E * H, I]
    shared_w1: PackedMXFP6Tensor   # [2I, H]
    shared_w2: PackedMXFP6Tensor   # [H, I]
    expert_map: torch.Tensor | None = None  # global expert id -> local id or -1 (expert parallel)

    @classmethod
    def random(cls, device, shape: MoeShape = MoeShape(), seed: int = 4000, experts: int | None = None):
        """Weights ~ N(0, 0.02) quantized to packed MXFP6 on the device."""
        gen = torch.Generator(device=device).manual_seed(seed)
        h, i = shape.hidden, shape.intermediate
        e = shape.experts if experts is None else experts

        def make(rows, cols):
            chunks = []
            step = max(1, (1 << 26) // cols)  # quantize in slabs to bound the BF16 staging memory
            for lo in range(0, rows, step):
                n = min(step, rows - lo)
                w = (torch.randn((n, cols), generator=gen, device=device) * 0.02).to(torch.bfloat16)
                chunks.append(quantize_mxfp6(w))
            if len(chunks) == 1:
                return chunks[0]
            assert step % 128 == 0
            return PackedMXFP6Tensor(torch.cat([c.values for c in chunks]),
                                     torch.cat([c.scales for c in chunks]), rows, cols)

        return cls(shape, make(e * 2 * i, h), make(e * h, i), make(2 * i, h), make(h, i))

    @property
    def local_experts(self) -> int:
        return self.w1.rows // (2 * self.shape.intermediate)

    def workspace(self, tokens: int) -> MoeLayerState:
        device = self.w1.values.device
        local = MoeShape(self.shape.hidden, self.shape.intermediate, self.local_experts, self.shape.topk)
        output = torch.empty((tokens, self.shape.hidden), dtype=torch.bfloat16, device=device)
        decode = None
        if self._decode_applies(tokens):
            decode = replace(Qwen35MoeB1Workspace.allocate(device, local, batch=tokens), output=output)
        return MoeLayerState(
            Qwen35GroupedWorkspace.allocate(tokens, device, local),
            SharedExpertWorkspace.allocate(tokens, device, self.shape),
            output,
            torch.cuda.Stream(device) if device.type == "cuda" else None,
            torch.cuda.Event() if device.type == "cuda" else None,
            torch.cuda.Event() if device.type == "cuda" else None,
            decode,
        )

    def _decode_applies(self, tokens: int) -> bool:
        # the reduce kernel keeps one accumulator per route of a token: top-8 + shared at most,
        # and a down projection of at most 2048 inputs
        return (tokens <= DECODE_MAX_TOKENS and self.expert_map is None and self.shape.topk <= 8
                and self.shape.intermediate <= 2048 and self.shape.intermediate % 128 == 0
                and self.shape.hidden % 128 == 0 and self.shape.hidden <= 8192)

    def forward(self, state: MoeLayerState, hidden: torch.Tensor, router_logits: torch.Tensor,
                shared_gate: torch.Tensor | None, with_shared: bool = True) -> torch.Tensor:
        """Queue the layer on the current stream without allocating: the decode schedule
        for small batches, the grouped schedule otherwise."""
        if state.decode is not None and with_shared and shared_gate is not None:
            return self.forward_decode(state, hidden, router_logits, shared_gate)
        return self.forward_grouped(state, hidden, router_logits, shared_gate, with_shared)

    def forward_decode(self, state: MoeLayerState, hidden: torch.Tensor, router_logits: torch.Tensor,
                       shared_gate: torch.Tensor) -> torch.Tensor:
        """Three launches: top-k + quantization, W1 routes with SwiGLU, W2 routes + reduce;
        the shared expert is one more route of every token."""
        e, i, h = self.local_experts, self.shape.intermediate, self.shape.hidden
        return qwen35_moe_decode_logits_out(
            state.decode, hidden, router_logits, shared_gate,
            self.w1.values.view(e, 2 * i, h * 3 // 4), self.w1.scales,
            self.w2.values.view(e, h, i * 3 // 4), self.w2.scales, self.shared_w1, self.shared_w2,
            renormalize=True)

    def forward_grouped(self, state: MoeLayerState, hidden: torch.Tensor, router_logits: torch.Tensor,
                        shared_gate: torch.Tensor | None, with_shared: bool = True,
                        renormalize: bool = True) -> torch.Tensor:
        """The grouped schedule.  The shared expert runs on a side
        stream between the quantization and the final reduce (the reference's
        benchmark overlaps it the same way); under capture both branches land in
        the one graph."""
        e, i, h = self.local_experts, self.shape.intermediate, self.shape.hidden
        ws = state.workspace
        qwen35_topk_quant_route_out(
            ws.quantized, ws.input_scales, ws.packed_input_scales, ws.topk_weights, ws.topk_ids,
            ws.permuted, ws.grouped_input_scales, ws.expert_cursors, ws.expert_offsets,
            ws.scale_offsets, ws.inverse_permutation, hidden, router_logits,
            source_tokens=ws.source_tokens, renormalize=renormalize, expert_map=self.expert_map)
        shared_out = None
        overlap = with_shared and state.side_stream is not None
        if overlap:
            current = torch.cuda.current_stream(hidden.device)
            state.fork.record(current)
            state.side_stream.wait_event(state.fork)
            with torch.cuda.stream(state.side_stream):
                shared_out = shared_expert_out(state.shared, ws, self.shared_w1, self.shared_w2)
                state.join.record(state.side_stream)
        _grouped_experts_out(ws, self.w1.values.view(e, 2 * i, h * 3 // 4), self.w1.scales,
                             self.w2.values.view(e, h, i * 3 // 4), self.w2.scales)
        if overlap:
            torch.cuda.current_stream(hidden.device).wait_event(state.join)
        elif with_shared:
            shared_out = shared_expert_out(state.shared, ws, self.shared_w1, self.shared_w2)
        return qwen35_grouped_reduce_out(ws, state.output, shared_out,
                                         shared_gate if with_shared else None)
