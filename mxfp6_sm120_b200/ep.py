"""Expert-parallel routed MoE across the GPUs of one node.

Experts are dealt to ranks in contiguous blocks (rank r owns experts
``[r * E / G, (r + 1) * E / G)``, the partition the reference's ``expert_map`` /
``local_experts`` hook describes, csrc/moe.cu:4243-4261).  Tokens are data parallel:
every rank brings its own ``B_local`` rows.

One exchange step each way, both with fixed shapes so the layer captures into a
CUDA graph:

* dispatch - every rank's MXFP8 rows (H bytes + H/32 scale bytes) and top-k
  ids/weights are exchanged with ``all_gather``: with top-8 of 256 experts over at
  most 8 ranks a token needs most ranks anyway, so the dense form of the
  all-to-all costs at most ~1.5x the exact one and needs no capacity padding;
* local work - routing keeps only the routes whose expert is local
  (``expert_map``), grouped W1 (fused SiLU*mul + MXFP8) and W2 run on them, and the
  reducer forms this rank's partial output for EVERY token;
* combine - ``all_to_all_single`` sends each source rank the partial rows of its
  own tokens; a final reduce sums the G partials in rank order and adds the gated
  shared expert, which each rank computes for its own tokens only.

Top-k is computed once per token by its source rank.  The collectives run on the
compute stream through ``torch.distributed`` (NCCL over NVLink).
"""

from __future__ import annotations

from dataclasses import dataclass, replace

import torch
import torch.distributed as dist

from .moe_layer import MoeLayer
from .moe_ops import moe_reduce_out, qwen35_route_mxfp8_out, qwen35_topk_quant_out
from .ops import PackedMXFP6Tensor, packed_scale_numel
from .qwen35 import (
    MoeShape,
    Qwen35GroupedWorkspace,
    SharedExpertWorkspace,
    _grouped_experts_out,
    shared_expert_out,
)


def expert_range(experts: int, world: int, rank: int) -> tuple[int, int]:
    """Experts ``[begin, end)`` owned by ``rank`` (contiguous, as even as possible)."""
    base, extra = divmod(experts, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def make_expert_map(experts: int, world: int, rank: int, device) -> torch.Tensor:
    """int32 ``[experts]``: global expert id -> local id on this rank, or -1."""
    begin, end = expert_range(experts, world, rank)
    table = torch.full((experts,), -1, dtype=torch.int32)
    table[begin:end] = torch.arange(end - begin, dtype=torch.int32)
    return table.to(device)


def shard_expert_weights(weight: PackedMXFP6Tensor, experts: int, world: int,
                         rank: int) -> PackedMXFP6Tensor:
    """Rows of ``[E * rows_per_expert, K]`` packed weights that belong to this rank."""
    begin, end = expert_range(experts, world, rank)
    rows_per_expert = weight.rows // experts
    if rows_per_expert % 128:
        raise ValueError("expert matrices must have a multiple of 128 rows")
    row_bytes = weight.k * 3 // 4
    scale_bytes_per_row_block = ((weight.k // 32 + 3) // 4) * 512
    lo, hi = begin * rows_per_expert, end * rows_per_expert
    return PackedMXFP6Tensor(
        weight.values[lo * row_bytes : hi * row_bytes],
        weight.scales[lo // 128 * scale_bytes_per_row_block : hi // 128 * scale_bytes_per_row_block],
        hi - lo,
        weight.k,
    )


@dataclass
class EpState:
    """Fixed-shape buffers of one expert-parallel layer call."""

    local: Qwen35GroupedWorkspace        # quantization + top-k of this rank's tokens
    gathered: Qwen35GroupedWorkspace     # routing / experts over the tokens of all ranks
    shared: SharedExpertWorkspace
    partial: torch.Tensor                # [G * B_local, H] this rank's partial for every token
    received: torch.Tensor               # [G * B_local, H] partials of my tokens from every rank
    ones: torch.Tensor                   # [B_local, G] combine weights
    gather_index: torch.Tensor           # [B_local * G] row of partial g for token t
    output: torch.Tensor
    # peer-memory exchange (decode batches): dispatch payload offsets in buffer 0 of the
    # symmetric block, the summed partial rows of this rank's tokens, and a trivial index
    dispatch: tuple | None = None
    combined: torch.Tensor | None = None
    identity: torch.Tensor | None = None
    # the shared expert of this rank's tokens runs beside the exchange and the routed experts
    side_stream: object | None = None
    fork: object | None = None
    join: object | None = None


class ExpertParallelMoe:
    """One MoE layer whose routed experts are sharded over ``group``."""

    # Up to this many tokens over all ranks the two exchanges run as one peer-memory kernel
    # each (tp_fused.SymmetricBlocks) instead of four all-gathers and an all-to-all: five
    # NCCL launches cost about 185 us of a 310 us layer at 4096 tokens on 8 GPUs, where the
    # bytes themselves (7.7 MB gathered, 14.7 MB summed per rank) are worth about 40 us.
    PEER_MAX_TOKENS = 4096

    def __init__(self, layer: MoeLayer, group=None, peer=None):
        self.group = group
        self.peer = peer
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.shape = layer.shape
        device = layer.w1.values.device
        experts = layer.shape.experts
        self.w1 = shard_expert_weights(layer.w1, experts, self.world, self.rank)
        self.w2 = shard_expert_weights(layer.w2, experts, self.world, self.rank)
        self.shared_w1, self.shared_w2 = layer.shared_w1, layer.shared_w2
        self.local_experts = self.w1.rows // (2 * layer.shape.intermediate)
        self.expert_map = make_expert_map(experts, self.world, self.rank, device)

    def state(self, local_tokens: int) -> EpState:
        device = self.w1.values.device
        shape, world = self.shape, self.world
        total = local_tokens * world
        local_shape = MoeShape(shape.hidden, shape.intermediate, self.local_experts, shape.topk)
        index = (torch.arange(world).view(1, world) * local_tokens
                 + torch.arange(local_tokens).view(local_tokens, 1)).reshape(-1)
        if self.peer is not None and world > 1 and total <= self.PEER_MAX_TOKENS:
            return self._peer_state(local_tokens, local_shape, index)
        return EpState(
            Qwen35GroupedWorkspace.allocate(local_tokens, device, shape),
            Qwen35GroupedWorkspace.allocate(total, device, local_shape),
            SharedExpertWorkspace.allocate(local_tokens, device, shape),
            torch.empty((total, shape.hidden), dtype=torch.bfloat16, device=device),
            torch.empty((total, shape.hidden), dtype=torch.bfloat16, device=device),
            torch.ones((local_tokens, world), dtype=torch.float32, device=device),
            index.to(torch.int32).to(device),
            torch.empty((local_tokens, shape.hidden), dtype=torch.bfloat16, device=device),
            side_stream=torch.cuda.Stream(device) if device.type == "cuda" else None,
            fork=torch.cuda.Event() if device.type == "cuda" else None,
            join=torch.cuda.Event() if device.type == "cuda" else None,
        )

    def _peer_state(self, local_tokens: int, local_shape: MoeShape, index: torch.Tensor) -> EpState:
        """State whose exchanged tensors live in the symmetric block: this rank's MXFP8 rows,
        scale rows, top-k ids and weights in buffer 0 (written in place by the top-k kernel),
        its partial outputs for every token in buffer 1."""
        device = self.w1.values.device
        shape, world, peer = self.shape, self.world, self.peer
        total = local_tokens * world

        def align(v: int) -> int:
            return (v + 255) // 256 * 256

        q_bytes = local_tokens * shape.hidden
        s_bytes = local_tokens * shape.hidden // 32
        k_bytes = local_tokens * shape.topk * 4
        off_q, off_s = 0, align(q_bytes)
        off_i = off_s + align(s_bytes)
        off_w = off_i + align(k_bytes)
        local = Qwen35GroupedWorkspace.allocate(local_tokens, device, shape)
        local = replace(
            local,
            quantized=peer.view(0, off_q, (local_tokens, shape.hidden), torch.uint8),
            input_scales=peer.view(0, off_s, (local_tokens, shape.hidden // 32), torch.uint8),
            topk_ids=peer.view(0, off_i, (local_tokens, shape.topk), torch.int32),
            topk_weights=peer.view(0, off_w, (local_tokens, shape.topk), torch.float32),
        )
        return EpState(
            local,
            Qwen35GroupedWorkspace.allocate(total, device, local_shape),
            SharedExpertWorkspace.allocate(local_tokens, device, shape),
            peer.view(1, 0, (total, shape.hidden), torch.bfloat16),
            torch.empty((0,), dtype=torch.bfloat16, device=device),
            torch.ones((local_tokens, 1), dtype=torch.float32, device=device),
            index.to(torch.int32).to(device),
            torch.empty((local_tokens, shape.hidden), dtype=torch.bfloat16, device=device),
            dispatch=(off_q, off_s, off_i, off_w),
            combined=torch.empty((local_tokens, shape.hidden), dtype=torch.bfloat16, device=device),
            identity=torch.arange(local_tokens, dtype=torch.int32, device=device),
            side_stream=torch.cuda.Stream(device),
            fork=torch.cuda.Event(),
            join=torch.cuda.Event(),
        )

    def forward(self, state: EpState, hidden: torch.Tensor, router_logits: torch.Tensor,
                shared_gate: torch.Tensor | None) -> torch.Tensor:
        shape = self.shape
        loc, ws = state.local, state.gathered
        e, i, h = self.local_experts, shape.intermediate, shape.hidden
        # 1. quantize + top-k on this rank's tokens
        qwen35_topk_quant_out(loc.quantized, loc.input_scales, loc.packed_input_scales,
                              loc.topk_weights, loc.topk_ids, hidden, router_logits,
                              renormalize=True)
        # The shared expert needs only this rank's quantized rows: it runs on a side stream
        # from here to the final reduce (under capture both branches land in the one graph).
        shared_out = None
        if state.side_stream is not None:
            current = torch.cuda.current_stream(hidden.device)
            state.fork.record(current)
            state.side_stream.wait_event(state.fork)
            with torch.cuda.stream(state.side_stream):
                shared_out = shared_expert_out(state.shared, loc, self.shared_w1, self.shared_w2)
                state.join.record(state.side_stream)
        # 2. dispatch: rows, scales, ids and weights of every rank
        if state.dispatch is not None:
            off_q, off_s, off_i, off_w = state.dispatch
            self.peer.allgather(0, [(off_q, ws.quantized), (off_s, ws.input_scales),
                                    (off_i, ws.topk_ids), (off_w, ws.topk_weights)])
        elif self.world > 1:
            dist.all_gather_into_tensor(ws.quantized, loc.quantized, group=self.group)
            dist.all_gather_into_tensor(ws.input_scales, loc.input_scales, group=self.group)
            dist.all_gather_into_tensor(ws.topk_ids, loc.topk_ids, group=self.group)
            dist.all_gather_into_tensor(ws.topk_weights, loc.topk_weights, group=self.group)
        else:
            ws.quantized.copy_(loc.quantized)
            ws.input_scales.copy_(loc.input_scales)
            ws.topk_ids.copy_(loc.topk_ids)
            ws.topk_weights.copy_(loc.topk_weights)
        # 3. local experts only: routes of other ranks' experts get inverse = -1
        qwen35_route_mxfp8_out(ws.quantized, ws.input_scales, ws.topk_ids, ws.permuted,
                               ws.grouped_input_scales, ws.expert_cursors, ws.expert_offsets,
                               ws.scale_offsets, ws.inverse_permutation,
                               source_tokens=ws.source_tokens, expert_map=self.expert_map)
        _grouped_experts_out(ws, self.w1.values.view(e, 2 * i, h * 3 // 4), self.w1.scales,
                             self.w2.values.view(e, h, i * 3 // 4), self.w2.scales)
        moe_reduce_out(state.partial, ws.routed_output, ws.topk_weights, ws.inverse_permutation)
        # 4. combine: partial rows of my tokens from every rank
        if state.dispatch is not None:
            # one kernel sums them over peer memory; the shared expert joins in the last reduce
            self.peer.reduce_scatter(1, state.combined)
            shared_out = self._join_shared(state, loc, shared_out, hidden.device)
            moe_reduce_out(state.output, state.combined, state.ones, state.identity, shared_out,
                           shared_gate)
            return state.output
        if self.world > 1:
            dist.all_to_all_single(state.received, state.partial, group=self.group)
        else:
            state.received.copy_(state.partial)
        # 5. shared expert on my tokens, then the final sum in rank order
        shared_out = self._join_shared(state, loc, shared_out, hidden.device)
        moe_reduce_out(state.output, state.received, state.ones, state.gather_index, shared_out,
                       shared_gate)
        return state.output

    def _join_shared(self, state: EpState, loc, shared_out, device):
        if state.side_stream is not None:
            torch.cuda.current_stream(device).wait_event(state.join)
            return shared_out
        return shared_expert_out(state.shared, loc, self.shared_w1, self.shared_w2)
