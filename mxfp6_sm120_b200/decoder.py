"""Decode / prefill step of a dense decoder whose linears all run W6A8.

The reference stops at the operator surface and leaves the model step to its serving
runtime (docs/runtime-integration.md:13-22); its benchmarks name the projection shapes
of a 27B-class decoder (benchmarks/model_shapes.py:9-15).  This module is the caller
side of those shapes: per layer

    x  -> [residual add +] RMSNorm + MXFP8 quantize (one kernel)
       -> QKV projection (W6A8 GEMM) -> BF16 attention (torch SDPA, grouped-query)
       -> MXFP8 quantize -> output projection (W6A8, row-parallel + all-reduce under TP)
       -> residual add + RMSNorm + MXFP8 quantize (one kernel)
       -> gate/up projection with fused SiLU*mul + MXFP8 (or GEMM + activation kernel for
          prefill batches) -> down projection (W6A8, row-parallel + all-reduce under TP)

with every buffer preallocated so that the whole step captures into one CUDA graph.
Tensor parallelism splits attention heads and the MLP intermediate over the ranks of
one node (column-parallel QKV and gate/up, row-parallel output and down projections).
No rotary embedding is applied: attention is the plain BF16 kernel the benchmark
configuration asks for.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn.functional as F

from .moe_ops import dense_w1_silu_mxfp8_out, silu_and_mul_mxfp8_packed_out
from .ops import (
    MXFP8Tensor,
    PackedMXFP6Tensor,
    _quantize_mxfp8_raw,
    gemm_w6a8,
    packed_scale_numel,
    quantize_mxfp6,
    rmsnorm_quantize_mxfp8,
)

# Up to this many tokens the row-parallel projections are reduced inside the norm kernel over
# peer memory (a decode batch: the flag round trip and a few KB per row); larger batches are
# bandwidth-bound collectives and go through NCCL (8192 tokens, 2 GPUs: 194 ms against 202 ms).
PEER_ALLREDUCE_MAX_TOKENS = 512

# From this many tokens on the gate/up projection runs as a plain GEMM followed by the
# activation kernel (the fused epilogue's four warps per SM become the bottleneck).
UNFUSED_MLP_MIN_TOKENS = 2048


@dataclass(frozen=True)
class DecoderConfig:
    """27B-class dense decoder of the benchmark configuration."""

    hidden: int = 5120
    q_heads: int = 24
    kv_heads: int = 4
    head_dim: int = 256
    intermediate: int = 17408
    layers: int = 64
    eps: float = 1e-6

    def local(self, world: int) -> "LocalShape":
        if self.q_heads % world or self.intermediate % (128 * world):
            raise ValueError(f"{world} ranks do not divide the heads / intermediate size")
        # Fewer KV heads than ranks: ranks share (replicate) a KV head.
        kv = self.kv_heads // world if self.kv_heads % world == 0 else 1
        if self.kv_heads % world and world % self.kv_heads:
            raise ValueError(f"{world} ranks do not divide or multiply the KV heads")
        q = self.q_heads // world
        if (q * self.head_dim) % 128 or (kv * self.head_dim) % 128:
            raise ValueError("per-rank head blocks must be multiples of 128 features")
        return LocalShape(q, kv, self.intermediate // world)


@dataclass(frozen=True)
class LocalShape:
    q_heads: int
    kv_heads: int
    intermediate: int


@dataclass
class DecoderLayer:
    """One rank's weights of a layer."""

    ln1: torch.Tensor                # [hidden] BF16
    ln2: torch.Tensor
    qkv: PackedMXFP6Tensor           # [(q + 2 kv) * head_dim, hidden], q rows, k rows, v rows
    o: PackedMXFP6Tensor             # [hidden, q * head_dim]
    gate_up: PackedMXFP6Tensor       # [2 * inter, hidden], gate rows then up rows
    down: PackedMXFP6Tensor          # [hidden, inter]


def _slice_rows(weight: PackedMXFP6Tensor, begin: int, end: int) -> PackedMXFP6Tensor:
    """Rows ``[begin, end)`` (multiples of 128) of a packed weight: contiguous bytes."""
    row_bytes = weight.k * 3 // 4
    block = ((weight.k // 32 + 3) // 4) * 512
    return PackedMXFP6Tensor(weight.values.view(-1)[begin * row_bytes : end * row_bytes],
                             weight.scales.view(-1)[begin // 128 * block : end // 128 * block],
                             end - begin, weight.k)


def _cat_rows(parts: list[PackedMXFP6Tensor]) -> PackedMXFP6Tensor:
    return PackedMXFP6Tensor(torch.cat([p.values.view(-1) for p in parts]),
                             torch.cat([p.scales.view(-1) for p in parts]),
                             sum(p.rows for p in parts), parts[0].k)


def shard_layer(layer: DecoderLayer, cfg: DecoderConfig, world: int, rank: int) -> DecoderLayer:
    """This rank's slice of a full layer: heads and intermediate columns in contiguous
    blocks; output and down projections are split along K (row-parallel)."""
    from .tp import shard_row_parallel

    if world == 1:
        return layer
    loc = cfg.local(world)
    hd = cfg.head_dim
    q0 = rank * loc.q_heads * hd
    kv_index = rank * cfg.kv_heads // world          # shared head when kv_heads < world
    k_base = cfg.q_heads * hd
    v_base = k_base + cfg.kv_heads * hd
    kv0 = kv_index * hd if cfg.kv_heads < world else rank * loc.kv_heads * hd
    qkv = _cat_rows([
        _slice_rows(layer.qkv, q0, q0 + loc.q_heads * hd),
        _slice_rows(layer.qkv, k_base + kv0, k_base + kv0 + loc.kv_heads * hd),
        _slice_rows(layer.qkv, v_base + kv0, v_base + kv0 + loc.kv_heads * hd),
    ])
    i0 = rank * loc.intermediate
    gate_up = _cat_rows([
        _slice_rows(layer.gate_up, i0, i0 + loc.intermediate),
        _slice_rows(layer.gate_up, cfg.intermediate + i0, cfg.intermediate + i0 + loc.intermediate),
    ])

    def row_parallel(weight: PackedMXFP6Tensor) -> PackedMXFP6Tensor:
        shard = shard_row_parallel(weight.values, weight.scales, weight.rows, weight.k, world, rank)
        return PackedMXFP6Tensor(shard.values, shard.scales, shard.rows, shard.k)

    return DecoderLayer(layer.ln1, layer.ln2, qkv, row_parallel(layer.o), gate_up,
                        row_parallel(layer.down))


def random_layer(cfg: DecoderConfig, device, generator: torch.Generator,
                 shape: LocalShape | None = None) -> DecoderLayer:
    """Random-init layer (weights N(0, 0.02), norm weights near 1) of ``shape`` (default: the
    full, unsharded sizes), quantized to MXFP6 on the GPU."""
    shape = shape or cfg.local(1)
    hd, h = cfg.head_dim, cfg.hidden

    def weight(rows: int, k: int) -> PackedMXFP6Tensor:
        # Generated in row blocks so that the BF16 staging stays small beside 64 layers.
        parts = []
        step = max(128, (1 << 25) // k // 128 * 128)
        for r0 in range(0, rows, step):
            r = min(step, rows - r0)
            w = torch.randn((r, k), generator=generator, device=device, dtype=torch.float32)
            parts.append(quantize_mxfp6((w * 0.02).to(torch.bfloat16)))
        return parts[0] if len(parts) == 1 else _cat_rows(parts)

    def norm() -> torch.Tensor:
        n = torch.randn((h,), generator=generator, device=device, dtype=torch.float32)
        return (1.0 + 0.1 * n).to(torch.bfloat16)

    return DecoderLayer(norm(), norm(),
                        weight((shape.q_heads + 2 * shape.kv_heads) * hd, h),
                        weight(h, shape.q_heads * hd),
                        weight(2 * shape.intermediate, h),
                        weight(h, shape.intermediate))


@dataclass
class DecoderWorkspace:
    """Preallocated buffers of one step for a fixed token count."""

    tokens: int
    x: torch.Tensor               # [T, hidden] BF16 residual stream (input, updated in place)
    a_values: torch.Tensor        # MXFP8 of the normalised activation, K = hidden
    a_scales: torch.Tensor
    qkv: torch.Tensor             # [T, (q + 2 kv) * head_dim] BF16
    attn: torch.Tensor            # [T, q * head_dim] BF16
    b_values: torch.Tensor        # MXFP8 of attn, K = q * head_dim
    b_scales: torch.Tensor
    proj: torch.Tensor            # [T, hidden] BF16 output of the o / down projections
    mlp_values: torch.Tensor      # [T, inter] MXFP8 of silu(gate) * up
    mlp_scales: torch.Tensor
    gate_up: torch.Tensor | None  # [T, 2 * inter] BF16, prefill batches only


class DenseDecoder:
    """``layers`` decoder layers of one rank, with the step functions."""

    def __init__(self, cfg: DecoderConfig, layers: list[DecoderLayer], world: int = 1,
                 rank: int = 0, group=None, peer=None):
        self.cfg, self.layers, self.world, self.rank, self.group = cfg, layers, world, rank, group
        self.shape = cfg.local(world)
        self.device = layers[0].ln1.device
        # tp_fused.SymmetricBlocks: the two all-reduces of a layer run inside the following
        # residual + norm + quantize kernel over peer memory instead of NCCL.
        self.peer = peer

    @classmethod
    def random(cls, cfg: DecoderConfig, device, seed: int = 5000, world: int = 1, rank: int = 0,
               group=None, layers: int | None = None, peer=None) -> "DenseDecoder":
        """Random-init decoder; under TP every rank draws its own local-shape weights."""
        gen = torch.Generator(device=device).manual_seed(seed + rank)
        shape = cfg.local(world)
        count = cfg.layers if layers is None else layers
        return cls(cfg, [random_layer(cfg, device, gen, shape) for _ in range(count)], world, rank,
                   group, peer)

    def weight_bytes(self) -> int:
        total = 0
        for layer in self.layers:
            for w in (layer.qkv, layer.o, layer.gate_up, layer.down):
                total += w.values.numel() + w.scales.numel()
        return total

    def workspace(self, tokens: int) -> DecoderWorkspace:
        cfg, shape, dev = self.cfg, self.shape, self.device
        hd = cfg.head_dim
        qkv_n = (shape.q_heads + 2 * shape.kv_heads) * hd
        attn_k = shape.q_heads * hd
        u8 = dict(dtype=torch.uint8, device=dev)
        bf = dict(dtype=torch.bfloat16, device=dev)
        unfused = tokens >= UNFUSED_MLP_MIN_TOKENS
        return DecoderWorkspace(
            tokens,
            torch.zeros((tokens, cfg.hidden), **bf),
            torch.empty(tokens * cfg.hidden, **u8),
            torch.empty(packed_scale_numel(tokens, cfg.hidden), **u8),
            torch.empty((tokens, qkv_n), **bf),
            torch.empty((tokens, attn_k), **bf),
            torch.empty(tokens * attn_k, **u8),
            torch.empty(packed_scale_numel(tokens, attn_k), **u8),
            torch.empty((tokens, cfg.hidden), **bf),
            torch.empty((tokens, shape.intermediate), **u8),
            torch.empty(packed_scale_numel(tokens, shape.intermediate), **u8),
            torch.empty((tokens, 2 * shape.intermediate), **bf) if unfused else None,
        )

    def new_kv_cache(self, batch: int, context: int) -> list[tuple[torch.Tensor, torch.Tensor]]:
        """Per layer ``(k, v)`` of ``[batch, kv_heads, context, head_dim]`` BF16 (random fill)."""
        gen = torch.Generator(device=self.device).manual_seed(7000 + self.rank)
        shape = (batch, self.shape.kv_heads, context, self.cfg.head_dim)
        cache = []
        for _ in self.layers:
            k = torch.randn(shape, generator=gen, device=self.device, dtype=torch.bfloat16)
            v = torch.randn(shape, generator=gen, device=self.device, dtype=torch.bfloat16)
            cache.append((k, v))
        return cache

    # ------------------------------------------------------------------ one layer
    def _all_reduce(self, tensor: torch.Tensor) -> None:
        if self.world > 1:
            dist.all_reduce(tensor, group=self.group)

    def _projection_out(self, ws: DecoderWorkspace) -> torch.Tensor:
        """Where a row-parallel projection writes: the next peer buffer, or ws.proj."""
        if self._use_peer(ws):
            return self.peer.next_partial(ws.tokens, self.cfg.hidden)
        return ws.proj

    def _use_peer(self, ws: DecoderWorkspace) -> bool:
        return self.peer is not None and ws.tokens <= PEER_ALLREDUCE_MAX_TOKENS

    def _add_norm_quantize(self, ws: DecoderWorkspace, weight: torch.Tensor) -> MXFP8Tensor:
        """x += (all-reduced) projection output; returns MXFP8(RMSNorm(x) * weight)."""
        if self._use_peer(ws):
            return self.peer.allreduce_rmsnorm_quantize(ws.x, weight, self.cfg.eps, ws.a_values,
                                                        ws.a_scales)
        self._all_reduce(ws.proj)
        return rmsnorm_quantize_mxfp8(ws.x, weight, self.cfg.eps, residual=ws.proj,
                                      values=ws.a_values, scales=ws.a_scales)

    def _layer(self, ws: DecoderWorkspace, layer: DecoderLayer, attention, first: bool) -> None:
        cfg, shape = self.cfg, self.shape
        tokens, hd = ws.tokens, cfg.head_dim
        # x (+ down projection of the previous layer) -> norm -> MXFP8
        if first:
            a = rmsnorm_quantize_mxfp8(ws.x, layer.ln1, cfg.eps, values=ws.a_values,
                                       scales=ws.a_scales)
        else:
            a = self._add_norm_quantize(ws, layer.ln1)
        gemm_w6a8(a, layer.qkv, out_dtype=torch.bfloat16, out=ws.qkv)
        q_dim, kv_dim = shape.q_heads * hd, shape.kv_heads * hd
        q = ws.qkv[:, :q_dim].view(tokens, shape.q_heads, hd)
        k = ws.qkv[:, q_dim : q_dim + kv_dim].view(tokens, shape.kv_heads, hd)
        v = ws.qkv[:, q_dim + kv_dim :].view(tokens, shape.kv_heads, hd)
        attention(q, k, v, ws.attn)
        _quantize_mxfp8_raw(ws.attn, ws.b_values, ws.b_scales, None)
        b = MXFP8Tensor(ws.b_values, ws.b_scales, tokens, q_dim)
        gemm_w6a8(b, layer.o, out_dtype=torch.bfloat16, out=self._projection_out(ws))
        # x += attention output -> norm -> MXFP8
        a = self._add_norm_quantize(ws, layer.ln2)
        if ws.gate_up is not None:
            gemm_w6a8(a, layer.gate_up, out_dtype=torch.bfloat16, out=ws.gate_up)
            silu_and_mul_mxfp8_packed_out(ws.mlp_values, ws.mlp_scales, ws.gate_up)
        else:
            dense_w1_silu_mxfp8_out(ws.mlp_values, ws.mlp_scales,
                                    ws.a_values.view(tokens, cfg.hidden), ws.a_scales,
                                    layer.gate_up.values, layer.gate_up.scales)
        m = MXFP8Tensor(ws.mlp_values.view(-1), ws.mlp_scales, tokens, shape.intermediate)
        gemm_w6a8(m, layer.down, out_dtype=torch.bfloat16, out=self._projection_out(ws))

    def _run(self, ws: DecoderWorkspace, attention_of_layer) -> torch.Tensor:
        for index, layer in enumerate(self.layers):
            self._layer(ws, layer, attention_of_layer(index), index == 0)
        # The last layer's MLP output joins the residual stream.
        if self._use_peer(ws):
            # Same kernel; its normalised output (against the first layer's weight) is unused.
            self._add_norm_quantize(ws, self.layers[0].ln1)
        else:
            self._all_reduce(ws.proj)
            ws.x.add_(ws.proj)
        return ws.x

    # ------------------------------------------------------------------ the two steps
    def decode_step(self, ws: DecoderWorkspace, cache: list[tuple[torch.Tensor, torch.Tensor]],
                    position: int) -> torch.Tensor:
        """One new token for each of ``ws.tokens`` sequences: ``ws.x`` holds their hidden
        states and is updated in place; ``cache[layer]`` rows ``[:, :, :position]`` are the
        context and row ``position`` receives the new key / value."""
        def attention_of_layer(index: int):
            k_cache, v_cache = cache[index]

            def attention(q, k, v, out):
                k_cache[:, :, position].copy_(k)
                v_cache[:, :, position].copy_(v)
                o = F.scaled_dot_product_attention(
                    q.unsqueeze(2), k_cache[:, :, : position + 1], v_cache[:, :, : position + 1],
                    enable_gqa=True)
                out.view(q.shape[0], q.shape[1], q.shape[2]).copy_(o.squeeze(2))

            return attention

        return self._run(ws, attention_of_layer)

    def prefill(self, ws: DecoderWorkspace) -> torch.Tensor:
        """Causal self-attention over the ``ws.tokens`` tokens of ONE sequence in ``ws.x``."""
        def attention_of_layer(index: int):
            def attention(q, k, v, out):
                o = F.scaled_dot_product_attention(
                    q.transpose(0, 1).unsqueeze(0), k.transpose(0, 1).unsqueeze(0),
                    v.transpose(0, 1).unsqueeze(0), is_causal=True, enable_gqa=True)
                out.view(q.shape[0], q.shape[1], q.shape[2]).copy_(o.squeeze(0).transpose(0, 1))

            return attention

        return self._run(ws, attention_of_layer)
