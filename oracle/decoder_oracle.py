"""CPU restatement of the dense decoder step (test infrastructure, not a product path).

Only tests may import this module.  Every linear is the decoded-FP32 matmul the reference's
tests use as ground truth (tests/test_ops.py:1426-1443) on MXFP8-quantized activations
(csrc/quantization.cu:96-144) and decoded MXFP6 weights; the layer around it (RMSNorm with one
rounding, BF16 residual stream, grouped-query attention in FP32 on BF16 operands, SiLU*mul with
the reference's BF16 roundings, csrc/moe.cu:5199-5205) is what `mxfp6_sm120_b200/decoder.py`
runs on the GPU.  Parity of the layer glue is unpinned by the reference (it has no model step).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from . import mx_oracle as o


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return F.rms_norm(x.float(), (x.shape[-1],), weight.float(), eps).to(torch.bfloat16)


def linear(x: torch.Tensor, weight, out_dtype=torch.bfloat16) -> torch.Tensor:
    """``weight`` = (codes [N,K] uint8, logical scales [N,K/32] uint8)."""
    a_codes, a_scales = o.quantize_mxfp8(x)
    return o.gemm_w6a8(a_codes, a_scales, weight[0], weight[1], out_dtype=out_dtype)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool) -> torch.Tensor:
    """q [B, Hq, Tq, D], k/v [B, Hkv, Tk, D] BF16 -> BF16; query heads share KV heads in
    contiguous groups."""
    group = q.shape[1] // k.shape[1]
    kf = k.float().repeat_interleave(group, dim=1)
    vf = v.float().repeat_interleave(group, dim=1)
    return F.scaled_dot_product_attention(q.float(), kf, vf, is_causal=causal).to(torch.bfloat16)


def layer_step(x, residual, layer, cfg, shape, attend):
    """Returns (x after the attention residual, MLP output to add next).

    ``layer`` = dict(ln1, ln2, qkv, o, gate_up, down) with decoded-weight pairs; ``attend``
    maps (q, k, v) of shapes [T, H, D] to [T, Hq * D]."""
    if residual is not None:
        x = (x.float() + residual.float()).to(torch.bfloat16)
    hd = cfg.head_dim
    qkv = linear(rms_norm(x, layer["ln1"], cfg.eps), layer["qkv"])
    q_dim, kv_dim = shape.q_heads * hd, shape.kv_heads * hd
    t = x.shape[0]
    q = qkv[:, :q_dim].view(t, shape.q_heads, hd)
    k = qkv[:, q_dim : q_dim + kv_dim].view(t, shape.kv_heads, hd)
    v = qkv[:, q_dim + kv_dim :].view(t, shape.kv_heads, hd)
    attn = attend(q, k, v)
    x = (x.float() + linear(attn, layer["o"]).float()).to(torch.bfloat16)
    gate_up = linear(rms_norm(x, layer["ln2"], cfg.eps), layer["gate_up"], out_dtype=None)
    act = o.silu_and_mul_bf16(gate_up).to(torch.bfloat16)
    return x, linear(act, layer["down"])


def prefill(x, layers, cfg, shape):
    def attend(q, k, v):
        out = attention(q.transpose(0, 1).unsqueeze(0), k.transpose(0, 1).unsqueeze(0),
                        v.transpose(0, 1).unsqueeze(0), True)
        return out.squeeze(0).transpose(0, 1).reshape(q.shape[0], -1)

    residual = None
    for layer in layers:
        x, residual = layer_step(x, residual, layer, cfg, shape, attend)
    return (x.float() + residual.float()).to(torch.bfloat16)


def decode_step(x, layers, caches, position, cfg, shape):
    """``caches[i]`` = (k, v) [B, Hkv, >= position + 1, D] BF16, rows < position filled."""
    residual = None
    for layer, (k_cache, v_cache) in zip(layers, caches):
        def attend(q, k, v, k_cache=k_cache, v_cache=v_cache):
            k_cache = k_cache.clone()
            v_cache = v_cache.clone()
            k_cache[:, :, position] = k
            v_cache[:, :, position] = v
            out = attention(q.unsqueeze(2), k_cache[:, :, : position + 1],
                            v_cache[:, :, : position + 1], False)
            return out.squeeze(2).reshape(q.shape[0], -1)

        x, residual = layer_step(x, residual, layer, cfg, shape, attend)
    return (x.float() + residual.float()).to(torch.bfloat16)
