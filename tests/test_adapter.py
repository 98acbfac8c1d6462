"""The serving-framework adapter: linear kernel and routed-experts runner.

Mirrors what the reference's vLLM glue does with the library
(examples/vllm/patches/vllm-v0.25.1-mxfp6.patch:326-470 for the linear scheme,
examples/vllm/adapter/mxfp6_tp2_vllm.py:403-565 for the experts runner): weights arrive as
checkpoint tensors, are prepared once, and every forward goes through the dispatcher.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

import mxfp6_sm120_b200 as mx
from mxfp6_sm120_b200 import adapter, checkpoint as ck
from oracle import mx_oracle as o

DEV = "cuda:0"


def test_linear_kernel_prepares_checkpoint_tensors_once():
    rng = np.random.default_rng(9)
    n, k = 256, 512
    codes = rng.integers(0, 64, (n, k), dtype=np.uint8)
    scales = rng.integers(110, 130, (n, k // 32), dtype=np.uint8)
    layer = torch.nn.Module()
    layer.weight = torch.nn.Parameter(torch.from_numpy(o.pack_fp6(codes).reshape(n, -1)), requires_grad=False)
    layer.weight_scale = torch.nn.Parameter(torch.from_numpy(scales), requires_grad=False)
    kernel = adapter.MxFp6LinearKernel(n, k)
    kernel.process_weights_after_loading(layer)
    assert np.array_equal(layer.weight_scale.numpy(), o.pack_scales(scales))
    assert np.array_equal(layer.weight.numpy().reshape(-1), o.pack_fp6(codes).reshape(-1))
    with pytest.raises(ValueError):
        adapter.MxFp6LinearKernel(n + 4, k)
    with pytest.raises(ValueError):
        adapter.MxFp6LinearKernel(n, k + 64)
    with pytest.raises(ValueError):
        kernel.process_weights_after_loading(layer)   # the scales are packed already
    assert adapter.is_problem_supported(1000, 1024) and not adapter.is_problem_supported(1000, 1000)


@pytest.mark.gpu
def test_linear_kernel_applies_weights_like_the_package_call():
    gen = torch.Generator(device="cpu").manual_seed(41)
    n, k = 1024, 2048
    w = (torch.randn((n, k), generator=gen) * 0.02).to(torch.bfloat16).to(DEV)
    packed = mx.quantize_mxfp6(w)
    layer = torch.nn.Module()
    layer.weight = torch.nn.Parameter(packed.values.view(n, -1), requires_grad=False)
    layer.weight_scale = torch.nn.Parameter(mx.unpack_scales(packed.scales, n, k), requires_grad=False)
    kernel = adapter.MxFp6LinearKernel(n, k)
    kernel.process_weights_after_loading(layer)
    x = torch.randn((3, 7, k), generator=gen).to(torch.bfloat16).to(DEV)
    bias = torch.randn((n,), generator=gen).to(torch.bfloat16).to(DEV)
    got = kernel.apply_weights(layer, x, bias)
    want = mx.gemm_from_float(x.reshape(-1, k), packed, out_dtype=torch.bfloat16) + bias
    assert got.shape == (3, 7, n) and torch.equal(got.reshape(-1, n), want)
    assert mx.device_status() == 0


@pytest.mark.gpu
def test_experts_runner_matches_the_layer_object_for_decode_and_prefill_batches():
    from mxfp6_sm120_b200.moe_layer import MoeLayer

    dev = torch.device(DEV)
    shape = mx.MoeShape(hidden=1024, intermediate=256, experts=16, topk=8)
    layer = MoeLayer.random(dev, shape, seed=91)
    e, i, h = shape.experts, shape.intermediate, shape.hidden
    gen = torch.Generator(device=dev).manual_seed(92)
    gate_w = (torch.randn((e + 1, h), generator=gen, device=dev) * 0.05).to(torch.bfloat16)
    stacked = lambda routed, shared: mx.PackedMXFP6Tensor(
        torch.cat([routed.values, shared.values]), torch.cat([routed.scales, shared.scales]),
        routed.rows + shared.rows, routed.k)
    weights = ck.MoeLayerCheckpoint(h, i, e, stacked(layer.w1, layer.shared_w1),
                                    stacked(layer.w2, layer.shared_w2), gate_w)
    runner = adapter.MxFp6MoERunner(weights, max_tokens=64)
    for tokens in (1, 5, 40, 150):     # decode schedule, grouped schedule, chunks of 64
        hidden = torch.randn((tokens, h), generator=gen, device=dev).to(torch.bfloat16)
        got = runner.forward(hidden).clone()
        parts = []
        for lo in range(0, tokens, 64):
            chunk = hidden[lo: lo + 64].contiguous()
            logits = torch.empty((chunk.shape[0], e), dtype=torch.bfloat16, device=dev)
            gate = torch.empty((chunk.shape[0],), dtype=torch.bfloat16, device=dev)
            q = torch.empty((chunk.shape[0], h), dtype=torch.float8_e4m3fn, device=dev)
            qs = torch.empty((chunk.shape[0], h // 32), dtype=torch.uint8, device=dev)
            tw = torch.empty((chunk.shape[0], 8), dtype=torch.float32, device=dev)
            ti = torch.empty((chunk.shape[0], 8), dtype=torch.int32, device=dev)
            mx.qwen35_router_quant_out(q, qs, logits, tw, ti, gate, chunk, gate_w, renormalize=True)
            parts.append(layer.forward(layer.workspace(chunk.shape[0]), chunk, logits, gate).clone())
        assert torch.equal(got, torch.cat(parts))
    assert len(runner._states) == 5    # 1, 5, 40, 64 and the 22-token tail
    assert mx.device_status() == 0
