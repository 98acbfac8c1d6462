"""``torch.ops.mxfp6.*``: the dispatcher names external callers of the reference use.

CPU part: every operator the reference registers (tests/golden/torch_op_schemas.json, made
from its ``m.def`` strings by tests/golden/make_torch_op_schemas.py) exists here with the
identical schema.  GPU part: calls through the dispatcher, written the way the reference's
vLLM integration writes them (examples/vllm/patches/vllm-v0.25.1-mxfp6.patch:277-300), give
the bytes of the package-level calls, which the other GPU tests check against the oracle.
"""

from __future__ import annotations

import json

import pytest
import torch

import mxfp6_sm120_b200 as mx

DEV = "cuda:0"


def test_every_reference_operator_is_registered_with_its_schema(golden_dir):
    assert mx.torch_ops.REGISTERED
    golden = json.loads((golden_dir / "torch_op_schemas.json").read_text())
    assert sorted(golden) == sorted(mx.torch_ops.operator_names())
    for name, schema in golden.items():
        got = str(getattr(torch.ops.mxfp6, name).default._schema)
        assert got == "mxfp6::" + schema, name


def test_registration_is_idempotent():
    assert mx.torch_ops.register() is True


@pytest.mark.gpu
def test_gemm_w6a8_through_the_dispatcher_as_the_vllm_patch_calls_it():
    gen = torch.Generator(device="cpu").manual_seed(31)
    rows, n, k = 24, 2048, 5120
    x = torch.randn((rows, k), generator=gen).to(torch.bfloat16).to(DEV)
    w = (torch.randn((n, k), generator=gen) * 0.02).to(torch.bfloat16).to(DEV)
    weight_values, weight_scale = torch.ops.mxfp6.quantize_mxfp6(w)
    quantized_x, input_scale = torch.ops.mxfp6.quantize_mxfp8(x)
    assert quantized_x.dtype == torch.float8_e4m3fn and tuple(quantized_x.shape) == (rows, k)
    for dtype in (torch.bfloat16, torch.float16):
        output = torch.ops.mxfp6.gemm_w6a8(quantized_x.view(torch.uint8), weight_values, input_scale,
                                           weight_scale, rows, n, k, 1.0, dtype)
        want = mx.gemm_w6a8(mx.quantize_mxfp8(x), mx.quantize_mxfp6(w), out_dtype=dtype)
        assert output.dtype == dtype and torch.equal(output, want)
    fused = torch.ops.mxfp6.gemm_from_float(x, weight_values, weight_scale, n, 1.0, torch.bfloat16)
    assert torch.equal(fused, mx.gemm_from_float(x, mx.quantize_mxfp6(w), out_dtype=torch.bfloat16))
    assert torch.ops.mxfp6.w6a8_config_abi(x) == mx.w6a8_config_abi()
    explicit = torch.ops.mxfp6.gemm_w6a8_config(quantized_x.view(torch.uint8), weight_values, input_scale,
                                                weight_scale, rows, n, k, 1.0, 10, 1, 0, torch.bfloat16)
    rel = float((explicit.float() - fused.float()).norm() / fused.float().norm())
    assert rel <= 1e-3
    try:
        assert torch.ops.mxfp6.set_w6a8_config(x, rows, n, k, 10, 1, 0, torch.bfloat16)
        assert mx.gemm_w6a8_plan(rows, n, k)["tile_tokens"] == mx.w6a8_configs()[10]["tile_tokens"]
    finally:
        torch.ops.mxfp6.set_w6a8_config(x, rows, n, k, -1, 1, 0, torch.bfloat16)
    stats = torch.ops.mxfp6.workspace_stats(x)
    assert stats == mx.workspace_stats(DEV)
    assert mx.device_status() == 0


@pytest.mark.gpu
def test_format_and_moe_operators_through_the_dispatcher():
    gen = torch.Generator(device="cpu").manual_seed(32)
    codes = torch.randint(0, 64, (256, 512), generator=gen, dtype=torch.uint8).to(DEV)
    packed = torch.ops.mxfp6.pack_fp6(codes)
    assert torch.equal(torch.ops.mxfp6.unpack_fp6(packed, 256, 512), codes)
    assert torch.equal(torch.ops.mxfp6.pad_fp6(packed), mx.pad_fp6(packed))
    logical = torch.randint(100, 140, (256, 16), generator=gen, dtype=torch.uint8).to(DEV)
    atoms = torch.ops.mxfp6.pack_scales(logical, 256, 512)
    assert torch.equal(torch.ops.mxfp6.unpack_scales(atoms, 256, 512), logical)

    tokens, topk, experts, n, k = 3, 2, 5, 256, 512
    source = torch.randn((tokens, k), generator=gen).to(torch.bfloat16).to(DEV)
    weight = mx.quantize_mxfp6(torch.randn((experts * n, k), generator=gen).to(torch.bfloat16).to(DEV))
    stack = weight.values.view(experts, n, k * 3 // 4)
    ids = torch.tensor([[0, 3], [2, 1], [3, 0]], dtype=torch.int32, device=DEV)
    activation, scales = torch.ops.mxfp6.quantize_mxfp8_logical(source)
    got = torch.empty((tokens * (topk + 1), n), dtype=torch.bfloat16, device=DEV)
    assert torch.ops.mxfp6.array_gemm_w6a8_out(got, activation, scales, stack, weight.scales, ids, True) is None
    want = torch.empty_like(got)
    mx.array_gemm_w6a8_out(want, activation, scales, stack, weight.scales, ids, True)
    assert torch.equal(got, want)
    weights = torch.rand((tokens, topk), generator=gen).to(DEV)
    gate = torch.randn((tokens,), generator=gen).to(torch.bfloat16).to(DEV)
    reduced = torch.empty((tokens, n), dtype=torch.bfloat16, device=DEV)
    torch.ops.mxfp6.moe_reduce_array_out(reduced, got, weights, gate)
    want_reduced = torch.empty_like(reduced)
    mx.moe_reduce_array_out(want_reduced, want, weights, gate)
    assert torch.equal(reduced, want_reduced)
    assert mx.device_status() == 0


def test_every_implementation_binds_the_arguments_of_its_schema():
    """The dispatcher calls an implementation with ALL schema arguments, positionally (defaults
    filled in).  Most operators are exercised on the GPU through the package functions, not
    through the dispatcher, so the binding of each one is checked here without a GPU."""
    import inspect

    from mxfp6_sm120_b200 import torch_ops

    for name, implementation in torch_ops._IMPLEMENTATIONS.items():
        schema = getattr(torch.ops.mxfp6, name).default._schema
        count = len(schema.arguments)
        signature = inspect.signature(implementation)
        try:
            signature.bind(*([None] * count))
        except TypeError as error:  # too many or too few positional parameters
            raise AssertionError(f"{name}: implementation does not take {count} arguments: {error}")
        # and it must not need more than the schema provides
        required = [p for p in signature.parameters.values()
                    if p.default is inspect.Parameter.empty
                    and p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD)]
        assert len(required) <= count, name
