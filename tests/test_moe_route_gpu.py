"""Decode-batch MoE: one single-row GEMM per route, checked against the CPU oracle.

Mirrors the reference's tests of its array and split-K operators
(tests/test_ops.py:232-393 ``test_array_w6a8``, :395-480 ``test_fused_array_silu_mxfp8``,
:483-596 ``test_fused_array_w2_reduce``, :599-760 ``test_qwen35_b1_specialization``):
route GEMMs against the decoded FP32 matmul (rel-Frobenius <= 1e-3, the reference uses
rtol 2e-3), the fused SwiGLU epilogue bit for bit against the unfused chain, the fused
W2 + reduce bit for bit against route GEMM -> ``moe_reduce_array_out``, and the whole decode
schedule against the oracle's layer (identical expert ids, cosine >= 0.999).
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import mx_oracle as o

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
GEMM_REL_FRO = 1.0e-3


def _rel_fro(got, want) -> float:
    got, want = got.float().cpu(), want.float().cpu()
    return float((got - want).norm() / want.norm().clamp_min(1e-30))


@pytest.fixture(scope="module", autouse=True)
def _status_clean(mx):
    yield
    torch.cuda.synchronize()
    assert mx.device_status() == 0


def _stack(mx, experts, n, k, seed, scale=1.0):
    gen = torch.Generator(device=DEV).manual_seed(seed)
    w = (torch.randn((experts * n, k), generator=gen, device=DEV) * scale).to(torch.bfloat16)
    packed = mx.quantize_mxfp6(w)
    codes = mx.unpack_fp6(packed.values, experts * n, k).cpu().numpy().reshape(experts, n, k)
    scales = mx.unpack_scales(packed.scales, experts * n, k).cpu().numpy().reshape(experts, n, k // 32)
    return packed, packed.values.view(experts, n, k * 3 // 4), codes, scales


def _route_expert(ids, token, lane, topk, experts):
    return experts - 1 if lane == topk else int(ids[token, lane])


@pytest.mark.parametrize("tokens,topk,experts,n,k", [(4, 2, 5, 128, 128), (3, 8, 12, 384, 2048),
                                                      (8, 4, 9, 256, 640), (1, 1, 2, 128, 256)])
@pytest.mark.parametrize("ids_dtype", [torch.int32, torch.int64])
def test_route_gemm_matches_oracle_in_route_order(mx, tokens, topk, experts, n, k, ids_dtype):
    packed, values, codes, scales = _stack(mx, experts, n, k, seed=12036 + n)
    gen = torch.Generator(device="cpu").manual_seed(77 + tokens)
    source = torch.randn((tokens, k), generator=gen).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(experts, generator=gen)[:topk] for _ in range(tokens)]).to(ids_dtype)
    act, act_scales = mx.quantize_mxfp8_logical(source.to(DEV))
    a_codes, a_scales = o.quantize_mxfp8_torch(source)
    assert np.array_equal(act.view(torch.uint8).cpu().numpy(), a_codes)
    assert np.array_equal(act_scales.cpu().numpy(), a_scales)

    for include_shared in (False, True):
        lanes = topk + int(include_shared)
        for out_dtype in (torch.bfloat16, torch.float16):
            got = torch.full((tokens * lanes, n), float("nan"), dtype=out_dtype, device=DEV)
            mx.array_gemm_w6a8_out(got, act, act_scales, values, packed.scales, ids.to(DEV), include_shared)
            want = torch.stack([
                o.gemm_w6a8(a_codes[r // lanes][None], a_scales[r // lanes][None],
                            codes[_route_expert(ids, r // lanes, r % lanes, topk, experts)],
                            scales[_route_expert(ids, r // lanes, r % lanes, topk, experts)],
                            out_dtype=out_dtype)[0]
                for r in range(tokens * lanes)])
            assert _rel_fro(got, want) <= GEMM_REL_FRO, (include_shared, out_dtype)
            again = torch.empty_like(got)
            mx.array_gemm_w6a8_out(again, act, act_scales, values, packed.scales, ids.to(DEV), include_shared)
            assert torch.equal(got, again)

    # one activation row per route instead of one per token (the form W2 takes)
    lanes = topk + 1
    rows = torch.randn((tokens * lanes, k), generator=gen).to(torch.bfloat16)
    act_r, scales_r = mx.quantize_mxfp8_logical(rows.to(DEV))
    r_codes, r_scales = o.quantize_mxfp8_torch(rows)
    got = torch.empty((tokens * lanes, n), dtype=torch.bfloat16, device=DEV)
    mx.array_gemm_w6a8_out(got, act_r, scales_r, values, packed.scales, ids.to(DEV), True)
    want = torch.stack([
        o.gemm_w6a8(r_codes[r][None], r_scales[r][None],
                    codes[_route_expert(ids, r // lanes, r % lanes, topk, experts)],
                    scales[_route_expert(ids, r // lanes, r % lanes, topk, experts)])[0]
        for r in range(tokens * lanes)])
    assert _rel_fro(got, want) <= GEMM_REL_FRO


def test_route_operators_reject_bad_operands(mx):
    packed, values, _, _ = _stack(mx, 3, 128, 128, seed=5)
    act, act_scales = mx.quantize_mxfp8_logical(torch.randn((2, 128), device=DEV).to(torch.bfloat16))
    ids = torch.tensor([[0], [1]], dtype=torch.int32, device=DEV)
    out = torch.empty((2, 128), dtype=torch.bfloat16, device=DEV)
    mx.array_gemm_w6a8_out(out, act, act_scales, values, packed.scales, ids)
    with pytest.raises(ValueError):
        mx.array_gemm_w6a8_out(out[:1], act, act_scales, values, packed.scales, ids)
    with pytest.raises(ValueError):
        mx.array_gemm_w6a8_out(out, act, act_scales[:, :2], values, packed.scales, ids)
    with pytest.raises(ValueError):
        mx.array_gemm_w6a8_out(out, act, act_scales, values, packed.scales, ids.float())
    with pytest.raises(ValueError):
        mx.array_gemm_w6a8_out(out.float(), act, act_scales, values, packed.scales, ids)
    with pytest.raises(ValueError):
        mx.array_gemm_w6a8_out(out, act, act_scales, values.view(3 * 128, 96), packed.scales, ids)
    # an id outside the stack leaves that route's row as it was (the reference skips it too)
    bad = torch.tensor([[7], [1]], dtype=torch.int32, device=DEV)
    marked = torch.full((2, 128), 3.0, dtype=torch.bfloat16, device=DEV)
    mx.array_gemm_w6a8_out(marked, act, act_scales, values, packed.scales, bad)
    assert torch.equal(marked[0], torch.full((128,), 3.0, dtype=torch.bfloat16, device=DEV))
    assert torch.equal(marked[1], out[1])


@pytest.mark.parametrize("tokens,topk,experts,inter,k", [(1, 2, 5, 256, 2048), (5, 3, 7, 128, 256),
                                                          (8, 8, 20, 512, 2048)])
def test_fused_w1_swiglu_equals_the_unfused_chain(mx, tokens, topk, experts, inter, k):
    packed, values, codes, scales = _stack(mx, experts, 2 * inter, k, seed=12037 + inter, scale=0.05)
    gen = torch.Generator(device="cpu").manual_seed(91 + tokens)
    source = torch.randn((tokens, k), generator=gen).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(experts - 1, generator=gen)[:topk] for _ in range(tokens)]).to(torch.int32)
    act, act_scales = mx.quantize_mxfp8_logical(source.to(DEV))
    routes = tokens * (topk + 1)

    gate_up = torch.empty((routes, 2 * inter), dtype=torch.bfloat16, device=DEV)
    mx.array_gemm_w6a8_out(gate_up, act, act_scales, values, packed.scales, ids.to(DEV), True)
    want, want_scales = mx.silu_and_mul_mxfp8_logical(gate_up)
    got = torch.zeros((routes, inter), dtype=torch.uint8, device=DEV)
    got_scales = torch.zeros((routes, inter // 32), dtype=torch.uint8, device=DEV)
    mx.array_gemm_w6a8_silu_mxfp8_out(got, got_scales, act, act_scales, values, packed.scales,
                                      ids.to(DEV), True)
    assert torch.equal(got_scales, want_scales)
    assert torch.equal(got, want.view(torch.uint8))

    # the shared expert as a separate matrix: the same bytes as with the shared expert last
    sep = torch.zeros_like(got)
    sep_scales = torch.zeros_like(got_scales)
    last = mx.PackedMXFP6Tensor(
        values[experts - 1:].contiguous().view(-1),
        packed.scales.view(experts, -1)[experts - 1:].contiguous().view(-1), 2 * inter, k)
    mx.qwen35_w1_splitk_silu_mxfp8_out(
        sep, sep_scales, None, act, act_scales, values[: experts - 1].contiguous(),
        packed.scales.view(experts, -1)[: experts - 1].contiguous().view(-1), ids.to(DEV), True,
        last.values.view(1, 2 * inter, -1), last.scales)
    assert torch.equal(sep, got) and torch.equal(sep_scales, got_scales)

    # and the oracle's chain on the oracle's own accumulators agrees up to rounding ties
    a_codes, a_scales = o.quantize_mxfp8_torch(source)
    lanes = topk + 1
    acc = torch.stack([
        o.gemm_w6a8(a_codes[r // lanes][None], a_scales[r // lanes][None],
                    codes[_route_expert(ids, r // lanes, r % lanes, topk, experts)],
                    scales[_route_expert(ids, r // lanes, r % lanes, topk, experts)], out_dtype=None)[0]
        for r in range(routes)])
    o_codes, o_scales = o.silu_and_mul_mxfp8(acc)
    mine = o.dequant_mxfp8(got.cpu().numpy(), got_scales.cpu().numpy())
    theirs = o.dequant_mxfp8(o_codes, o_scales)
    assert _rel_fro(mine, theirs) <= 2e-2
    assert float((torch.as_tensor(got.cpu().numpy() != o_codes)).float().mean()) <= 0.02


@pytest.mark.parametrize("tokens,topk,experts,n,k,out_dtype", [
    (1, 8, 10, 128, 256, torch.bfloat16), (2, 8, 12, 2048, 512, torch.bfloat16),
    (8, 8, 20, 2048, 512, torch.bfloat16), (3, 4, 6, 256, 1024, torch.float16),
    (4, 1, 3, 384, 128, torch.bfloat16)])
def test_fused_w2_reduce_equals_route_gemm_then_reduce(mx, tokens, topk, experts, n, k, out_dtype):
    packed, values, codes, scales = _stack(mx, experts, n, k, seed=12038 + n)
    gen = torch.Generator(device="cpu").manual_seed(17 + tokens)
    lanes = topk + 1
    routes = tokens * lanes
    source = torch.randn((routes, k), generator=gen).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(experts - 1, generator=gen)[:topk] for _ in range(tokens)]).to(torch.int32)
    weights = torch.rand((tokens, topk), generator=gen)
    gate = torch.randn((tokens, 5), generator=gen).to(torch.bfloat16)   # the LAST column is the gate
    act, act_scales = mx.quantize_mxfp8_logical(source.to(DEV))
    ids_d, weights_d, gate_d = ids.to(DEV), weights.to(DEV), gate.to(DEV)

    combined = torch.empty((routes, n), dtype=out_dtype, device=DEV)
    mx.array_gemm_w6a8_out(combined, act, act_scales, values, packed.scales, ids_d, True)
    want = torch.empty((tokens, n), dtype=out_dtype, device=DEV)
    mx.moe_reduce_array_out(want, combined, weights_d, gate_d)

    # the unfused reduce against the oracle's: gated shared row first, then the routes in order
    inverse = torch.tensor([[t * lanes + l for l in range(topk)] for t in range(tokens)], dtype=torch.int32)
    shared_rows = combined.cpu()[topk::lanes]
    oracle = o.moe_reduce(combined.cpu(), weights, inverse, shared_rows, gate, out_dtype=out_dtype)
    assert _rel_fro(want, oracle) <= 1e-3

    got = torch.full_like(want, float("nan"))
    mx.array_gemm_w6a8_reduce_out(got, act, act_scales, values, packed.scales, ids_d, weights_d, gate_d)
    assert torch.equal(got, want)

    # the shared expert's rows computed elsewhere
    rows = torch.arange(routes).view(tokens, lanes)[:, :topk].reshape(-1).to(DEV)
    external = torch.full_like(want, float("nan"))
    mx.array_gemm_w6a8_reduce_out(
        external, act[rows].contiguous(), act_scales[rows].contiguous(),
        values[: experts - 1].contiguous(), packed.scales.view(experts, -1)[: experts - 1].contiguous().view(-1),
        ids_d, weights_d, gate_d, combined[topk::lanes].contiguous())
    assert torch.equal(external, want)

    # the shared expert as a separate matrix, through the split-K name
    separate = torch.full_like(want, float("nan"))
    mx.qwen35_w2_splitk_reduce_out(
        separate, None, act, act_scales, values[: experts - 1].contiguous(),
        packed.scales.view(experts, -1)[: experts - 1].contiguous().view(-1), ids_d, weights_d,
        gate_d[:, -1].contiguous(), values[experts - 1:].contiguous(),
        packed.scales.view(experts, -1)[experts - 1:].contiguous().view(-1))
    assert torch.equal(separate, want)


def test_router_logits_topk_and_quantization(mx):
    batch, hidden, experts = 5, 2048, 256
    gen = torch.Generator(device="cpu").manual_seed(12039)
    x = torch.randn((batch, hidden), generator=gen).to(torch.bfloat16)
    gate_w = (torch.randn((experts + 1, hidden), generator=gen) * 0.05).to(torch.bfloat16)
    q = torch.empty((batch, hidden), dtype=torch.float8_e4m3fn, device=DEV)
    qs = torch.empty((batch, hidden // 32), dtype=torch.uint8, device=DEV)
    logits = torch.empty((batch, experts), dtype=torch.bfloat16, device=DEV)
    tw = torch.empty((batch, 8), dtype=torch.float32, device=DEV)
    ti = torch.empty((batch, 8), dtype=torch.int32, device=DEV)
    sg = torch.empty((batch,), dtype=torch.bfloat16, device=DEV)
    for renormalize in (False, True):
        mx.qwen35_router_quant_out(q, qs, logits, tw, ti, sg, x.to(DEV), gate_w.to(DEV), renormalize=renormalize)
        full = x.float() @ gate_w.float().t()
        torch.testing.assert_close(logits.float().cpu(), full[:, :experts], rtol=2 ** -7, atol=2e-2)
        torch.testing.assert_close(sg.float().cpu(), full[:, experts], rtol=2 ** -7, atol=2e-2)
        want_w, want_i = o.softmax_topk(logits.cpu(), 8, renormalize)     # on the GPU's own BF16 logits
        assert torch.equal(ti.cpu(), want_i)
        torch.testing.assert_close(tw.cpu(), want_w, rtol=1e-5, atol=1e-7)
        codes, scales = o.quantize_mxfp8_torch(x)
        assert np.array_equal(q.view(torch.uint8).cpu().numpy(), codes)
        assert np.array_equal(qs.cpu().numpy(), scales)
    # the shared expert's gate row as a tensor of its own
    sg2 = torch.empty_like(sg)
    logits2 = torch.empty_like(logits)
    mx.qwen35_router_quant_out(q, qs, logits2, tw, ti, sg2, x.to(DEV), gate_w[:experts].contiguous().to(DEV),
                               renormalize=True, shared_gate_weight=gate_w[experts:].contiguous().to(DEV))
    assert torch.equal(logits2, logits) and torch.equal(sg2, sg)


def _layer_weights(mx, shape, seed=4000):
    gen = torch.Generator(device=DEV).manual_seed(seed)
    h, i, e = shape.hidden, shape.intermediate, shape.experts
    make = lambda rows, cols: mx.quantize_mxfp6(
        (torch.randn((rows, cols), generator=gen, device=DEV) * 0.02).to(torch.bfloat16))
    return make(e * 2 * i, h), make(e * h, i), make(2 * i, h), make(h, i)


def _oracle_decode_layer(mx, shape, w1, w2, sw1, sw2, hidden, logits, gate, ids):
    e, i, h = shape.experts, shape.intermediate, shape.hidden
    w1v, w2v = w1.values.view(e, -1), w2.values.view(e, -1)
    w1s = mx.unpack_scales(w1.scales, e * 2 * i, h).view(e, 2 * i, h // 32)
    w2s = mx.unpack_scales(w2.scales, e * h, i).view(e, h, i // 32)
    w1c, w1l, w2c, w2l = {}, {}, {}, {}
    for x in sorted(set(ids.flatten().tolist())):
        w1c[x] = mx.unpack_fp6(w1v[x], 2 * i, h).cpu().numpy()
        w2c[x] = mx.unpack_fp6(w2v[x], h, i).cpu().numpy()
        w1l[x], w2l[x] = w1s[x].cpu().numpy(), w2s[x].cpu().numpy()
    sc, sd = mx.unpack_operand(sw1), mx.unpack_operand(sw2)
    shared = (sc[0].cpu().numpy(), sc[1].cpu().numpy(), sd[0].cpu().numpy(), sd[1].cpu().numpy())
    return o.moe_layer(hidden, logits, w1c, w1l, w2c, w2l, shared, gate, shape.topk, True)


@pytest.fixture(scope="module")
def named_layer(mx):
    shape = mx.MoeShape()
    weights = _layer_weights(mx, shape)
    yield shape, weights
    del weights
    torch.cuda.empty_cache()


@pytest.mark.parametrize("tokens", [1, 2, 3, 4, 8, 16, 24, 32])
def test_decode_schedule_named_config_against_oracle_and_graph(mx, named_layer, tokens):
    """Hidden 2048, 256 experts + shared, top-8, intermediate 512: three launches per layer."""
    shape, (w1, w2, sw1, sw2) = named_layer
    e, i, h = shape.experts, shape.intermediate, shape.hidden
    gen = torch.Generator(device="cpu").manual_seed(4100 + tokens)
    hidden = torch.randn((tokens, h), generator=gen).to(torch.bfloat16)
    logits = torch.randn((tokens, e), generator=gen).to(torch.bfloat16)
    gate = torch.randn((tokens,), generator=gen).to(torch.bfloat16)
    ws = mx.Qwen35MoeB1Workspace.allocate(DEV, shape, batch=tokens)
    w1v, w2v = w1.values.view(e, 2 * i, h * 3 // 4), w2.values.view(e, h, i * 3 // 4)
    hidden_d, logits_d, gate_d = hidden.to(DEV), logits.to(DEV), gate.to(DEV)

    def step():
        return mx.qwen35_moe_decode_logits_out(ws, hidden_d, logits_d, gate_d, w1v, w1.scales, w2v, w2.scales,
                                               sw1, sw2, renormalize=True)

    out = step().clone()
    want, want_ids = _oracle_decode_layer(mx, shape, w1, w2, sw1, sw2, hidden, logits, gate, ws.topk_ids.cpu())
    assert torch.equal(ws.topk_ids.cpu(), want_ids)
    # two launches (top-k and quantization inside the W1 kernel) and three launches give the
    # same bytes, ids and weights; the default picks one of them by the size of the grids
    assert mx.moe_decode_layer_supported(tokens, shape.topk, e, h, i)
    assert mx.moe_decode_layer_preferred(tokens, shape.topk, e, h, i)
    ws3 = mx.Qwen35MoeB1Workspace.allocate(DEV, shape, batch=tokens)
    three = mx.qwen35_moe_decode_logits_out(ws3, hidden_d, logits_d, gate_d, w1v, w1.scales, w2v, w2.scales,
                                            sw1, sw2, renormalize=True, two_launches=False)
    assert torch.equal(three, out)
    ws2 = mx.Qwen35MoeB1Workspace.allocate(DEV, shape, batch=tokens)
    two = mx.qwen35_moe_decode_logits_out(ws2, hidden_d, logits_d, gate_d, w1v, w1.scales, w2v, w2.scales,
                                          sw1, sw2, renormalize=True, two_launches=True)
    assert torch.equal(two, out)
    assert torch.equal(ws2.topk_ids, ws.topk_ids) and torch.equal(ws2.topk_weights, ws.topk_weights)
    # and with W2 selecting the experts again for itself instead of reading W1's ids
    own = torch.empty_like(out)
    mx.moe_decode_layer_out(own, ws2.activation, ws2.activation_scales, ws2.topk_weights, ws2.topk_ids,
                            hidden_d, logits_d, gate_d, w1v, w1.scales, w2v, w2.scales,
                            sw1.values.view(1, 2 * i, -1), sw1.scales, sw2.values.view(1, h, -1), sw2.scales,
                            renormalize=True, w2_own_routing=True)
    assert torch.equal(own, out)
    assert torch.equal(ws3.topk_ids, ws.topk_ids) and torch.equal(ws3.topk_weights, ws.topk_weights)
    assert torch.equal(ws3.activation.view(torch.uint8), ws.activation.view(torch.uint8))
    assert torch.equal(ws3.activation_scales, ws.activation_scales)
    per_token = torch.nn.functional.cosine_similarity(out.float().cpu(), want.float(), dim=1)
    assert float(per_token.min()) >= 0.999
    assert _rel_fro(out, want) <= 2e-2

    # the grouped schedule on the same inputs: same roundings, so nearly the same bytes
    from mxfp6_sm120_b200.moe_layer import MoeLayer

    layer = MoeLayer(shape, w1, w2, sw1, sw2)
    state = layer.workspace(tokens)
    assert state.decode is not None      # the layer object takes this schedule for these batches
    assert torch.equal(layer.forward(state, hidden_d, logits_d, gate_d), out)
    grouped = layer.forward_grouped(state, hidden_d, logits_d, gate_d)
    assert _rel_fro(out, grouped) <= 5e-3

    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        step()
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            step()
        for _ in range(20):
            graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(ws.output, out)


def test_b1_schedule_with_router_and_stacked_shared_expert(mx):
    """The reference's calling form: the gate matrix in, the shared expert last in both stacks
    (python/mxfp6/qwen35.py:384-432)."""
    shape = mx.MoeShape(hidden=1024, intermediate=256, experts=32, topk=8)
    e, i, h = shape.experts, shape.intermediate, shape.hidden
    w1, w1v, w1c, w1s = _stack(mx, e + 1, 2 * i, h, seed=31, scale=0.02)
    w2, w2v, w2c, w2s = _stack(mx, e + 1, h, i, seed=32, scale=0.02)
    gen = torch.Generator(device="cpu").manual_seed(33)
    gate_w = (torch.randn((e + 1, h), generator=gen) * 0.05).to(torch.bfloat16)
    for batch in (1, 4):
        hidden = torch.randn((batch, h), generator=gen).to(torch.bfloat16)
        ws = mx.Qwen35MoeB1Workspace.allocate(DEV, shape, batch=batch)
        out = mx.qwen35_moe_b1_out(ws, hidden.to(DEV), gate_w.to(DEV), w1v, w1.scales, w2v, w2.scales,
                                   renormalize=True)
        assert out.data_ptr() == ws.output.data_ptr()
        ids = ws.topk_ids.cpu()
        codes1 = {x: w1c[x] for x in set(ids.flatten().tolist())}
        scales1 = {x: w1s[x] for x in codes1}
        codes2 = {x: w2c[x] for x in codes1}
        scales2 = {x: w2s[x] for x in codes1}
        want, want_ids = o.moe_layer(hidden, ws.routed_logits.cpu(), codes1, scales1, codes2, scales2,
                                     (w1c[e], w1s[e], w2c[e], w2s[e]), ws.shared_gate.cpu(), 8, True)
        assert torch.equal(ids, want_ids)
        per_token = torch.nn.functional.cosine_similarity(out.float().cpu(), want.float(), dim=1)
        assert float(per_token.min()) >= 0.999
        # the two-launch form on the same logits, shared expert last in both stacks, no renormalisation
        two = torch.empty_like(out)
        act = torch.zeros_like(ws.activation)
        act_scales = torch.zeros_like(ws.activation_scales)
        tw, ti = torch.zeros_like(ws.topk_weights), torch.zeros_like(ws.topk_ids)
        for renormalize in (True, False):
            ref = mx.qwen35_moe_b1_out(ws, hidden.to(DEV), gate_w.to(DEV), w1v, w1.scales, w2v, w2.scales,
                                       renormalize=renormalize).clone()
            mx.moe_decode_layer_out(two, act, act_scales, tw, ti, hidden.to(DEV), ws.routed_logits,
                                    ws.shared_gate, w1v, w1.scales, w2v, w2.scales, renormalize=renormalize)
            assert torch.equal(two, ref) and torch.equal(ti, ws.topk_ids) and torch.equal(tw, ws.topk_weights)
