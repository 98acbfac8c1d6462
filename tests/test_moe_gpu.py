"""GPU parity tests of the routed-MoE path against the CPU oracle.

Expert ids must be identical, byte outputs bit-exact, grouped GEMMs within
rel-Frobenius 1e-3 and the whole layer within cosine >= 0.999 of the decoded CPU
path (the tolerances named by the hot-path contract).
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import mx_oracle as o

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _cpu_gen(seed):
    return torch.Generator(device="cpu").manual_seed(seed)


def _rel_fro(got, want) -> float:
    got, want = got.float().cpu(), want.float().cpu()
    return float((got - want).norm() / want.norm().clamp_min(1e-30))


@pytest.fixture(scope="module", autouse=True)
def _status_clean(mx):
    yield
    assert mx.device_status() == 0, "a bounded device wait expired during the tests"


@pytest.mark.parametrize("tokens,experts,topk", [(1, 256, 8), (7, 256, 8), (96, 256, 8), (33, 64, 4), (5, 40, 6)])
def test_topk_ids_and_weights(mx, tokens, experts, topk):
    gen = _cpu_gen(4100 + tokens)
    hidden = torch.randn((tokens, 2048), generator=gen).to(torch.bfloat16)
    logits = torch.randn((tokens, experts), generator=gen).to(torch.bfloat16)
    logits[0, 3] = logits[0, 17]  # a tie: the smaller id must win
    for renorm in (False, True):
        q = torch.empty((tokens, 2048), dtype=torch.uint8, device=DEV)
        ls = torch.empty((tokens, 64), dtype=torch.uint8, device=DEV)
        ps = torch.empty(mx.packed_scale_numel(tokens, 2048), dtype=torch.uint8, device=DEV)
        w = torch.empty((tokens, topk), dtype=torch.float32, device=DEV)
        ids = torch.empty((tokens, topk), dtype=torch.int32, device=DEV)
        mx.qwen35_topk_quant_out(q, ls, ps, w, ids, hidden.to(DEV), logits.to(DEV), renormalize=renorm)
        want_w, want_ids = o.softmax_topk(logits, topk, renorm)
        assert torch.equal(ids.cpu(), want_ids)
        torch.testing.assert_close(w.cpu(), want_w, rtol=1e-6, atol=1e-8)
        codes, scales = o.quantize_mxfp8_torch(hidden)
        assert np.array_equal(q.cpu().numpy(), codes)
        assert np.array_equal(ls.cpu().numpy(), scales)
        assert np.array_equal(mx.unpack_scales(ps, tokens, 2048).cpu().numpy(), scales)


def test_routing_invariants_and_expert_map(mx):
    tokens, experts, topk, hidden = 50, 32, 4, 256
    gen = _cpu_gen(3)
    act = torch.randint(0, 0x78, (tokens, hidden), generator=gen, dtype=torch.uint8)
    scales = torch.randint(120, 130, (tokens, hidden // 32), generator=gen, dtype=torch.uint8)
    ids = torch.stack([torch.randperm(experts, generator=gen)[:topk] for _ in range(tokens)]).to(torch.int32)
    permuted = torch.zeros((tokens * topk, hidden), dtype=torch.uint8, device=DEV)
    grouped, offsets, soff, inverse = mx.route_mxfp8_out(
        act.to(DEV), scales.to(DEV), ids.to(DEV), None, experts, permuted)
    counts = torch.bincount(ids.flatten().long(), minlength=experts)
    assert offsets.cpu().tolist() == [0, *torch.cumsum(counts, 0).tolist()]
    assert soff.cpu().tolist() == o.grouped_scale_offsets(offsets.cpu().numpy()).tolist()
    inv = inverse.cpu().long()
    assert sorted(inv.tolist()) == list(range(tokens * topk))  # a permutation
    flat = ids.flatten().long()
    rows = permuted.cpu()
    for route in range(tokens * topk):
        e, row = int(flat[route]), int(inv[route])
        assert int(offsets[e]) <= row < int(offsets[e + 1])
        assert torch.equal(rows[row], act[route // topk])
    # scales follow their rows into the grouped packed layout
    logical_permuted = torch.empty((tokens * topk, hidden // 32), dtype=torch.uint8)
    logical_permuted[inv] = scales.repeat_interleave(topk, dim=0)
    want, _ = o.pack_grouped_scales(logical_permuted.numpy(), offsets.cpu().numpy())
    got = grouped.cpu().numpy()[: want.size]
    written = want != 0x7F
    assert np.array_equal(got[written], want[written])
    # expert parallel: only experts 8..15 are local, everything else is dropped
    expert_map = torch.full((experts,), -1, dtype=torch.int32)
    expert_map[8:16] = torch.arange(8, dtype=torch.int32)
    _, loc_off, _, loc_inv = mx.route_mxfp8_out(
        act.to(DEV), scales.to(DEV), ids.to(DEV), expert_map.to(DEV), 8, permuted)
    local_counts = counts[8:16]
    assert loc_off.cpu().tolist() == [0, *torch.cumsum(local_counts, 0).tolist()]
    dropped = (flat < 8) | (flat >= 16)
    assert bool((loc_inv.cpu()[dropped] == -1).all())
    assert bool((loc_inv.cpu()[~dropped] >= 0).all())


@pytest.mark.parametrize("tokens,topk,hidden,routed_experts", [(5, 3, 128, 4), (70, 8, 512, 24)])
def test_shared_group_routing_and_reduce(mx, tokens, topk, hidden, routed_experts):
    """``include_shared``: one trailing always-hit group, token t at its row t, and the
    reduction that takes the shared rows from the tail of the routed output (the case of the
    reference's tests/test_ops.py:1309-1381, plus a batch that spans several scale atoms)."""
    gen = _cpu_gen(17)
    act = torch.randint(0, 0x78, (tokens, hidden), generator=gen, dtype=torch.uint8)
    scales = torch.randint(120, 130, (tokens, hidden // 32), generator=gen, dtype=torch.uint8)
    ids = torch.stack([torch.randperm(routed_experts, generator=gen)[:topk]
                       for _ in range(tokens)]).to(torch.int32)
    routes = tokens * topk
    experts = routed_experts + 1
    permuted = torch.zeros((routes + tokens, hidden), dtype=torch.uint8, device=DEV)
    grouped, offsets, soff, inverse = mx.route_mxfp8_out(
        act.to(DEV), scales.to(DEV), ids.to(DEV), None, experts, permuted, include_shared=True)
    counts = torch.bincount(ids.flatten().long(), minlength=routed_experts).tolist() + [tokens]
    want_offsets = [0, *np.cumsum(counts).tolist()]
    assert offsets.cpu().tolist() == want_offsets
    assert soff.cpu().tolist() == o.grouped_scale_offsets(np.asarray(want_offsets)).tolist()
    shared_start = int(offsets[routed_experts])
    assert shared_start == routes and int(offsets[-1]) == routes + tokens
    rows = permuted.cpu()
    assert torch.equal(rows[shared_start:], act)  # token order
    inv = inverse.cpu().long()
    assert tuple(inv.shape) == (routes,) and sorted(inv.tolist()) == list(range(routes))
    flat = ids.flatten().long()
    for route in range(routes):
        e, row = int(flat[route]), int(inv[route])
        assert want_offsets[e] <= row < want_offsets[e + 1]
        assert torch.equal(rows[row], act[route // topk])
    # the scales of all rows, shared ones included, in the grouped packed layout
    logical_permuted = torch.empty((routes + tokens, hidden // 32), dtype=torch.uint8)
    logical_permuted[inv] = scales.repeat_interleave(topk, dim=0)
    logical_permuted[shared_start:] = scales
    want, _ = o.pack_grouped_scales(logical_permuted.numpy(), np.asarray(want_offsets))
    got = grouped.cpu().numpy()[: want.size]
    written = want != 0x7F
    assert np.array_equal(got[written], want[written])

    # the preallocated form writes the same offsets and rows, and the row -> token list
    cursors = torch.empty(experts, dtype=torch.int32, device=DEV)
    offsets2 = torch.empty(experts + 1, dtype=torch.int64, device=DEV)
    soff2 = torch.empty(experts + 1, dtype=torch.int64, device=DEV)
    inverse2 = torch.empty(routes, dtype=torch.int32, device=DEV)
    permuted2 = torch.zeros_like(permuted)
    packed2 = torch.full_like(grouped, 0x7F)
    source_tokens = torch.full((routes + tokens,), -7, dtype=torch.int32, device=DEV)
    mx.qwen35_route_mxfp8_out(act.to(DEV), scales.to(DEV), ids.to(DEV), permuted2, packed2, cursors,
                              offsets2, soff2, inverse2, include_shared=True,
                              source_tokens=source_tokens)
    assert offsets2.cpu().tolist() == want_offsets and soff2.cpu().tolist() == soff.cpu().tolist()
    assert cursors.cpu().tolist() == counts
    src = source_tokens.cpu().long()
    assert src[shared_start:].tolist() == list(range(tokens))
    assert torch.equal(permuted2.cpu(), act[src])
    inv2 = inverse2.cpu().long()
    assert torch.equal(src[inv2], torch.arange(routes) // topk)

    # the final reduction with the shared rows taken from the tail of the routed output
    routed_output = torch.randn((routes + tokens, hidden), generator=gen).to(torch.bfloat16)
    weights = torch.rand((tokens, topk), generator=gen)
    weights /= weights.sum(dim=1, keepdim=True)
    gate = torch.randn((tokens, 1), generator=gen).to(torch.bfloat16)
    out = torch.empty((tokens, hidden), dtype=torch.bfloat16, device=DEV)
    routed_dev = routed_output.to(DEV)
    mx.moe_reduce_out(out, routed_dev, weights.to(DEV), inverse,
                      routed_dev[shared_start: shared_start + tokens], gate.to(DEV))
    want_out = o.moe_reduce(routed_output, weights, inverse.cpu(), routed_output[shared_start:], gate)
    assert _rel_fro(out, want_out) <= 1e-3  # FP32 fused multiply-adds against the oracle's separate ones
    assert float((out.float().cpu() - want_out.float()).abs().max()) <= 2.0**-7 * float(want_out.float().abs().max())
    # reading the shared rows in place equals reading a separate copy of them, bit for bit
    out_copy = torch.empty_like(out)
    mx.moe_reduce_out(out_copy, routed_dev, weights.to(DEV), inverse,
                      routed_dev[shared_start: shared_start + tokens].clone(), gate.to(DEV))
    assert torch.equal(out, out_copy)

    # without the flag the trailing expert is an ordinary one, and the flag needs two experts
    with pytest.raises(ValueError):
        mx.route_mxfp8_out(act.to(DEV), scales.to(DEV), ids.to(DEV), None, 1, permuted,
                           include_shared=True)
    with pytest.raises(ValueError):
        mx.route_mxfp8_out(act.to(DEV), scales.to(DEV), ids.to(DEV), None, experts,
                           permuted[:routes], include_shared=True)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_silu_and_mul_variants_bit_exact(mx, dtype):
    rows, inter = 37, 256
    x = (torch.randn((rows, 2 * inter), generator=_cpu_gen(8)) * 3).to(dtype)
    want_codes, want_scales = o.silu_and_mul_mxfp8(x)
    values, logical = mx.silu_and_mul_mxfp8_logical(x.to(DEV))
    assert np.array_equal(values.view(torch.uint8).cpu().numpy(), want_codes)
    assert np.array_equal(logical.cpu().numpy(), want_scales)
    out = torch.empty((rows, inter), dtype=torch.uint8, device=DEV)
    packed = torch.full((mx.packed_scale_numel(rows, inter),), 0x7F, dtype=torch.uint8, device=DEV)
    mx.silu_and_mul_mxfp8_packed_out(out, packed, x.to(DEV))
    assert np.array_equal(out.cpu().numpy(), want_codes)
    assert np.array_equal(packed.cpu().numpy(), o.pack_scales(want_scales))
    offsets = torch.tensor([0, 5, 5, 30, 37], dtype=torch.int64)
    v2, gs, soff = mx.silu_and_mul_mxfp8_grouped(x.to(DEV), offsets.to(DEV))
    want_grouped, want_soff = o.pack_grouped_scales(want_scales, offsets.numpy())
    assert soff.cpu().tolist() == want_soff.tolist()
    assert np.array_equal(gs.cpu().numpy()[: want_grouped.size], want_grouped)
    assert np.array_equal(v2.view(torch.uint8).cpu().numpy(), want_codes)


def _grouped_case(mx, counts, n, k, seed):
    gen = _cpu_gen(seed)
    experts = len(counts)
    m = sum(counts)
    offsets = torch.tensor((0, *np.cumsum(counts).tolist()), dtype=torch.int64)
    a = torch.randn((m, k), generator=gen).to(torch.bfloat16)
    w = (torch.randn((experts * n, k), generator=gen) * 0.02).to(torch.bfloat16)
    a_q, a_s = o.quantize_mxfp8_torch(a)
    weight = mx.quantize_mxfp6(w.to(DEV))
    w_codes, w_scales = mx.unpack_operand(weight)
    grouped, soff = mx.pack_grouped_scales(torch.from_numpy(a_s).to(DEV), offsets.to(DEV))
    return (offsets, torch.from_numpy(a_q).to(DEV), grouped, soff, weight,
            (a_q, a_s, w_codes.cpu().numpy(), w_scales.cpu().numpy()))


@pytest.mark.parametrize("counts,n,k", [((1, 0, 3, 129, 2), 128, 128), ((5, 70, 0, 200, 1, 64), 256, 512),
                                        ((300, 17), 128, 1024)])
def test_grouped_gemm_matches_oracle(mx, counts, n, k):
    offsets, a_dev, grouped, soff, weight, (a_q, a_s, w_q, w_s) = _grouped_case(mx, counts, n, k, 12035)
    experts = len(counts)
    w3 = weight.values.view(experts, n, k * 3 // 4)
    for tile in (0, 64, 128, 192, 256):
        out = torch.full((sum(counts), n), float("nan"), dtype=torch.bfloat16, device=DEV)
        mx.grouped_gemm_w6a8_out(out, a_dev, grouped, w3, weight.scales, offsets.to(DEV), soff, tile_n=tile)
        for e, rows in enumerate(counts):
            if rows == 0:
                continue
            lo = int(offsets[e])
            want = o.gemm_w6a8(a_q[lo : lo + rows], a_s[lo : lo + rows], w_q[e * n : (e + 1) * n],
                               w_s[e * n : (e + 1) * n], out_dtype=torch.bfloat16)
            assert _rel_fro(out[lo : lo + rows], want) <= 1e-3


@pytest.mark.parametrize("counts,inter,k", [((1, 0, 3, 129, 2), 128, 256), ((40, 9, 0, 77), 256, 512)])
def test_fused_w1_epilogue_equals_unfused_path(mx, counts, inter, k):
    """Grouped W1 + SiLU*mul + MXFP8 in one kernel must equal grouped GEMM (BF16)
    followed by the stand-alone SiLU kernel, byte for byte (the reference checks its
    fused kernels the same way, tests/test_ops.py:453-459)."""
    n = 2 * inter
    offsets, a_dev, grouped, soff, weight, _ = _grouped_case(mx, counts, n, k, 77)
    experts = len(counts)
    w3 = weight.values.view(experts, n, k * 3 // 4)
    rows = sum(counts)
    h1 = mx.grouped_gemm_w6a8(a_dev, grouped, w3, weight.scales, offsets.to(DEV), soff)
    want_v, want_s, _ = mx.silu_and_mul_mxfp8_grouped(h1, offsets.to(DEV), soff)
    for tile in (0, 64, 128):
        out = torch.zeros((rows, inter), dtype=torch.uint8, device=DEV)
        out_scales = torch.full_like(want_s, 0x7F)
        mx.qwen35_grouped_w1_silu_mxfp8_out(out, out_scales, a_dev, grouped, w3, weight.scales,
                                            offsets.to(DEV), soff, tile_tokens=tile)
        assert torch.equal(out, want_v.view(torch.uint8))
        assert torch.equal(out_scales, want_s)


def test_reduce_matches_oracle_and_gate_identity(mx):
    tokens, topk, hidden = 13, 8, 2048
    gen = _cpu_gen(31)
    routed = torch.randn((tokens * topk, hidden), generator=gen).to(torch.bfloat16)
    shared = torch.randn((tokens, hidden), generator=gen).to(torch.bfloat16)
    weights = torch.rand((tokens, topk), generator=gen)
    weights = weights / weights.sum(dim=1, keepdim=True)
    inverse = torch.randperm(tokens * topk, generator=gen).to(torch.int32)
    gate = torch.randn((tokens, 1), generator=gen).to(torch.bfloat16)
    out = torch.empty((tokens, hidden), dtype=torch.bfloat16, device=DEV)
    mx.moe_reduce_out(out, routed.to(DEV), weights.to(DEV), inverse.to(DEV), shared.to(DEV), gate.to(DEV))
    want = o.moe_reduce(routed, weights, inverse, shared, gate)
    assert _rel_fro(out, want) <= 1e-3
    assert float((out.float().cpu() - want.float()).abs().max()) <= 2.0**-7 * float(want.float().abs().max())
    # gate logit 20 passes the shared row, gate 0 halves it
    zeros = torch.zeros((tokens, topk), device=DEV)
    ones = torch.ones((tokens, hidden), dtype=torch.bfloat16, device=DEV)
    for logit, expect in ((20.0, 1.0), (0.0, 0.5)):
        g = torch.full((tokens,), logit, dtype=torch.float32, device=DEV)
        mx.moe_reduce_out(out, routed.to(DEV), zeros, inverse.to(DEV), ones, g)
        assert bool((out.float() == expect).all())
    # dropped routes (-1) are skipped
    inverse2 = inverse.clone()
    inverse2[::3] = -1
    mx.moe_reduce_out(out, routed.to(DEV), weights.to(DEV), inverse2.to(DEV))
    w2 = weights.clone().flatten()
    w2[::3] = 0
    want2 = o.moe_reduce(routed, w2.view(tokens, topk), inverse.clamp_min(0), None, None)
    assert _rel_fro(out, want2) <= 1e-3


def _layer_case(mx, tokens, shape, seed=4000):
    """Random layer: weights are quantized on the GPU (bit-exact with the oracle by
    the dense tests) and only the experts a batch hits are decoded on the CPU."""
    gen = torch.Generator(device=DEV).manual_seed(seed)
    h, i, e = shape.hidden, shape.intermediate, shape.experts
    w1 = mx.quantize_mxfp6((torch.randn((e * 2 * i, h), generator=gen, device=DEV) * 0.02).to(torch.bfloat16))
    w2 = mx.quantize_mxfp6((torch.randn((e * h, i), generator=gen, device=DEV) * 0.02).to(torch.bfloat16))
    sw1 = mx.quantize_mxfp6((torch.randn((2 * i, h), generator=gen, device=DEV) * 0.02).to(torch.bfloat16))
    sw2 = mx.quantize_mxfp6((torch.randn((h, i), generator=gen, device=DEV) * 0.02).to(torch.bfloat16))
    cgen = _cpu_gen(4100 + tokens)
    hidden = torch.randn((tokens, h), generator=cgen).to(torch.bfloat16)
    logits = torch.randn((tokens, e), generator=cgen).to(torch.bfloat16)
    gate = torch.randn((tokens,), generator=cgen).to(torch.bfloat16)
    return w1, w2, sw1, sw2, hidden, logits, gate


def _run_layer(mx, shape, w1, w2, sw1, sw2, hidden, logits, gate):
    tokens = hidden.shape[0]
    ws = mx.Qwen35GroupedWorkspace.allocate(tokens, DEV, shape)
    shared = mx.SharedExpertWorkspace.allocate(tokens, DEV, shape)
    out = torch.empty((tokens, shape.hidden), dtype=torch.bfloat16, device=DEV)
    e, i, h = shape.experts, shape.intermediate, shape.hidden
    w1v, w2v = w1.values.view(e, 2 * i, h * 3 // 4), w2.values.view(e, h, i * 3 // 4)

    hidden_d, logits_d, gate_d = hidden.to(DEV), logits.to(DEV), gate.to(DEV)

    def step():
        mx.qwen35_grouped_gemm_out(ws, hidden_d, logits_d, w1v, w1.scales, w2v, w2.scales)
        mx.shared_expert_out(shared, ws, sw1, sw2)
        mx.qwen35_grouped_reduce_out(ws, out, shared.output, gate_d)

    step()
    return out, ws, step


def _oracle_layer(mx, shape, w1, w2, sw1, sw2, hidden, logits, gate, ids):
    e, i, h = shape.experts, shape.intermediate, shape.hidden
    used = sorted(set(ids.flatten().tolist()))
    w1c = {}
    w1v = w1.values.view(e, -1)
    w2v = w2.values.view(e, -1)
    w1s_all = mx.unpack_scales(w1.scales, e * 2 * i, h).view(e, 2 * i, h // 32)
    w2s_all = mx.unpack_scales(w2.scales, e * h, i).view(e, h, i // 32)

    class Lazy(dict):
        def __missing__(self, key):
            raise KeyError(key)

    w1_codes, w1_scales, w2_codes, w2_scales = Lazy(), Lazy(), Lazy(), Lazy()
    for x in used:
        w1_codes[x] = mx.unpack_fp6(w1v[x], 2 * i, h).cpu().numpy()
        w2_codes[x] = mx.unpack_fp6(w2v[x], h, i).cpu().numpy()
        w1_scales[x] = w1s_all[x].cpu().numpy()
        w2_scales[x] = w2s_all[x].cpu().numpy()
    sc = mx.unpack_operand(sw1)
    sd = mx.unpack_operand(sw2)
    shared = (sc[0].cpu().numpy(), sc[1].cpu().numpy(), sd[0].cpu().numpy(), sd[1].cpu().numpy())
    return o.moe_layer(hidden, logits, w1_codes, w1_scales, w2_codes, w2_scales, shared, gate,
                       shape.topk, True)


@pytest.mark.parametrize("tokens", [1, 4, 24, 96, 700])
def test_moe_layer_small_shape(mx, tokens):
    shape = mx.MoeShape(hidden=512, intermediate=256, experts=32, topk=4)
    case = _layer_case(mx, tokens, shape)
    out, ws, _ = _run_layer(mx, shape, *case)
    want, want_ids = _oracle_layer(mx, shape, *case, ids=ws.topk_ids.cpu())
    assert torch.equal(ws.topk_ids.cpu(), want_ids)
    cos = torch.nn.functional.cosine_similarity(out.float().cpu().flatten(), want.float().flatten(), dim=0)
    assert float(cos) >= 0.999
    assert _rel_fro(out, want) <= 2e-2


@pytest.mark.parametrize("tokens", [5, 40])
def test_preallocated_routing_on_workspace_buffers(mx, tokens):
    """``qwen35_route_mxfp8_out`` on the buffers a workspace allocates: with the caller's ids
    (``qwen35_grouped_moe_out``) and with an expert map over a workspace sized for the local
    experts only, the way the expert-parallel layer calls it."""
    shape = mx.MoeShape(hidden=512, intermediate=256, experts=32, topk=4)
    case = _layer_case(mx, tokens, shape)
    w1, w2, sw1, sw2, hidden, logits, gate = case
    _, ws0, _ = _run_layer(mx, shape, *case)
    e, i, h, k = shape.experts, shape.intermediate, shape.hidden, shape.topk
    want = torch.empty((tokens, h), dtype=torch.bfloat16, device=DEV)
    mx.moe_reduce_out(want, ws0.routed_output, ws0.topk_weights, ws0.inverse_permutation)
    ws1 = mx.Qwen35GroupedWorkspace.allocate(tokens, DEV, shape)
    got = torch.empty_like(want)
    mx.qwen35_grouped_moe_out(ws1, got, hidden.to(DEV), w1.values.view(e, 2 * i, h * 3 // 4), w1.scales,
                              w2.values.view(e, h, i * 3 // 4), w2.scales, ws0.topk_weights,
                              ws0.topk_ids)
    assert torch.equal(got, want)  # a row's result does not depend on where it sits in its group

    local = 8
    expert_map = torch.full((e,), -1, dtype=torch.int32)
    expert_map[8:16] = torch.arange(local, dtype=torch.int32)
    ws2 = mx.Qwen35GroupedWorkspace.allocate(tokens, DEV, mx.MoeShape(h, i, local, k))
    mx.qwen35_route_mxfp8_out(ws0.quantized, ws0.input_scales, ws0.topk_ids, ws2.permuted,
                              ws2.grouped_input_scales, ws2.expert_cursors, ws2.expert_offsets,
                              ws2.scale_offsets, ws2.inverse_permutation,
                              source_tokens=ws2.source_tokens, expert_map=expert_map.to(DEV))
    flat = ws0.topk_ids.cpu().flatten().long()
    counts = torch.bincount(flat, minlength=e)[8:16]
    assert ws2.expert_offsets.cpu().tolist() == [0, *torch.cumsum(counts, 0).tolist()]
    inv = ws2.inverse_permutation.cpu()
    is_local = (flat >= 8) & (flat < 16)
    assert bool((inv[~is_local] == -1).all()) and bool((inv[is_local] >= 0).all())
    kept = inv[is_local].long()
    assert torch.equal(ws2.source_tokens.cpu()[kept].long(), torch.nonzero(is_local).flatten() // k)
    assert torch.equal(ws2.permuted.cpu()[kept], ws0.quantized.cpu()[torch.nonzero(is_local).flatten() // k])
    # a scale buffer that is too small is refused on the host, before any launch
    with pytest.raises(ValueError):
        mx.qwen35_route_mxfp8_out(ws0.quantized, ws0.input_scales, ws0.topk_ids, ws2.permuted,
                                  ws2.grouped_input_scales[:64], ws2.expert_cursors,
                                  ws2.expert_offsets, ws2.scale_offsets, ws2.inverse_permutation)


@pytest.mark.parametrize("tokens", [3, 40, 300])
def test_shared_expert_as_trailing_group_matches_the_layer(mx, tokens):
    """The reference's other way to run the shared expert: as group E of the grouped GEMMs
    (benchmarks/benchmark_qwen35_moe_layer.py:700-760) - ``include_shared`` routing, W1 and W2
    over E+1 weight matrices, and the reduction reading the shared rows from the tail of the
    routed output.  Same layer, so it must agree with the dense shared-expert path and the oracle."""
    shape = mx.MoeShape(hidden=512, intermediate=256, experts=32, topk=4)
    case = _layer_case(mx, tokens, shape)
    w1, w2, sw1, sw2, hidden, logits, gate = case
    out, ws, _ = _run_layer(mx, shape, *case)
    e, i, h, k = shape.experts, shape.intermediate, shape.hidden, shape.topk
    w1_all = torch.cat([w1.values.reshape(-1), sw1.values.reshape(-1)]).view(e + 1, 2 * i, h * 3 // 4)
    w1s_all = torch.cat([w1.scales.reshape(-1), sw1.scales.reshape(-1)]).view(e + 1, -1)
    w2_all = torch.cat([w2.values.reshape(-1), sw2.values.reshape(-1)]).view(e + 1, h, i * 3 // 4)
    w2s_all = torch.cat([w2.scales.reshape(-1), sw2.scales.reshape(-1)]).view(e + 1, -1)
    routes = tokens * k
    rows = routes + tokens
    permuted = torch.empty((rows, h), dtype=torch.uint8, device=DEV)
    grouped, offsets, soff, inverse = mx.route_mxfp8_out(
        ws.quantized, ws.input_scales, ws.topk_ids, None, e + 1, permuted, include_shared=True)
    assert int(offsets[e]) == routes and int(offsets[e + 1]) == rows
    activated = torch.empty((rows, i), dtype=torch.uint8, device=DEV)
    activated_scales = torch.full((int(soff[-1]) * ((i // 32 + 3) // 4 * 4),), 0x7F,
                                  dtype=torch.uint8, device=DEV)
    mx.qwen35_grouped_w1_silu_mxfp8_out(activated, activated_scales, permuted, grouped, w1_all,
                                        w1s_all, offsets, soff)
    routed_output = torch.empty((rows, h), dtype=torch.bfloat16, device=DEV)
    mx.grouped_gemm_w6a8_out(routed_output, activated, activated_scales, w2_all, w2s_all, offsets, soff)
    got = torch.empty_like(out)
    mx.moe_reduce_out(got, routed_output, ws.topk_weights, inverse, routed_output[routes:],
                      gate.to(DEV))
    assert _rel_fro(got, out) <= 5e-3  # the dense path may split K; the grouped one does not
    want, _ = _oracle_layer(mx, shape, *case, ids=ws.topk_ids.cpu())
    cos = torch.nn.functional.cosine_similarity(got.float().cpu().flatten(), want.float().flatten(), dim=0)
    assert float(cos) >= 0.999
    assert _rel_fro(got, want) <= 2e-2


@pytest.mark.parametrize("tokens", [1, 2, 4, 8, 16, 24, 32, 64, 96])
def test_moe_layer_named_config_and_graph_replay(mx, tokens):
    """Hidden 2048, 256 experts, top-8, intermediate 512, shared expert with sigmoid gate:
    every decode batch of the named configuration against the decoded CPU layer."""
    shape = mx.MoeShape()
    case = _layer_case(mx, tokens, shape)
    out, ws, step = _run_layer(mx, shape, *case)
    want, want_ids = _oracle_layer(mx, shape, *case, ids=ws.topk_ids.cpu())
    assert torch.equal(ws.topk_ids.cpu(), want_ids)
    cos = torch.nn.functional.cosine_similarity(out.float().cpu().flatten(), want.float().flatten(), dim=0)
    assert float(cos) >= 0.999
    per_token = torch.nn.functional.cosine_similarity(out.float().cpu(), want.float(), dim=1)
    assert float(per_token.min()) >= 0.999
    if tokens not in (1, 8, 32):
        return
    # the whole layer replays from one CUDA graph with identical results
    first = out.clone()
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
    assert torch.equal(out, first)


@pytest.mark.parametrize("tokens,full_size", [(700, False), (4096, True)])
def test_prefill_batches_run_w1_unfused_with_identical_bytes(mx, tokens, full_size):
    """From 16384 routed rows on, W1 is a grouped GEMM into the front of routed_output
    followed by the SiLU*mul/MXFP8 kernel; the fused kernel gives the same bytes."""
    from mxfp6_sm120_b200 import qwen35

    shape = mx.MoeShape() if full_size else mx.MoeShape(hidden=512, intermediate=256, experts=32, topk=4)
    case = _layer_case(mx, tokens, shape)
    threshold = qwen35.UNFUSED_W1_MIN_ROUTES
    outs = {}
    try:
        for name, value in (("unfused", 1), ("fused", 1 << 60)):
            qwen35.UNFUSED_W1_MIN_ROUTES = value
            out, ws, _ = _run_layer(mx, shape, *case)
            outs[name] = out.clone()
    finally:
        qwen35.UNFUSED_W1_MIN_ROUTES = threshold
    # Rows land in their expert's block in arrival order, so only the layer output (which
    # the reduce gathers back per token) is comparable between two runs.
    assert torch.equal(outs["unfused"], outs["fused"])
    if full_size:
        assert tokens * shape.topk >= threshold  # the default takes the unfused path here
    assert mx.device_status() == 0


def test_moe_layer_named_config_prefill_batch_against_oracle(mx):
    """4096 tokens of the named configuration: expert ids of the whole batch against the
    oracle's softmax top-k, and the layer output of 16 sampled tokens against the decoded
    CPU layer run on those tokens alone (a token's output depends on no other token)."""
    shape = mx.MoeShape()
    tokens = 4096
    case = _layer_case(mx, tokens, shape)
    w1, w2, sw1, sw2, hidden, logits, gate = case
    out, ws, _ = _run_layer(mx, shape, *case)
    _, want_ids_all = o.softmax_topk(logits, shape.topk, True)
    assert torch.equal(ws.topk_ids.cpu(), want_ids_all)
    sample = torch.tensor([0, 1, 2, 127, 128, 129, 1000, 2047, 2048, 3000, 3333, 4000, 4093, 4094,
                           4095, 777])
    want, want_ids = _oracle_layer(mx, shape, w1, w2, sw1, sw2, hidden[sample], logits[sample],
                                   gate[sample], ids=ws.topk_ids.cpu()[sample])
    assert torch.equal(ws.topk_ids.cpu()[sample], want_ids)
    got = out.float().cpu()[sample]
    per_token = torch.nn.functional.cosine_similarity(got, want.float(), dim=1)
    assert float(per_token.min()) >= 0.999
    assert _rel_fro(got, want) <= 2e-2
    assert mx.device_status() == 0
