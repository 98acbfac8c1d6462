"""Checkpoint reader: logical OCP-MX scales + packed 6-bit codes -> kernel operand layout.

CPU part: against the oracle's ``pack_fp6`` / ``pack_scales`` on random codes, through
``.pt`` and ``.safetensors`` files, whole and tensor-parallel sliced the way the reference's
loader slices (benchmarks/benchmark_qwen35_moe_layer.py:363-376).  GPU part: a layer
written to disk and read back computes the same bytes as the layer in memory.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

import mxfp6_sm120_b200 as mx
from mxfp6_sm120_b200 import checkpoint as ck
from oracle import mx_oracle as o

PREFIX = "model.language_model.layers.0.mlp"


def _random_layer(experts, hidden, inter, seed):
    rng = np.random.default_rng(seed)
    w1_codes = rng.integers(0, 64, (experts + 1, 2 * inter, hidden), dtype=np.uint8)
    w2_codes = rng.integers(0, 64, (experts + 1, hidden, inter), dtype=np.uint8)
    w1_scales = rng.integers(110, 130, (experts + 1, 2 * inter, hidden // 32), dtype=np.uint8)
    w2_scales = rng.integers(110, 130, (experts + 1, hidden, inter // 32), dtype=np.uint8)
    gate = torch.from_numpy(rng.standard_normal((experts + 1, hidden)).astype(np.float32)).to(torch.bfloat16)
    pack = lambda codes: torch.from_numpy(
        np.stack([o.pack_fp6(c).reshape(c.shape[0], -1) for c in codes]))
    tensors = ck.moe_layer_tensors(PREFIX, hidden, inter, pack(w1_codes), torch.from_numpy(w1_scales),
                                   pack(w2_codes), torch.from_numpy(w2_scales), gate)
    return tensors, (w1_codes, w1_scales, w2_codes, w2_scales, gate)


def test_pack_scales_host_matches_the_oracle_layout():
    rng = np.random.default_rng(3)
    for rows, groups in ((128, 4), (300, 10), (1, 1), (257, 64)):
        logical = rng.integers(0, 255, (rows, groups), dtype=np.uint8)
        got = ck.pack_scales_host(torch.from_numpy(logical)).numpy()
        assert np.array_equal(got, o.pack_scales(logical))


@pytest.mark.parametrize("suffix", [".pt", ".safetensors"])
def test_moe_layer_round_trip_and_tensor_parallel_slices(tmp_path, suffix):
    experts, hidden, inter = 3, 256, 256
    tensors, (w1c, w1s, w2c, w2s, gate) = _random_layer(experts, hidden, inter, seed=11)
    path = tmp_path / ("layer" + suffix)
    ck.save_tensors(tensors, path)
    layer = ck.load_moe_layer(path, PREFIX, experts)
    assert (layer.hidden, layer.intermediate, layer.experts) == (hidden, inter, experts)
    assert np.array_equal(layer.w1.values.numpy(), o.pack_fp6(w1c.reshape(-1, hidden)).reshape(-1))
    assert np.array_equal(layer.w1.scales.numpy(), o.pack_scales(w1s.reshape(-1, hidden // 32)))
    assert np.array_equal(layer.w2.values.numpy(), o.pack_fp6(w2c.reshape(-1, inter)).reshape(-1))
    assert np.array_equal(layer.w2.scales.numpy(), o.pack_scales(w2s.reshape(-1, inter // 32)))
    assert torch.equal(layer.combined_gate, gate)
    assert (layer.w1.rows, layer.w1.k, layer.w2.rows, layer.w2.k) == (4 * 512, 256, 4 * 256, 256)

    for rank in (0, 1):   # two ranks: rows of gate / up, input columns of down
        half = ck.load_moe_layer(path, PREFIX, experts, tp_rank=rank, tp_size=2)
        lo, hi = rank * 128, (rank + 1) * 128
        want_w1 = np.concatenate([w1c[:, lo:hi], w1c[:, inter + lo: inter + hi]], axis=1)
        want_w1s = np.concatenate([w1s[:, lo:hi], w1s[:, inter + lo: inter + hi]], axis=1)
        assert half.intermediate == 128
        assert np.array_equal(half.w1.values.numpy(), o.pack_fp6(want_w1.reshape(-1, hidden)).reshape(-1))
        assert np.array_equal(half.w1.scales.numpy(), o.pack_scales(want_w1s.reshape(-1, hidden // 32)))
        assert np.array_equal(half.w2.values.numpy(),
                              o.pack_fp6(w2c[:, :, lo:hi].reshape(-1, 128)).reshape(-1))
        assert np.array_equal(half.w2.scales.numpy(),
                              o.pack_scales(w2s[:, :, lo // 32: hi // 32].reshape(-1, 4)))
    with pytest.raises(ValueError):
        ck.load_moe_layer(path, PREFIX, experts, tp_rank=0, tp_size=4)   # 64 rows per rank
    with pytest.raises(KeyError):
        ck.load_moe_layer(path, PREFIX, experts + 1)


def test_dense_linear_directory_with_index_and_slices(tmp_path):
    rng = np.random.default_rng(5)
    n, k = 384, 512
    codes = rng.integers(0, 64, (n, k), dtype=np.uint8)
    scales = rng.integers(100, 140, (n, k // 32), dtype=np.uint8)
    tensors = {"model.layers.3.self_attn.o_proj.weight": torch.from_numpy(o.pack_fp6(codes).reshape(n, -1)),
               "model.layers.3.self_attn.o_proj.weight_scale": torch.from_numpy(scales)}
    ck.save_tensors(tensors, tmp_path / "model-00001-of-00001.safetensors")
    name = "model.layers.3.self_attn.o_proj"
    for with_index in (False, True):
        if with_index:
            (tmp_path / "model.safetensors.index.json").write_text(
                '{"weight_map": {"%s.weight": "model-00001-of-00001.safetensors", '
                '"%s.weight_scale": "model-00001-of-00001.safetensors"}}' % (name, name))
        full = ck.load_linear(tmp_path, name)
        assert (full.rows, full.k) == (n, k)
        assert np.array_equal(full.values.numpy(), o.pack_fp6(codes).reshape(-1))
        assert np.array_equal(full.scales.numpy(), o.pack_scales(scales))
        assert np.array_equal(full.logical_scales.numpy(), scales)
    rows = ck.load_linear(tmp_path, name, rows=slice(128, 384))          # column-parallel shard
    assert np.array_equal(rows.values.numpy(), o.pack_fp6(codes[128:]).reshape(-1))
    assert np.array_equal(rows.scales.numpy(), o.pack_scales(scales[128:]))
    cols = ck.load_linear(tmp_path, name, input_columns=slice(256, 512))  # row-parallel shard
    assert (cols.rows, cols.k) == (n, 256)
    assert np.array_equal(cols.values.numpy(), o.pack_fp6(codes[:, 256:]).reshape(-1))
    assert np.array_equal(cols.scales.numpy(), o.pack_scales(scales[:, 8:]))
    with pytest.raises(ValueError):
        ck.load_linear(tmp_path, name, input_columns=slice(64, 512))
    with pytest.raises(KeyError):
        ck.load_linear(tmp_path, "model.layers.4.self_attn.o_proj")


@pytest.mark.gpu
def test_layer_read_from_disk_computes_what_the_layer_in_memory_does(tmp_path):
    from mxfp6_sm120_b200.moe_layer import MoeLayer

    dev = torch.device("cuda", 0)
    shape = mx.MoeShape(hidden=1024, intermediate=256, experts=16, topk=8)
    layer = MoeLayer.random(dev, shape, seed=77)
    e, i, h = shape.experts, shape.intermediate, shape.hidden
    gen = torch.Generator(device=dev).manual_seed(78)
    gate_w = (torch.randn((e + 1, h), generator=gen, device=dev) * 0.05).to(torch.bfloat16)

    def logical(p):
        return mx.unpack_scales(p.scales, p.rows, p.k)

    w1_codes = torch.cat([layer.w1.values.view(e, 2 * i, -1), layer.shared_w1.values.view(1, 2 * i, -1)])
    w2_codes = torch.cat([layer.w2.values.view(e, h, -1), layer.shared_w2.values.view(1, h, -1)])
    w1_scales = torch.cat([logical(layer.w1).view(e, 2 * i, -1), logical(layer.shared_w1).view(1, 2 * i, -1)])
    w2_scales = torch.cat([logical(layer.w2).view(e, h, -1), logical(layer.shared_w2).view(1, h, -1)])
    path = tmp_path / "layer.safetensors"
    ck.save_tensors(ck.moe_layer_tensors(PREFIX, h, i, w1_codes, w1_scales, w2_codes, w2_scales, gate_w), path)

    loaded = ck.load_moe_layer(path, PREFIX, e, device=dev)
    again = loaded.moe_layer()
    assert torch.equal(again.w1.values, layer.w1.values) and torch.equal(again.shared_w2.values, layer.shared_w2.values)
    assert torch.equal(mx.unpack_scales(again.w1.scales, again.w1.rows, h), logical(layer.w1))

    for tokens in (2, 40):
        hidden = torch.randn((tokens, h), generator=gen, device=dev).to(torch.bfloat16)
        logits = (hidden.float() @ gate_w[:e].float().t()).to(torch.bfloat16)
        gate = (hidden.float() @ gate_w[e].float()).to(torch.bfloat16)
        want = layer.forward(layer.workspace(tokens), hidden, logits, gate).clone()
        got = again.forward(again.workspace(tokens), hidden, logits, gate)
        assert torch.equal(got, want)

    # the reference's calling form on the stacks as loaded: gate matrix in, three launches
    ws = mx.Qwen35MoeB1Workspace.allocate(dev, shape, batch=2)
    hidden = torch.randn((2, h), generator=gen, device=dev).to(torch.bfloat16)
    out = mx.qwen35_moe_b1_out(ws, hidden, loaded.combined_gate, *loaded.stacks(), renormalize=True)
    want = layer.forward(layer.workspace(2), hidden, ws.routed_logits, ws.shared_gate)
    assert torch.equal(out, want)
    assert mx.device_status() == 0
