"""CPU (gloo, world_size 2) test of the expert-parallel choreography.

The collectives, the expert partition, the expert map and the combine index are
the ones ``mxfp6_sm120_b200.ep`` uses; the per-rank expert math is the CPU oracle.
The combined result must equal the oracle's single-process layer.
"""

from __future__ import annotations

import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mxfp6_sm120_b200 import ep
from oracle import mx_oracle as o

HIDDEN, INTER, EXPERTS, TOPK, LOCAL_TOKENS = 128, 64, 8, 2, 3


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _layer():
    gen = torch.Generator(device="cpu").manual_seed(1)
    w1 = (torch.randn((EXPERTS, 2 * INTER, HIDDEN), generator=gen) * 0.05).to(torch.bfloat16)
    w2 = (torch.randn((EXPERTS, HIDDEN, INTER), generator=gen) * 0.05).to(torch.bfloat16)
    w1q = [o.quantize_mxfp6(w1[e]) for e in range(EXPERTS)]
    w2q = [o.quantize_mxfp6(w2[e]) for e in range(EXPERTS)]
    return w1q, w2q


def _tokens(world):
    gen = torch.Generator(device="cpu").manual_seed(2)
    hidden = torch.randn((world * LOCAL_TOKENS, HIDDEN), generator=gen).to(torch.bfloat16)
    logits = torch.randn((world * LOCAL_TOKENS, EXPERTS), generator=gen).to(torch.bfloat16)
    return hidden, logits


def _expert_rows(x, w1, w2):
    h1 = x @ o.dequant_mxfp6(*w1).t()
    codes, scales = o.silu_and_mul_mxfp8(h1)
    return (o.dequant_mxfp8(codes, scales) @ o.dequant_mxfp6(*w2).t()).to(torch.bfloat16)


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        w1q, w2q = _layer()
        hidden_all, logits_all = _tokens(world)
        mine = slice(rank * LOCAL_TOKENS, (rank + 1) * LOCAL_TOKENS)
        hidden, logits = hidden_all[mine], logits_all[mine]
        # 1. local quantize + top-k
        weights, ids = o.softmax_topk(logits, TOPK, True)
        codes, scales = o.quantize_mxfp8_torch(hidden)
        # 2. dispatch (dense all-gather of rows, ids, weights)
        def gather(t):
            parts = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(parts, t.contiguous())
            return torch.cat(parts)
        g_codes, g_scales = gather(torch.from_numpy(codes)), gather(torch.from_numpy(scales))
        g_ids, g_weights = gather(ids), gather(weights)
        # 3. local experts through the expert map
        expert_map = ep.make_expert_map(EXPERTS, world, rank, "cpu")
        begin, end = ep.expert_range(EXPERTS, world, rank)
        assert expert_map[begin:end].tolist() == list(range(end - begin))
        acts = o.dequant_mxfp8(g_codes.numpy(), g_scales.numpy())
        partial = torch.zeros((world * LOCAL_TOKENS, HIDDEN), dtype=torch.float32)
        for t in range(world * LOCAL_TOKENS):
            for r in range(TOPK):
                local = int(expert_map[int(g_ids[t, r])])
                if local < 0:
                    continue
                e = begin + local
                partial[t] += g_weights[t, r] * _expert_rows(acts[t : t + 1], w1q[e], w2q[e])[0].float()
        partial = partial.to(torch.bfloat16)
        # 4. combine: all-to-all of the partial rows, then the sum in rank order
        received = torch.empty_like(partial)
        dist.all_to_all_single(received, partial)
        index = (torch.arange(world).view(1, world) * LOCAL_TOKENS
                 + torch.arange(LOCAL_TOKENS).view(LOCAL_TOKENS, 1))
        out = received.float()[index].sum(dim=1).to(torch.bfloat16)
        # single-process oracle over all tokens
        w1c = {e: w1q[e][0] for e in range(EXPERTS)}
        w1s = {e: w1q[e][1] for e in range(EXPERTS)}
        w2c = {e: w2q[e][0] for e in range(EXPERTS)}
        w2s = {e: w2q[e][1] for e in range(EXPERTS)}
        want, want_ids = o.moe_layer(hidden_all, logits_all, w1c, w1s, w2c, w2s, None, None, TOPK, True)
        cos = torch.nn.functional.cosine_similarity(out.float().flatten(), want[mine].float().flatten(), dim=0)
        results[rank] = (bool(torch.equal(ids, want_ids[mine])), float(cos))
    finally:
        dist.destroy_process_group()


def test_expert_parallel_choreography_matches_single_process_oracle():
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    for rank in range(world):
        same_ids, cos = results[rank]
        assert same_ids and cos >= 0.999


def test_expert_ranges_partition_the_experts():
    for experts, world in ((256, 8), (256, 3), (8, 2), (10, 4)):
        edges = [ep.expert_range(experts, world, r) for r in range(world)]
        assert edges[0][0] == 0 and edges[-1][1] == experts
        assert all(a[1] == b[0] for a, b in zip(edges, edges[1:]))
        total = sum((ep.make_expert_map(experts, world, r, "cpu") >= 0).sum().item() for r in range(world))
        assert total == experts
