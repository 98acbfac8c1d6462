"""Expert-parallel MoE on 2, 4 and 8 GPUs against the single-GPU layer (each case is
skipped when the box has fewer GPUs).

Each rank is a child process (one process per GPU, NCCL).  With NVLS off and no
rank leaving mid-step, as the pool's rules for multi-rank tests ask.
"""

from __future__ import annotations

import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, results) -> None:
    import torch.distributed as dist

    import mxfp6_sm120_b200 as mx
    from mxfp6_sm120_b200.ep import ExpertParallelMoe
    from mxfp6_sm120_b200.moe_layer import MoeLayer

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    device = torch.device("cuda", rank)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    shape = mx.MoeShape(hidden=512, intermediate=256, experts=32, topk=4)
    layer = MoeLayer.random(device, shape, seed=7)  # same seed: identical weights on every rank
    local_tokens = 5
    gen = torch.Generator(device="cpu").manual_seed(11)
    hidden = torch.randn((world * local_tokens, shape.hidden), generator=gen).to(torch.bfloat16).to(device)
    logits = torch.randn((world * local_tokens, shape.experts), generator=gen).to(torch.bfloat16).to(device)
    gate = torch.randn((world * local_tokens,), generator=gen).to(torch.bfloat16).to(device)
    # single-GPU result over all tokens
    state = layer.workspace(world * local_tokens)
    want = layer.forward(state, hidden, logits, gate).clone()
    want_ids = (state.decode if state.decode is not None else state.workspace).topk_ids
    # expert parallel over the ranks
    mine = slice(rank * local_tokens, (rank + 1) * local_tokens)
    moe = ExpertParallelMoe(layer)
    ep_state = moe.state(local_tokens)
    got = moe.forward(ep_state, hidden[mine].contiguous(), logits[mine].contiguous(), gate[mine].contiguous())
    torch.cuda.synchronize()
    cos = torch.nn.functional.cosine_similarity(got.float().flatten(), want[mine].float().flatten(), dim=0)
    same_ids = torch.equal(ep_state.local.topk_ids, want_ids[mine])
    # the same layer with both exchanges over peer memory (one kernel each), eager and replayed
    from mxfp6_sm120_b200.tp_fused import SymmetricBlocks

    peer = SymmetricBlocks(world * local_tokens, shape.hidden, device)
    moe_p = ExpertParallelMoe(layer, peer=peer)
    state_p = moe_p.state(local_tokens)
    assert state_p.dispatch is not None
    args = (hidden[mine].contiguous(), logits[mine].contiguous(), gate[mine].contiguous())
    got_p = moe_p.forward(state_p, *args).clone()
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        dist.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            moe_p.forward(state_p, *args)
        for _ in range(3):
            graph.replay()
        stream.synchronize()
    replay_equal = bool(torch.equal(state_p.output, got_p))
    cos_p = torch.nn.functional.cosine_similarity(got_p.float().flatten(), want[mine].float().flatten(), dim=0)
    same_ids_p = torch.equal(state_p.local.topk_ids, want_ids[mine])
    results[rank] = (bool(same_ids and same_ids_p), float(min(cos, cos_p)), mx.device_status(),
                     replay_equal)
    dist.barrier()
    torch.cuda.synchronize()
    os._exit(0)  # no NCCL teardown: every rank has reported and is between steps


@pytest.mark.parametrize("world", [2, 4, 8])
def test_expert_parallel_matches_single_gpu_layer(world):
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    for rank in range(world):
        same_ids, cos, status, replay_equal = results[rank]
        assert same_ids and cos >= 0.999 and status == 0 and replay_equal
