"""CPU (gloo, world_size 2) test of the symmetric-block set-up protocol.

The CUDA calls are replaced by a fake library: what is checked is the host choreography —
handles travel to every rank, and when ONE rank fails to allocate or to map a peer's block
EVERY rank raises (nobody is left waiting in a collective).
"""

from __future__ import annotations

import contextlib
import ctypes
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class _FakeLibrary:
    """alloc writes a recognisable handle; open fails on the rank / call it is told to."""

    def __init__(self, rank: int, fail_alloc: bool, fail_open: bool):
        self.rank, self.fail_alloc, self.fail_open = rank, fail_alloc, fail_open
        self.opened = []

    def mxfp6_tp_block_alloc(self, partial_bytes, block_ref, handle):
        if self.fail_alloc:
            return 2
        block_ref._obj.value = 0x1000 * (self.rank + 1)
        for i in range(64):
            handle[i] = (self.rank * 7 + i) % 256
        return 0

    def mxfp6_tp_block_open(self, handle, block_ref):
        if self.fail_open:
            return 2
        self.opened.append(bytes(handle))
        block_ref._obj.value = 0x100000 + handle[0]
        return 0


def _worker(rank, world, port, scenario, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from mxfp6_sm120_b200 import tp_fused

        fake = _FakeLibrary(rank, fail_alloc=(scenario == "alloc" and rank == 1),
                            fail_open=(scenario == "open" and rank == 0))

        def check(status):
            if status != 0:
                raise RuntimeError(f"fake CUDA error {status}")

        tp_fused.library = lambda: fake
        tp_fused.check = check
        tp_fused.load_library = lambda: None
        tp_fused._require_sm100 = lambda device: None
        torch.cuda.device = lambda device: contextlib.nullcontext()
        # The view over the block needs a GPU; the protocol under test ends before it.
        tp_fused.torch.as_tensor = lambda holder, device=None: torch.zeros(1, dtype=torch.uint8)
        try:
            blocks = tp_fused.SymmetricBlocks(4, 128, torch.device("cpu"))
            outcome = ("ok", [int(p) for p in blocks._blocks], fake.opened)
        except RuntimeError as error:
            outcome = ("raised", str(error), None)
        results[rank] = outcome
    finally:
        dist.destroy_process_group()


def _run(scenario):
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), scenario, results), nprocs=world, join=True)
    return [results[r] for r in range(world)]


def test_handles_reach_every_rank_and_blocks_are_ordered_by_rank():
    r0, r1 = _run("fine")
    assert r0[0] == "ok" and r1[0] == "ok"
    # own block at the own rank's slot, the peer's mapping at the peer's slot
    assert r0[1][0] == 0x1000 and r1[1][1] == 0x2000
    assert r0[1][1] == 0x100000 + 7 and r1[1][0] == 0x100000 + 0
    assert r0[2] == [bytes((7 + i) % 256 for i in range(64))]
    assert r1[2] == [bytes(i % 256 for i in range(64))]


def test_a_rank_that_cannot_map_a_peer_makes_every_rank_raise():
    for outcome in _run("open"):
        assert outcome[0] == "raised" and "rank 0" in outcome[1]


def test_a_rank_that_cannot_allocate_makes_every_rank_raise():
    for outcome in _run("alloc"):
        assert outcome[0] == "raised"
