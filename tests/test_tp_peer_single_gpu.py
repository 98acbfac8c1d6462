"""The peer-memory collectives of ``csrc/tp_fused.cu`` for 2, 4 and 8 ranks on ONE GPU.

Every "rank" owns a block allocated on the same device and only rank 0's kernel runs; the
flags of the other ranks are written by the test beforehand, so no kernel waits for another
kernel.  What is checked is the arithmetic (the sum runs over the ranks in order, in FP32,
rounded once to BF16) against plain torch, and the two error paths that leave the context
usable: a peer that never signals (status 301 after a short, bounded wait; the output is
untouched and the step still advances) and two steps in a row on one buffer (status 302).
The reference's reducer has neither check: it spins without a limit
(csrc/moe.cu:7774,7795).
"""

from __future__ import annotations

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

HEADER = 1024
STATE_OFFSET = 32  # eight 32-bit flags, then done_step / finished / last_buffer
FAR_STEP = 1 << 20


class _Blocks:
    """``world`` symmetric blocks on one device, viewed as bytes."""

    def __init__(self, mx, world: int, partial_bytes: int, device: torch.device):
        from mxfp6_sm120_b200._loader import check, library
        from mxfp6_sm120_b200.tp_fused import _DeviceBytes

        self.lib, self.check = library(), check
        self.world, self.partial_bytes, self.device = world, partial_bytes, device
        self.pointers, self.views = [], []
        for _ in range(world):
            block = ctypes.c_void_p()
            handle = (ctypes.c_ubyte * 64)()
            check(self.lib.mxfp6_tp_block_alloc(partial_bytes, ctypes.byref(block), handle))
            self.pointers.append(block.value)
            self.views.append(torch.as_tensor(_DeviceBytes(block.value, HEADER + 2 * partial_bytes),
                                              device=device))
        self.array = (ctypes.c_void_p * world)(*self.pointers)

    def partial(self, rank: int, buffer: int, rows: int, hidden: int) -> torch.Tensor:
        begin = HEADER + buffer * self.partial_bytes
        return self.views[rank][begin: begin + rows * hidden * 2].view(torch.bfloat16).view(rows, hidden)

    def peers_have_signalled(self) -> None:
        """Rank 0 finds every other rank's flag far ahead of any step it will reach."""
        flags = self.views[0][:32].view(torch.int32)
        flags[1: self.world] = FAR_STEP

    def state(self) -> tuple[int, int, int]:
        words = self.views[0][STATE_OFFSET: STATE_OFFSET + 12].view(torch.int32).cpu()
        return int(words[0]), int(words[1]), int(words[2])

    def free(self) -> None:
        torch.cuda.synchronize(self.device)
        self.views = []
        for pointer in self.pointers:
            self.check(self.lib.mxfp6_tp_block_free(ctypes.c_void_p(pointer)))


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _rank_order_sum(parts: list[torch.Tensor]) -> torch.Tensor:
    acc = torch.zeros_like(parts[0], dtype=torch.float32)
    for part in parts:  # FP32, rank 0 first: the order the kernels use
        acc = acc + part.float()
    return acc.to(torch.bfloat16)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_allreduce_reduce_scatter_allgather_sum_in_rank_order(mx, world):
    device = torch.device("cuda", 0)
    rows, hidden = 24, 2048
    blocks = _Blocks(mx, world, rows * hidden * 2, device)
    try:
        gen = torch.Generator(device=device).manual_seed(900 + world)
        parts = []
        for r in range(world):
            for buffer in (0, 1):
                p = torch.randn((rows, hidden), generator=gen, device=device).to(torch.bfloat16)
                blocks.partial(r, buffer, rows, hidden).copy_(p)
                if buffer == 0:
                    parts.append(p)
        parts1 = [blocks.partial(r, 1, rows, hidden).clone() for r in range(world)]
        blocks.peers_have_signalled()

        out = torch.zeros((rows, hidden), dtype=torch.bfloat16, device=device)
        blocks.check(blocks.lib.mxfp6_tp_allreduce_bf16(
            blocks.array, world, 0, 0, blocks.partial_bytes, out.data_ptr(), rows, hidden,
            _stream(device)))
        assert torch.equal(out, _rank_order_sum(parts))

        # reduce-scatter: rank 0 sums ITS slice (the first rows / world rows) of buffer 1
        per_rank = rows // world
        scattered = torch.zeros((per_rank, hidden), dtype=torch.bfloat16, device=device)
        blocks.check(blocks.lib.mxfp6_tp_reduce_scatter_bf16(
            blocks.array, world, 0, 1, blocks.partial_bytes, scattered.data_ptr(), per_rank,
            hidden, _stream(device)))
        assert torch.equal(scattered, _rank_order_sum([p[:per_rank] for p in parts1]))

        # all-gather of two segments of buffer 0: rank r's bytes land at r * segment size
        seg_bytes = [hidden * 2 * 3, 4096]
        offsets = [0, hidden * 2 * 8]
        dsts = [torch.zeros(world * b, dtype=torch.uint8, device=device) for b in seg_bytes]
        blocks.check(blocks.lib.mxfp6_tp_allgather(
            blocks.array, world, 0, 0, blocks.partial_bytes, 2,
            (ctypes.c_int64 * 2)(*offsets), (ctypes.c_int64 * 2)(*seg_bytes),
            (ctypes.c_void_p * 2)(*[d.data_ptr() for d in dsts]), _stream(device)))
        for s in range(2):
            for r in range(world):
                raw = parts[r].view(torch.uint8).reshape(-1)
                want = raw[offsets[s]: offsets[s] + seg_bytes[s]]
                assert torch.equal(dsts[s][r * seg_bytes[s]: (r + 1) * seg_bytes[s]], want)

        # fused form: x += bf16(sum); RMSNorm; MXFP8 == the single-GPU kernel on the same sum
        x = torch.randn((rows, hidden), generator=gen, device=device).to(torch.bfloat16)
        weight = (1.0 + 0.1 * torch.randn((hidden,), generator=gen, device=device)).to(torch.bfloat16)
        want_x = x.clone()
        want_q = mx.rmsnorm_quantize_mxfp8(want_x, weight, 1e-6, residual=_rank_order_sum(parts1))
        values = torch.zeros(rows * hidden, dtype=torch.uint8, device=device)
        scales = torch.zeros(mx.packed_scale_numel(rows, hidden), dtype=torch.uint8, device=device)
        blocks.check(blocks.lib.mxfp6_tp_allreduce_rmsnorm_quantize_mxfp8(
            blocks.array, world, 0, 1, blocks.partial_bytes, x.data_ptr(), weight.data_ptr(),
            ctypes.c_float(1e-6), rows, hidden, values.data_ptr(), scales.data_ptr(),
            _stream(device)))
        torch.cuda.synchronize()
        assert mx.device_status(device) == 0
        assert torch.equal(x, want_x)
        assert torch.equal(values, want_q.values)
        # padding rows of the packed scale buffers are not written: compare the real ones
        assert torch.equal(mx.unpack_scales(scales, rows, hidden),
                           mx.unpack_scales(want_q.scales, rows, hidden))
    finally:
        blocks.free()


def test_same_buffer_twice_is_refused_on_the_device(mx):
    device = torch.device("cuda", 0)
    rows, hidden, world = 8, 1024, 2
    blocks = _Blocks(mx, world, rows * hidden * 2, device)
    try:
        for r in range(world):
            blocks.partial(r, 0, rows, hidden).fill_(1.0)
        blocks.peers_have_signalled()
        out = torch.full((rows, hidden), -7.0, dtype=torch.bfloat16, device=device)
        call = lambda: blocks.check(blocks.lib.mxfp6_tp_allreduce_bf16(  # noqa: E731
            blocks.array, world, 0, 0, blocks.partial_bytes, out.data_ptr(), rows, hidden,
            _stream(device)))
        call()
        torch.cuda.synchronize()
        assert mx.device_status(device) == 0 and bool((out == 2.0).all())
        out.fill_(-7.0)
        call()  # buffer 0 again: a peer could still be reading it
        torch.cuda.synchronize()
        assert mx.device_status(device) == 302          # read and cleared
        assert bool((out == -7.0).all())                # no data was moved
        assert blocks.state()[0] == 2                   # the step advanced all the same
    finally:
        blocks.free()


def test_peer_that_never_signals_ends_as_status_301(mx):
    """The second block belongs to nobody: its flag is never written.  With a limit of
    about a millisecond the kernel gives up, reports 301, leaves ``out`` alone and advances
    the step, and the next call on the context works."""
    device = torch.device("cuda", 0)
    rows, hidden, world = 8, 1024, 2
    blocks = _Blocks(mx, world, rows * hidden * 2, device)
    lib = blocks.lib
    before = lib.mxfp6_tp_get_wait_limit()
    try:
        blocks.check(lib.mxfp6_tp_set_wait_limit(2_000_000))
        for r in range(world):
            blocks.partial(r, 0, rows, hidden).fill_(1.0)
            blocks.partial(r, 1, rows, hidden).fill_(3.0)
        out = torch.full((rows, hidden), -7.0, dtype=torch.bfloat16, device=device)
        blocks.check(lib.mxfp6_tp_allreduce_bf16(
            blocks.array, world, 0, 0, blocks.partial_bytes, out.data_ptr(), rows, hidden,
            _stream(device)))
        torch.cuda.synchronize()
        assert mx.device_status(device) == 301
        assert bool((out == -7.0).all())
        assert blocks.state()[0] == 1
        # the peer "arrives" after all: the next step (other buffer) completes normally
        blocks.peers_have_signalled()
        blocks.check(lib.mxfp6_tp_allreduce_bf16(
            blocks.array, world, 0, 1, blocks.partial_bytes, out.data_ptr(), rows, hidden,
            _stream(device)))
        torch.cuda.synchronize()
        assert mx.device_status(device) == 0
        assert bool((out == 6.0).all())
    finally:
        blocks.check(lib.mxfp6_tp_set_wait_limit(before))
        blocks.free()


@pytest.mark.parametrize("world", [2, 8])
def test_two_phase_allreduce_reduces_its_slice_in_place_and_gathers_by_rank(mx, world):
    """Rank 0's half of the two-phase all-reduce: its slice of rows is summed over all
    ranks (FP32, rank order) and written over its own copy, then the slices are gathered
    rank by rank.  The other ranks' kernels do not run here, so their slices arrive as
    they were: that pins the addressing of both phases."""
    device = torch.device("cuda", 0)
    rows, hidden = 64, 1024
    blocks = _Blocks(mx, world, rows * hidden * 2, device)
    try:
        gen = torch.Generator(device=device).manual_seed(40 + world)
        parts = []
        for r in range(world):
            p = torch.randn((rows, hidden), generator=gen, device=device).to(torch.bfloat16)
            blocks.partial(r, 1, rows, hidden).copy_(p)
            parts.append(p)
        blocks.peers_have_signalled()
        out = torch.zeros((rows, hidden), dtype=torch.bfloat16, device=device)
        blocks.check(blocks.lib.mxfp6_tp_allreduce_two_phase_bf16(
            blocks.array, world, 0, 1, blocks.partial_bytes, out.data_ptr(), rows, hidden,
            _stream(device)))
        torch.cuda.synchronize()
        assert mx.device_status(device) == 0          # two steps on one buffer, by design
        per = rows // world
        assert torch.equal(out[:per], _rank_order_sum([p[:per] for p in parts]))
        for r in range(1, world):
            assert torch.equal(out[r * per: (r + 1) * per], parts[r][r * per: (r + 1) * per])
        assert torch.equal(blocks.partial(0, 1, rows, hidden)[:per], out[:per])   # in place
        assert blocks.state()[0] == 2 and blocks.state()[2] == 2                  # steps, last buffer + 1
        # rows that the ranks cannot share evenly are refused
        assert blocks.lib.mxfp6_tp_allreduce_two_phase_bf16(
            blocks.array, world, 0, 0, blocks.partial_bytes, out.data_ptr(), rows - 1, hidden,
            _stream(device)) == 1
    finally:
        blocks.free()


@pytest.mark.parametrize("world", [2, 4])
def test_reduce_with_the_reference_argument_list_sums_caller_owned_buffers(mx, world):
    """``moe_reduce_tp2_out(..., signal_ptrs, buffer_ptrs, rank)`` as the reference's caller
    makes it (python/mxfp6/ops.py:950-1025): one signal area and one data buffer per rank.
    Rank 0 runs; the other ranks' partials and flags are in place beforehand."""
    device = torch.device("cuda", 0)
    tokens, hidden, topk = 6, 2048, 8
    gen = torch.Generator(device=device).manual_seed(1300 + world)
    routed = torch.randn((tokens * topk, hidden), generator=gen, device=device).to(torch.bfloat16)
    shared = torch.randn((tokens, hidden), generator=gen, device=device).to(torch.bfloat16)
    gate = torch.randn((tokens,), generator=gen, device=device).to(torch.bfloat16)
    weights = torch.rand((tokens, topk), generator=gen, device=device)
    inverse = torch.randperm(tokens * topk, generator=gen, device=device).to(torch.int32)
    signals = torch.zeros((world, 16), dtype=torch.int32, device=device)
    buffers = [torch.randn((tokens, hidden), generator=gen, device=device).to(torch.bfloat16)
               for _ in range(world)]
    signals[0, 1:world] = FAR_STEP   # rank 0 finds every peer far ahead of any step it reaches
    mine = torch.empty((tokens, hidden), dtype=torch.bfloat16, device=device)
    mx.moe_reduce_out(mine, routed, weights, inverse, shared, gate)
    want = _rank_order_sum([mine] + buffers[1:])

    out = torch.zeros((tokens, hidden), dtype=torch.bfloat16, device=device)
    for call in range(2):   # the single buffer is reused: the closing handshake allows it
        mx.moe_reduce_tp2_out(out, routed, weights, inverse, shared, gate,
                              [signals[r].data_ptr() for r in range(world)],
                              [b.data_ptr() for b in buffers], 0)
        torch.cuda.synchronize()
        assert mx.device_status(device) == 0
        assert torch.equal(out, want)
        assert torch.equal(buffers[0], mine)              # the partial went into rank 0's buffer
        state = signals[0, 8:11].cpu().tolist()           # done_step, finished, last_buffer
        assert state == [2 * (call + 1), 0, 2]
    with pytest.raises(ValueError):
        mx.moe_reduce_tp2_out(out, routed, weights, inverse, shared, gate,
                              [signals[0].data_ptr()], [b.data_ptr() for b in buffers], 0)
    with pytest.raises(ValueError):
        mx.moe_reduce_tp2_out(out, routed, weights, inverse, shared, gate,
                              [signals[r].data_ptr() for r in range(world)],
                              [b.data_ptr() for b in buffers], world)
