"""Run one operator on one synthetic shape a few times (for profilers and quick timing).

    python -m mxfp6_sm120_b200.run_shape --op gemm --m 16 --n 34816 --k 5120 --iters 3
    python -m mxfp6_sm120_b200.run_shape --op quantize --m 8192 --k 5120
    python -m mxfp6_sm120_b200.run_shape --op moe --m 32
    python -m mxfp6_sm120_b200.run_shape --op decode --m 32 --context 4000 --layers 2
    python -m mxfp6_sm120_b200.run_shape --op prefill --m 8192 --layers 1

Prints the mean device time per call: ``--iters`` calls are captured in one CUDA graph
and the replay is timed with CUDA events.
"""

from __future__ import annotations

import argparse

import torch

import mxfp6_sm120_b200 as mx


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--op", default="gemm", choices=["gemm", "quantize", "moe", "decode", "prefill"])
    parser.add_argument("--m", type=int, default=16)
    parser.add_argument("--n", type=int, default=34816)
    parser.add_argument("--k", type=int, default=5120)
    parser.add_argument("--iters", type=int, default=3)
    parser.add_argument("--tile", type=int, default=0)
    parser.add_argument("--splits", type=int, default=0)
    parser.add_argument("--context", type=int, default=4000)
    parser.add_argument("--layers", type=int, default=2)
    args = parser.parse_args()
    device = torch.device("cuda:0")
    gen = torch.Generator(device=device).manual_seed(0)
    a = torch.randn((args.m, args.k), generator=gen, device=device).to(torch.bfloat16)
    if args.op == "quantize":
        def call():
            return mx.quantize_mxfp8(a)
    elif args.op == "gemm":
        values = torch.randint(0, 256, (args.n * args.k * 3 // 4,), generator=gen, dtype=torch.uint8,
                               device=device)
        scales = torch.randint(118, 124, (mx.packed_scale_numel(args.n, args.k),), generator=gen,
                               dtype=torch.uint8, device=device)
        weight = mx.PackedMXFP6Tensor(values, scales, args.n, args.k)
        act = mx.quantize_mxfp8(a)

        def call():
            return mx.gemm_w6a8_config(act, weight, out_dtype=torch.bfloat16, tile_tokens=args.tile,
                                       splits=args.splits)
    elif args.op in ("decode", "prefill"):
        # --m sequences with --context cached tokens each, or one sequence of --m tokens,
        # through --layers layers of the 27B-class dense decoder.
        cfg = mx.DecoderConfig()
        model = mx.DenseDecoder.random(cfg, device, seed=5000, layers=args.layers)
        space = model.workspace(args.m)
        space.x.copy_(torch.randn((args.m, cfg.hidden), generator=gen, device=device).to(torch.bfloat16))
        if args.op == "decode":
            cache = model.new_kv_cache(args.m, args.context + 1)

            def call():
                return model.decode_step(space, cache, args.context)
        else:
            def call():
                return model.prefill(space)
    else:
        from mxfp6_sm120_b200.moe_layer import MoeLayer

        layer = MoeLayer.random(device, mx.MoeShape(), seed=4000)
        hidden = torch.randn((args.m, 2048), generator=gen, device=device).to(torch.bfloat16)
        logits = torch.randn((args.m, 256), generator=gen, device=device).to(torch.bfloat16)
        gate = torch.randn((args.m,), generator=gen, device=device).to(torch.bfloat16)
        state = layer.workspace(args.m)

        def call():
            return layer.forward(state, hidden, logits, gate)

    # Time graph replays so that host launch overhead does not hide short kernels.
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        call()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for _ in range(args.iters):
                call()
        graph.replay()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        graph.replay()
        stop.record(stream)
        stream.synchronize()
    print(f"{args.op} m={args.m} n={args.n} k={args.k}: {start.elapsed_time(stop) * 1e3 / args.iters:.1f} us per call")
    print("device status", mx.device_status())


if __name__ == "__main__":
    main()
