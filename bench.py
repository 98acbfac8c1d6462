"""Headline benchmark: the dense W6A8 projection sweep of a 27B-class decoder.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one pass over the 70 shapes of the sweep - five (N, K) projections x
fourteen batch sizes M - each as the call a user makes (BF16 activation ->
MXFP8 quantization -> tcgen05 W6A8 GEMM against packed MXFP6 weights), captured in
one CUDA graph and replayed.  Shapes run M-major so that the 270 MB of packed
weights cycle through the 126 MB L2 between two uses of the same matrix.
Rank 0 prints one JSON line; the value is whole-job TFLOP/s (2*M*N*K summed over
the sweep / step time, max over ranks).

With N > 1 the projections are sharded the way a tensor-parallel decoder shards
them: K = 5120 inputs are column-parallel (split N, no collective), the two
projections that reduce over a wide K (5120x6144, 5120x17408) are row-parallel
(split K) followed by an NCCL all-reduce of the BF16 partials.

``--impl reference`` times the reference's CPU path for the same metric (MXFP6
decode + MXFP8 quantize + FP32 matmul, restated in ``oracle/``) on the host cores.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

NK_SHAPES = [(7168, 5120), (5120, 6144), (34816, 5120), (5120, 17408), (2048, 5120)]
M_VALUES = [1, 2, 4, 8, 16, 24, 32, 64, 96, 512, 1024, 2048, 4096, 8192]
ROW_PARALLEL = {(5120, 6144), (5120, 17408)}
WORKLOAD = "dense W6A8 projection sweep: 5 (N,K) x 14 M, BF16 in -> MXFP8 quant -> GEMM vs packed MXFP6"


def sweep_flops() -> float:
    return float(sum(2 * m * n * k for m in M_VALUES for n, k in NK_SHAPES))


def gemm_bytes(m: int, n: int, k: int) -> int:
    """Algorithmic bytes of one pre-quantized GEMM call."""
    return n * k * 3 // 4 + n * k // 32 + m * k + m * k // 32 + m * n * 2


def load_peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        data["source"] = "measured"
        return data
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


# ------------------------------------------------------------------------------ clocks


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples: list[list[str]] = []
        self._proc: subprocess.Popen | None = None
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _run(self) -> None:
        assert self._proc is not None and self._proc.stdout is not None
        for line in self._proc.stdout:
            fields = [field.strip() for field in line.split(",")]
            if len(fields) >= 6:
                self.samples.append(fields)

    def __enter__(self):
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self._thread.start()
            time.sleep(0.3)  # first samples arrive before the timed region starts
            self.samples.clear()
        except OSError:
            self._proc = None
        return self

    def __exit__(self, *exc):
        if self._proc is not None:
            self._proc.terminate()
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()
            self._thread.join(timeout=5)

    def summary(self) -> dict:
        mhz = sorted(int(s[0]) for s in self.samples if s and s[0].isdigit())
        max_mhz = max((int(s[1]) for s in self.samples if len(s) > 1 and s[1].isdigit()), default=0)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for s in self.samples if len(s) >= 6
                          for i in range(4) if s[2 + i].lower().startswith("active")})
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": max_mhz or None,
                "reasons": reasons, "samples": len(mhz)}


# ------------------------------------------------------------------------------ CPU arm


CPU_SAMPLE_M = (1, 32, 512)
CPU_SAMPLE_ROWS = 4096  # output features of every projection the CPU arm computes


def cpu_reference_sample(threads: int) -> dict:
    """Times the CPU restatement of the path on a bounded sample of the sweep.

    Sample: the first 4096 output features of every one of the five projections at M in
    {1, 32, 512}: quantize the BF16 activation to MXFP8, decode both operands, FP32
    matmul, cast to BF16 (best of 2 each); throughput does not depend on the number of
    output features, the time to decode a whole weight does.  The weights are random
    codes and scales like the GPU arm's; their decode (the reference's helper, a dozen
    elementwise passes) happens once per projection and is reported beside the number.
    """
    from oracle import mx_oracle as o

    torch.set_num_threads(threads)
    flops = 0.0
    seconds = 0.0
    decode_s = 0.0
    rows = []
    for index, (n_full, k) in enumerate(NK_SHAPES):
        n = min(n_full, CPU_SAMPLE_ROWS)
        gen = torch.Generator(device="cpu").manual_seed(1000 + index)
        w_codes = torch.randint(0, 64, (n, k), generator=gen, dtype=torch.uint8).numpy()
        w_scales = torch.randint(118, 124, (n, k // 32), generator=gen, dtype=torch.uint8).numpy()
        t0 = time.perf_counter()
        w_deq = o.dequant_mxfp6(w_codes, w_scales)
        decode_s += time.perf_counter() - t0
        del w_codes, w_scales
        for m in CPU_SAMPLE_M:
            a = torch.randn((m, k), generator=torch.Generator(device="cpu").manual_seed(2000 + m)).to(
                torch.bfloat16)
            best = None
            for _ in range(2):
                t0 = time.perf_counter()
                a_codes, a_scales = o.quantize_mxfp8_torch(a)
                out = (o.dequant_mxfp8(a_codes, a_scales) @ w_deq.t()).to(torch.bfloat16)
                dt = time.perf_counter() - t0
                best = dt if best is None else min(best, dt)
            del out
            flops += 2.0 * m * n * k
            seconds += best
            rows.append({"m": m, "n": n_full, "n_computed": n, "k": k, "ms": round(best * 1e3, 2)})
        del w_deq
    return {"value": flops / seconds / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
            "sample": f"first {CPU_SAMPLE_ROWS} output features of all five (N,K) at M in {{1,32,512}}: "
                      "MXFP8 quantize + decode + FP32 matmul (best of 2 each; weight decode "
                      f"{decode_s:.1f} s for these rows, once per projection, not in the time)",
            "weight_decode_s": decode_s,
            "seconds": seconds, "rows": rows}


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    for _ in range(max(0, min(args.warmup, 1))):
        cpu_reference_sample(threads)
    t0 = time.perf_counter()
    results = [cpu_reference_sample(threads) for _ in range(max(1, min(args.steps, 3)))]
    wall = time.perf_counter() - t0
    value = sum(r["value"] for r in results) / len(results)
    base = results[-1]
    line = {
        "impl": "reference", "metric": "W6A8 GEMM TFLOP/s over the dense M sweep", "value": value,
        "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": len(results), "warmup": min(args.warmup, 1),
        "ms_per_step": wall / len(results) * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "mxfp6 x mxfp8 -> f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": base["sample"]},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": base["cores"],
                         "kind": base["kind"], "sample": base["sample"]},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------ GPU arm


def build_sweep(mx, device, rank: int, world: int):
    """Weights (random packed bytes; every 6-bit pattern is a valid E3M2 code) and
    BF16 activations for every shape, sharded for this rank."""
    from mxfp6_sm120_b200 import tp

    gen = torch.Generator(device=device).manual_seed(1000 + rank)
    layers = {}
    for index, (n, k) in enumerate(NK_SHAPES):
        if world == 1:
            n_loc, k_loc, mode = n, k, "full"
        elif (n, k) in ROW_PARALLEL:
            b, e = tp.shard_bounds(k, world, rank)
            n_loc, k_loc, mode = n, e - b, "row"
        else:
            b, e = tp.shard_bounds(n, world, rank)
            n_loc, k_loc, mode = e - b, k, "column"
        values = torch.randint(0, 256, (n_loc * k_loc * 3 // 4,), generator=gen, dtype=torch.uint8,
                               device=device)
        scales = torch.randint(118, 124, (mx.packed_scale_numel(n_loc, k_loc),), generator=gen,
                               dtype=torch.uint8, device=device)
        layers[(n, k)] = (mx.PackedMXFP6Tensor(values, scales, n_loc, k_loc), mode)
    acts = {}
    for m in M_VALUES:
        for (n, k), (weight, _) in layers.items():
            acts[(m, n, k)] = torch.randn((m, weight.k), generator=gen, device=device,
                                          dtype=torch.float32).to(torch.bfloat16)
    return layers, acts


MOE_BATCHES = [1, 2, 4, 8, 16, 24, 32, 64, 96, 4096]
# DRAM bytes of one launch of the group's kernel, from the ncu capture named here.
SMALL_M_TRAFFIC = {"traffic": 143.7e6, "launch": "M=16 N=34816 K=5120 (139.4 MB read + 3.5..5.3 MB "
                   "written per launch; algorithmic bytes of that launch 140.5e6)",
                   "source": "profiles/w6a8_stream_kernel_m16_k5120.md (dram__bytes_read.sum + "
                             "dram__bytes_write.sum, mean of three launches)"}
QUANT_M = [1, 8, 32, 512, 4096, 8192]


def quantizer_rows(mx, device, stream, peaks) -> dict:
    """The activation quantizer alone: BF16 [M, 5120] ~ N(0,1) with 0.1 % of the entries
    scaled by 50 -> E4M3 codes + packed UE8M0 scales.  20 launches per graph; from 512
    rows on they cycle through input / output sets that together exceed the L2, below
    that the kernel is launch-bound and the 10 KB..330 KB it moves stay in L2."""
    k = 5120
    rows = []
    for m in QUANT_M:
        gen = torch.Generator(device=device).manual_seed(100 + m)
        sets = 1 if m < 512 else max(2, (300 << 20) // (m * k * 3) + 1)
        inputs, values, scales = [], [], []
        for _ in range(sets):
            x = torch.randn((m, k), generator=gen, device=device)
            x = torch.where(torch.rand((m, k), generator=gen, device=device) < 1e-3, x * 50.0, x)
            inputs.append(x.to(torch.bfloat16))
            values.append(torch.empty(m * k, dtype=torch.uint8, device=device))
            scales.append(torch.empty(mx.packed_scale_numel(m, k), dtype=torch.uint8, device=device))
        reps = 20
        from mxfp6_sm120_b200.ops import _quantize_mxfp8_raw

        _quantize_mxfp8_raw(inputs[0], values[0], scales[0], None)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(reps):
                _quantize_mxfp8_raw(inputs[i % sets], values[i % sets], scales[i % sets], None)
        graph.replay()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        best = None
        for _ in range(3):
            start.record(stream)
            graph.replay()
            stop.record(stream)
            stream.synchronize()
            us = start.elapsed_time(stop) * 1e3 / reps
            best = us if best is None else min(best, us)
        byts = m * k * 3 + m * k // 32
        rows.append({"m": m, "k": k, "us": round(best, 2), "gbs": round(byts / best / 1e3, 1),
                     "hbm_frac": round(byts / best / 1e3 / float(peaks["hbm_gbs"]), 3)})
        del inputs, values, scales
    return {"config": "BF16 [M, 5120] ~ N(0,1), 0.1 % of entries x 50 -> MXFP8 (E4M3 + UE8M0 per 32), "
                      "bytes = 3*M*K + M*K/32", "peak": f"hbm_gbs ({peaks['source']})", "rows": rows}


def moe_layer_latency(mx, device, stream, peaks) -> dict:
    """Latency of one routed-MoE layer (hidden 2048, 256 experts, top-8, intermediate 512,
    gated shared expert), one CUDA graph per token batch.  ``us_warm`` = back-to-back
    replays of a graph holding one layer (the reference's method); ``us_warm_stacked`` = per
    layer when the graph holds twenty calls, as a decoder's graph does; ``us_cold`` = L2
    flushed between replays.  ``schedule`` names the path the layer object took."""
    from mxfp6_sm120_b200.moe_layer import MoeLayer

    shape = mx.MoeShape()
    layer = MoeLayer.random(device, shape, seed=4000)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    rows = []
    for batch in MOE_BATCHES:
        gen = torch.Generator(device=device).manual_seed(4100 + batch)
        hidden = torch.randn((batch, shape.hidden), generator=gen, device=device).to(torch.bfloat16)
        logits = torch.randn((batch, shape.experts), generator=gen, device=device).to(torch.bfloat16)
        gate = torch.randn((batch,), generator=gen, device=device).to(torch.bfloat16)
        state = layer.workspace(batch)
        layer.forward(state, hidden, logits, gate)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            layer.forward(state, hidden, logits, gate)
        for _ in range(3):
            graph.replay()
        reps = 50 if batch <= 96 else 10
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        for _ in range(reps):
            graph.replay()
        stop.record(stream)
        stream.synchronize()
        warm = start.elapsed_time(stop) * 1e3 / reps
        cold = []
        for _ in range(10):
            flush.fill_(1)
            start.record(stream)
            graph.replay()
            stop.record(stream)
            stream.synchronize()
            cold.append(start.elapsed_time(stop) * 1e3)
        cold.sort()
        stacked = None
        if batch <= 96:
            deep = torch.cuda.CUDAGraph()
            with torch.cuda.graph(deep, stream=stream):
                for _ in range(20):
                    layer.forward(state, hidden, logits, gate)
            for _ in range(2):
                deep.replay()
            start.record(stream)
            for _ in range(5):
                deep.replay()
            stop.record(stream)
            stream.synchronize()
            stacked = round(start.elapsed_time(stop) * 1e3 / 100, 1)
        decode = state.decode is not None
        used = int(torch.unique((state.decode if decode else state.workspace).topk_ids).numel())
        byts = (used + 1) * 2457600 + batch * shape.hidden * 4 + batch * shape.experts * 2
        flops = 9.0 * batch * 6291456
        cold_us = cold[len(cold) // 2]
        rows.append({"tokens": batch, "schedule": "decode" if decode else "grouped",
                     "us_warm": round(warm, 1), "us_warm_stacked": stacked, "us_cold": round(cold_us, 1),
                     "experts_hit": used, "gbs_cold": round(byts / cold_us / 1e3, 0),
                     "hbm_frac_cold": round(byts / cold_us / 1e3 / float(peaks["hbm_gbs"]), 3),
                     "tflops_warm": round(flops / warm / 1e6, 1)})
    return {"config": "hidden 2048, 256 experts, top-8 softmax renormalised, intermediate 512, "
                      "shared expert with sigmoid gate; router logits are inputs",
            "rows": rows}


def moe_layer_latency_ep(mx, device, stream, world: int, rank: int) -> dict:
    """The same layer with the 256 routed experts sharded over the ranks: all-gather
    dispatch of the MXFP8 rows, local grouped GEMMs, all-to-all combine.  Token batches
    are global; each rank brings batch / world tokens (batches smaller than the world
    size are skipped).  Latency = max over ranks of the graph replay time."""
    import torch.distributed as dist

    from mxfp6_sm120_b200.ep import ExpertParallelMoe
    from mxfp6_sm120_b200.moe_layer import MoeLayer

    from mxfp6_sm120_b200.tp_fused import SymmetricBlocks

    shape = mx.MoeShape()
    layer = MoeLayer.random(device, shape, seed=4000)
    try:  # raises on every rank alike when any rank could not map a peer's block
        peer = SymmetricBlocks(ExpertParallelMoe.PEER_MAX_TOKENS, shape.hidden, device)
    except RuntimeError:
        peer = None
    moe = ExpertParallelMoe(layer, peer=peer)
    del layer
    rows = []
    for batch in MOE_BATCHES:
        if batch % world:
            continue
        local = batch // world
        gen = torch.Generator(device=device).manual_seed(4100 + batch + rank)
        hidden = torch.randn((local, shape.hidden), generator=gen, device=device).to(torch.bfloat16)
        logits = torch.randn((local, shape.experts), generator=gen, device=device).to(torch.bfloat16)
        gate = torch.randn((local,), generator=gen, device=device).to(torch.bfloat16)
        state = moe.state(local)
        moe.forward(state, hidden, logits, gate)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            moe.forward(state, hidden, logits, gate)
        for _ in range(3):
            graph.replay()
        reps = 30 if batch <= 96 else 10
        dist.barrier()
        torch.cuda.synchronize(device)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        for _ in range(reps):
            graph.replay()
        stop.record(stream)
        stream.synchronize()
        t = torch.tensor([start.elapsed_time(stop) * 1e3 / reps], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        rows.append({"tokens": batch, "tokens_per_rank": local, "us_warm": round(float(t.item()), 1)})
    return {"config": f"expert parallel over {world} ranks ({shape.experts // world} experts each): "
                      "all-gather dispatch, all-to-all combine, shared expert replicated; up to "
                      f"{ExpertParallelMoe.PEER_MAX_TOKENS} tokens both exchanges are one "
                      "peer-memory kernel each, above that NCCL",
            "rows": rows}


def decoder_step_latency(mx, device, stream, world: int, rank: int) -> dict:
    """Decode (32 sequences, 4000-token context) and prefill (8192 tokens) step of the
    64-layer 27B-class dense decoder, every linear W6A8, CUDA-graph replayed; under
    torchrun the layers are tensor parallel (heads and MLP columns per rank, NCCL
    all-reduce after the two row-parallel projections).  Max over ranks."""
    import torch.distributed as dist

    cfg = mx.DecoderConfig()
    group = dist.group.WORLD if world > 1 else None
    with torch.cuda.stream(stream):
        model = mx.DenseDecoder.random(cfg, device, seed=5000, world=world, rank=rank, group=group)
    weight_bytes = model.weight_bytes()
    nccl_model = None
    if world > 1:
        # The product path reduces the row-parallel projections inside the residual + norm +
        # quantize kernel over peer memory; the NCCL all-reduce variant is timed beside it.
        from mxfp6_sm120_b200.tp_fused import SymmetricBlocks

        nccl_model = model
        try:  # raises on every rank alike when any rank could not map a peer's block
            peer = SymmetricBlocks(512, cfg.hidden, device, group)
            model = mx.DenseDecoder(cfg, nccl_model.layers, world, rank, group, peer)
        except RuntimeError:  # CUDA IPC not available between these GPUs: NCCL only
            nccl_model = None

    def timed(step, reps):
        with torch.cuda.stream(stream):
            step()
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                step()
            graph.replay()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize(device)
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record(stream)
            for _ in range(reps):
                graph.replay()
            stop.record(stream)
            stream.synchronize()
        t = torch.tensor([start.elapsed_time(stop) / reps], device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    out = {"config": "64 layers, hidden 5120, 24 query / 4 KV heads of 256, MLP 17408, RMSNorm; "
                     "BF16 attention (torch SDPA), all linears W6A8; random-init weights",
           "parallelism": "single GPU" if world == 1 else f"tp{world}",
           "weight_bytes_per_rank": weight_bytes}
    batch, context = 32, 4000
    ws = model.workspace(batch)
    cache = model.new_kv_cache(batch, context + 1)
    gen = torch.Generator(device=device).manual_seed(5100)
    ws.x.copy_(torch.randn((batch, cfg.hidden), generator=gen, device=device).to(torch.bfloat16))
    decode_ms = timed(lambda: model.decode_step(ws, cache, context), 5)
    kv_bytes = 2 * len(cache) * cache[0][0].numel() * 2
    out["decode"] = {"sequences": batch, "context": context, "ms_per_step": round(decode_ms, 3),
                     "tokens_per_s": round(batch / (decode_ms * 1e-3), 1),
                     "gbs_weights_plus_kv": round((weight_bytes + kv_bytes) / (decode_ms * 1e-3) / 1e9, 1)}
    if nccl_model is not None:
        out["decode"]["all_reduce"] = "fused into the norm kernel over peer memory"
        out["decode"]["ms_per_step_nccl_all_reduce"] = round(
            timed(lambda: nccl_model.decode_step(ws, cache, context), 5), 3)
    del cache, ws
    torch.cuda.empty_cache()
    tokens = 8192
    ws = model.workspace(tokens)
    ws.x.copy_(torch.randn((tokens, cfg.hidden), generator=gen, device=device).to(torch.bfloat16))
    prefill_ms = timed(lambda: model.prefill(ws), 2)
    prefill_nccl_ms = timed(lambda: nccl_model.prefill(ws), 2) if nccl_model is not None else None
    hd = cfg.head_dim
    linear_flops = 2.0 * tokens * cfg.layers * cfg.hidden * (
        (cfg.q_heads + 2 * cfg.kv_heads) * hd + cfg.q_heads * hd + 3 * cfg.intermediate)
    out["prefill"] = {"tokens": tokens, "ms_per_step": round(prefill_ms, 2),
                      "tokens_per_s": round(tokens / (prefill_ms * 1e-3), 1),
                      "linear_tflops_whole_job": round(linear_flops / (prefill_ms * 1e-3) / 1e12, 1)}
    if prefill_nccl_ms is not None:
        out["prefill"]["ms_per_step_nccl_all_reduce"] = round(prefill_nccl_ms, 2)
    del ws, model
    torch.cuda.empty_cache()
    return out


def _rel(got: torch.Tensor, want: torch.Tensor) -> float:
    return float((got.float() - want.float()).norm() / want.float().norm().clamp_min(1e-30))


def parity_check_sharded(mx, device, world: int, rank: int) -> dict:
    """Outside every timed region: the sharded paths the N-GPU run times against the same
    computation on one GPU.  A 5120 x 6144 projection from one seed on every rank, split
    by columns (no collective) and by rows (partials summed by the peer-memory kernel at 16
    rows, by NCCL at 512), against the unsharded GEMM; and one expert-parallel MoE layer
    against the single-GPU layer on this rank's tokens.  Max over ranks."""
    import torch.distributed as dist

    from mxfp6_sm120_b200 import tp
    from mxfp6_sm120_b200.ep import ExpertParallelMoe
    from mxfp6_sm120_b200.moe_layer import MoeLayer
    from mxfp6_sm120_b200.tp_fused import SymmetricBlocks

    n, k = 5120, 6144
    gen = torch.Generator(device=device).manual_seed(4242)  # the same tensors on every rank
    values = torch.randint(0, 256, (n * k * 3 // 4,), generator=gen, dtype=torch.uint8, device=device)
    scales = torch.randint(118, 124, (mx.packed_scale_numel(n, k),), generator=gen,
                           dtype=torch.uint8, device=device)
    full = mx.PackedMXFP6Tensor(values, scales, n, k)
    try:
        peer = SymmetricBlocks(16, n, device)
    except RuntimeError:
        peer = None
    row = tp.RowParallelLinear(mx, tp.shard_row_parallel(values, scales, n, k, world, rank), peer=peer)
    col = tp.ColumnParallelLinear(mx, tp.shard_column_parallel(values, scales, n, k, world, rank))
    cases = {}
    for m in (16, 512):
        a = torch.randn((m, k), generator=gen, device=device).to(torch.bfloat16)
        want = mx.gemm_from_float(a, full, out_dtype=torch.bfloat16)
        got_row = row(a[:, row.shard.begin:row.shard.end].contiguous())
        got_col = col(a)
        cases[f"row_parallel_m{m}"] = _rel(got_row, want)
        cases[f"column_parallel_m{m}"] = _rel(got_col, want[:, col.shard.begin:col.shard.end])
    torch.cuda.synchronize(device)
    if peer is not None:
        peer.close()
    # expert-parallel layer against the single-GPU layer on this rank's tokens
    shape = mx.MoeShape()
    layer = MoeLayer.random(device, shape, seed=4000)
    moe = ExpertParallelMoe(layer, peer=None)
    local = 8
    gen_t = torch.Generator(device=device).manual_seed(4300 + rank)
    hidden = torch.randn((local, shape.hidden), generator=gen_t, device=device).to(torch.bfloat16)
    logits = torch.randn((local, shape.experts), generator=gen_t, device=device).to(torch.bfloat16)
    gate = torch.randn((local,), generator=gen_t, device=device).to(torch.bfloat16)
    got = moe.forward(moe.state(local), hidden, logits, gate).clone()
    want = layer.forward(layer.workspace(local), hidden, logits, gate)
    cos = float(torch.nn.functional.cosine_similarity(got.float().flatten(), want.float().flatten(), dim=0))
    cases["expert_parallel_layer_1_minus_cos"] = 1.0 - cos
    del layer, moe
    torch.cuda.empty_cache()
    keys = sorted(cases)
    t = torch.tensor([cases[key] for key in keys], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    worst = {key: float(v) for key, v in zip(keys, t.tolist())}
    # Row-parallel partials are rounded to BF16 before they are summed: a few 1e-3 from the
    # unsharded sum; column-parallel differs only in the order of the K split.
    limits = {key: (1e-2 if key.startswith("row") else 1e-3) for key in keys}
    ok = all(worst[key] <= limits[key] for key in keys) and mx.device_status(device) == 0
    return {"ok": bool(ok), "max_rel": max(v for key, v in worst.items() if "parallel_m" in key),
            "cases": {key: float(f"{v:.3e}") for key, v in worst.items()},
            "limits": "row-parallel 1e-2, column-parallel 1e-3 (rel-Frobenius), layer 1 - cos 1e-3"}


def plan_row_sums(row_sum: str, world: int):
    """Host logic of the sharded sweep: the order of the (M, N, K) launches of a step and which
    row-parallel outputs one NCCL all-reduce sums (``groups``: lists of launch keys whose
    outputs share one buffer; the sum is issued after the LAST key of a group has run).

    One GPU: M-major in the listed order, nothing to sum.  Sharded: large batches first (their
    sums are the long pole) and row / column shapes alternating (row, column, row, column,
    column: every sum has a GEMM to run beside); with merged sums every prefill-sized
    row-parallel GEMM comes before all the others."""
    if world == 1:
        return [], [(m, n, k) for m in M_VALUES for (n, k) in NK_SHAPES]
    m_order = sorted(M_VALUES, reverse=True)
    rows_first = [s for s in NK_SHAPES if s in ROW_PARALLEL]
    columns = [s for s in NK_SHAPES if s not in ROW_PARALLEL]
    mixed = [rows_first[0], columns[0], rows_first[1]] + columns[1:]
    large = [m for m in m_order if m > 256]
    large_rows = [(m, *s) for m in large for s in rows_first]
    groups = []
    if row_sum == "nccl_pair":
        groups = [[(m, *s) for s in rows_first] for m in m_order]
    elif row_sum == "nccl_merged":
        groups = [large_rows[: len(rows_first)], large_rows[len(rows_first):]]
    elif row_sum == "nccl_early":
        groups = [large_rows[:1], large_rows[1:]]
    if row_sum in ("nccl_merged", "nccl_early"):
        order = (large_rows + [(m, *s) for m in large for s in columns]
                 + [(m, *s) for m in m_order if m <= 256 for s in mixed])
    else:
        order = [(m, *s) for m in m_order for s in mixed]
    return groups, order


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=100)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--row-sum", default="auto",
                        choices=["auto", "nccl", "nccl_pair", "nccl_merged", "nccl_early", "peer"],
                        help="N > 1: sum of the prefill-sized row-parallel outputs: one NCCL "
                             "all-reduce per projection, one per batch size over both projections' "
                             "outputs, two over all prefill batches, or this library's two-phase "
                             "peer-memory kernels.  auto = nccl_early at 8 GPUs, nccl_pair below "
                             "(measured TFLOP/s at 8 GPUs: nccl 4835, nccl_pair 5054, nccl_merged "
                             "5268, peer 4287; at 2 GPUs: 3070, 3168, 3006, 3037; nccl_early is "
                             "nccl_merged with its first sum one GEMM earlier)")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-e2e", action="store_true")
    parser.add_argument("--no-moe", action="store_true")
    parser.add_argument("--no-decoder", action="store_true")
    parser.add_argument("--no-per-shape", action="store_true",
                        help="skip the per-shape GEMM-only timing (used for profiler launch lists)")
    args = parser.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return

    import torch.distributed as dist

    import mxfp6_sm120_b200 as mx

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    warmup = max(3, args.warmup)
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    mx.load_library()  # ImportError if the CUDA library is missing: there is no fallback
    if not mx.is_available():
        raise RuntimeError("bench.py needs an sm_100 GPU and libmxfp6_b200.so")
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    peaks = load_peaks()

    parity = None
    if world > 1:
        parity = parity_check_sharded(mx, device, world, rank)
    if args.row_sum == "auto":
        args.row_sum = "nccl_early" if world >= 8 else "nccl_pair"

    layers, acts = build_sweep(mx, device, rank, world)
    outs = {key: torch.empty((key[0], layers[key[1:]][0].rows), dtype=torch.bfloat16, device=device)
            for key in acts}
    # Sharded: which row-parallel outputs one all-reduce sums.  nccl = one per projection;
    # nccl_pair = both projections of a batch size in one buffer; nccl_merged = the prefill
    # batches in two buffers (8192 rows; 4096 down to 512 rows), whose GEMMs all run first so
    # that two large all-reduces run beside every column-parallel GEMM of the step;
    # nccl_early = the same two all-reduces, the first one over the first GEMM's output alone
    # so that the sums start one GEMM into the step.
    rows_first = [s for s in NK_SHAPES if s in ROW_PARALLEL]
    sum_groups, order = plan_row_sums(args.row_sum, world)
    row_pairs = {}
    for group in sum_groups:
        width = layers[rows_first[0]][0].rows
        assert all(layers[key[1:]][0].rows == width for key in group)
        flat = torch.empty((sum(key[0] for key in group), width), dtype=torch.bfloat16, device=device)
        begin = 0
        for key in group:
            outs[key] = flat[begin: begin + key[0]]
            begin += key[0]
            row_pairs[key] = (flat, group[-1])   # summed after the group's last GEMM
    # Prefill-sized row-parallel sums (NCCL, bandwidth bound) run on a side stream beside the
    # GEMMs of the following shapes; the sweep's shapes do not depend on one another.
    reduce_stream = torch.cuda.Stream(device) if world > 1 else None

    def run_shape(key, a=None):
        weight, mode = layers[key[1:]]
        out = mx.gemm_from_float(acts[key] if a is None else a, weight, out_dtype=torch.bfloat16,
                                 out=outs[key])
        if mode == "row" and world > 1:
            pair = row_pairs.get(key)
            if pair is not None and key != pair[1]:
                return out          # summed together with the other outputs of its group
            computed = torch.cuda.Event()
            computed.record(torch.cuda.current_stream(device))
            reduce_stream.wait_event(computed)
            with torch.cuda.stream(reduce_stream):
                dist.all_reduce(out if pair is None else pair[0])
        return out

    def run_shape_peer(key, peer):
        """Row-parallel shape with a decode-sized output: partial into the symmetric block,
        then one peer-memory kernel sums the ranks' partials into the output."""
        weight, _ = layers[key[1:]]
        partial = peer.next_partial(key[0], weight.rows)
        mx.gemm_from_float(acts[key], weight, out_dtype=torch.bfloat16, out=partial)
        return peer.allreduce(outs[key])

    sweep_peer = big_peer = None
    if world > 1:
        from mxfp6_sm120_b200 import tp
        from mxfp6_sm120_b200.tp_fused import SymmetricBlocks

        try:  # raises on every rank alike when any rank could not map a peer's block
            sweep_peer = SymmetricBlocks(tp.PEER_ALLREDUCE_MAX_ROWS, max(n for n, _ in ROW_PARALLEL),
                                         device)
            if args.row_sum == "peer":
                big_peer = SymmetricBlocks(max(M_VALUES), max(n for n, _ in ROW_PARALLEL), device)
        except RuntimeError:
            sweep_peer = big_peer = None
    last_sum = [None]

    def run_shape_peer_big(key):
        """Row-parallel shape with a prefill-sized output: partial into the large symmetric
        block, then the two-phase peer-memory sum (every rank sums its slice of rows in place,
        all gather the slices) on the side stream.  A partial buffer is written again two sums
        later; the GEMM that does so waits for the sum in between, whose handshake shows that
        every peer has finished reading that buffer."""
        weight, _ = layers[key[1:]]
        current = torch.cuda.current_stream(device)
        if last_sum[0] is not None:
            current.wait_event(last_sum[0])
        partial = big_peer.next_partial(key[0], weight.rows)
        mx.gemm_from_float(acts[key], weight, out_dtype=torch.bfloat16, out=partial)
        computed = torch.cuda.Event()
        computed.record(current)
        reduce_stream.wait_event(computed)
        with torch.cuda.stream(reduce_stream):
            big_peer.allreduce_any(outs[key])
            done = torch.cuda.Event()
            done.record(reduce_stream)
        last_sum[0] = done
        return outs[key]

    def run_sweep():
        last_sum[0] = None
        for key in order:
            weight, mode = layers[key[1:]]
            if sweep_peer is not None and mode == "row" and key[0] <= tp.PEER_ALLREDUCE_MAX_ROWS:
                run_shape_peer(key, sweep_peer)
            elif big_peer is not None and mode == "row" and key[0] % world == 0:
                run_shape_peer_big(key)
            else:
                run_shape(key)
        if reduce_stream is not None:
            torch.cuda.current_stream(device).wait_stream(reduce_stream)  # the step ends with its sums

    stream = torch.cuda.Stream(device)
    with torch.cuda.stream(stream):
        # plan the split-K arena on the capture stream, then freeze it
        mx.begin_workspace_planning(device)
        run_sweep()
        mx.finalize_workspace_planning(device)
        run_sweep()
        stream.synchronize()
        if world > 1 and parity is not None:
            # The step's own summed outputs (grouped buffers, side stream) against the same
            # GEMM summed by a plain all-reduce of its own: largest and smallest prefill
            # batch of both row-parallel projections, and one decode batch (peer kernel).
            worst = 0.0
            for m in (max(M_VALUES), min(v for v in M_VALUES if v > 256), 16):
                for shape in rows_first:
                    key = (m, *shape)
                    want = mx.gemm_from_float(acts[key], layers[shape][0], out_dtype=torch.bfloat16)
                    dist.all_reduce(want)
                    worst = max(worst, _rel(outs[key], want))
            over_ranks = torch.tensor([worst], device=device)
            dist.all_reduce(over_ranks, op=dist.ReduceOp.MAX)
            worst = float(over_ranks.item())
            parity["cases"]["sweep_row_sums"] = round(worst, 6)
            parity["max_rel"] = max(parity["max_rel"], worst)
            parity["ok"] = bool(parity["ok"] and worst <= 1e-2)
            parity["limits"] += "; sweep_row_sums (the timed step's own summed outputs against GEMM + plain all-reduce) 1e-2"
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            run_sweep()
        launches_per_step = 2 * len(order) + (0 if world == 1 else 2 * len(M_VALUES))

        def barrier():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize(device)

        for _ in range(warmup):
            graph.replay()
        barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local_rank) as clocks:
            start.record(stream)
            for _ in range(args.steps):
                graph.replay()
            stop.record(stream)
            barrier()
        ms_total = start.elapsed_time(stop)
        if world > 1:
            t = torch.tensor([ms_total], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms_total = float(t.item())
        ms_per_step = ms_total / args.steps
        value = sweep_flops() / (ms_per_step * 1e-3) / 1e12

        # ---- where the step goes when it is sharded: quantizers alone, collectives alone
        breakdown = None
        if world > 1:
            def timed_graph(body) -> float:
                body()
                stream.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    body()
                g.replay()
                barrier()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                for _ in range(5):
                    g.replay()
                b.record(stream)
                barrier()
                t = torch.tensor([a.elapsed_time(b) / 5], device=device)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                return float(t.item())

            def quantizers_only():
                for key in order:
                    mx.quantize_mxfp8(acts[key])

            def collectives_only():
                for key in order:
                    _, mode = layers[key[1:]]
                    if mode != "row":
                        continue
                    if sweep_peer is not None and key[0] <= tp.PEER_ALLREDUCE_MAX_ROWS:
                        sweep_peer.next_partial(key[0], layers[key[1:]][0].rows)
                        sweep_peer.allreduce(outs[key])
                    elif big_peer is not None and key[0] % world == 0:
                        big_peer.allreduce_any(outs[key])
                    elif key in row_pairs:
                        if key == row_pairs[key][1]:
                            dist.all_reduce(row_pairs[key][0])
                    else:
                        dist.all_reduce(outs[key])

            breakdown = {"quantize": round(timed_graph(quantizers_only), 4),
                         "collective": round(timed_graph(collectives_only), 4)}

        # ---- GEMM kernel alone (pre-quantized activations), per shape, for the roofline
        per_shape = []
        gemm_ms = 0.0
        small_bytes = small_ms = 0.0
        small_by_m: dict[int, list[float]] = {}
        big_flops = big_ms = 0.0
        if (rank == 0 or world > 1) and not args.no_per_shape:
            quantized = {key: mx.quantize_mxfp8(acts[key]) for key in order}
            # Weight-streaming launches (M <= 96) cycle through copies of the weight that
            # together exceed the L2 (400 MB), 20 launches per graph; the compute-bound ones
            # repeat one weight 5 times.
            copies = {}
            for shape, (weight, _) in layers.items():
                count = max(2, min(16, (400 << 20) // weight.values.numel() + 1))
                copies[shape] = [weight] + [
                    mx.PackedMXFP6Tensor(weight.values.clone(), weight.scales.clone(), weight.rows,
                                         weight.k) for _ in range(count - 1)]
            for key in order:
                weight, _ = layers[key[1:]]
                pool = copies[key[1:]] if key[0] <= 96 else [weight]
                reps = 20 if key[0] <= 96 else 5
                g = torch.cuda.CUDAGraph()
                mx.gemm_w6a8(quantized[key], weight, out_dtype=torch.bfloat16, out=outs[key])
                stream.synchronize()
                with torch.cuda.graph(g, stream=stream):
                    for i in range(reps):
                        mx.gemm_w6a8(quantized[key], pool[i % len(pool)], out_dtype=torch.bfloat16,
                                     out=outs[key])
                shape_start = torch.cuda.Event(enable_timing=True)
                shape_stop = torch.cuda.Event(enable_timing=True)
                g.replay()
                shape_start.record(stream)
                g.replay()
                shape_stop.record(stream)
                stream.synchronize()
                us = shape_start.elapsed_time(shape_stop) * 1e3 / reps
                m = key[0]
                flops = 2.0 * m * weight.rows * weight.k
                byts = gemm_bytes(m, weight.rows, weight.k)
                per_shape.append({"m": m, "n": key[1], "k": key[2], "us": round(us, 2),
                                  "tflops": round(flops / us / 1e6, 1),
                                  "gbs": round(byts / us / 1e3, 0)})
                gemm_ms += us / 1e3
                if m <= 32:
                    small_bytes += byts
                    small_ms += us / 1e3
                    entry = small_by_m.setdefault(m, [0.0, 0.0])
                    entry[0] += byts
                    entry[1] += us
                if m >= 4096:
                    big_flops += flops
                    big_ms += us / 1e3

            del copies, quantized
            torch.cuda.empty_cache()
        small_per_m = {str(m): round(b / us / 1e3 / float(peaks["hbm_gbs"]), 3)
                       for m, (b, us) in sorted(small_by_m.items())}

        quant = None
        if rank == 0 and not args.no_per_shape:
            quant = quantizer_rows(mx, device, stream, peaks)

        # ---- end to end through the public API with host buffers
        e2e = None
        if not args.no_e2e and world == 1:
            host_in = {key: torch.empty(acts[key].shape, dtype=torch.bfloat16).pin_memory()
                       for key in order}
            host_out = {key: torch.empty(outs[key].shape, dtype=torch.bfloat16).pin_memory()
                        for key in order}
            for key in order:
                host_in[key].copy_(acts[key])
            h2d = sum(t.numel() * 2 for t in host_in.values())
            d2h = sum(t.numel() * 2 for t in host_out.values())

            # Three streams: the copy of the next shape's activations from pinned host memory
            # and the copy of the previous shape's output back overlap the GEMMs (PCIe is
            # full duplex), ordered per shape by events.
            copy_in, copy_out = torch.cuda.Stream(device), torch.cuda.Stream(device)

            def e2e_step():
                copy_in.wait_stream(stream)   # the previous step's GEMMs have read the inputs
                for key in order:
                    with torch.cuda.stream(copy_in):
                        acts[key].copy_(host_in[key], non_blocking=True)
                        arrived = torch.cuda.Event()
                        arrived.record(copy_in)
                    stream.wait_event(arrived)
                    out = run_shape(key)
                    computed = torch.cuda.Event()
                    computed.record(stream)
                    copy_out.wait_event(computed)
                    with torch.cuda.stream(copy_out):
                        host_out[key].copy_(out, non_blocking=True)
                stream.wait_stream(copy_in)
                stream.wait_stream(copy_out)   # the step ends when every output is on the host

            e2e_step()
            stream.synchronize()
            e_start, e_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            steps = max(1, min(args.steps, 3))
            e_start.record(stream)
            for _ in range(steps):
                e2e_step()
            e_stop.record(stream)
            stream.synchronize()
            e_ms = e_start.elapsed_time(e_stop) / steps
            e2e = {"value": sweep_flops() / (e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                   "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e_ms}

        moe = None
        if not args.no_moe and world == 1:
            moe = moe_layer_latency(mx, device, stream, peaks)
        elif not args.no_moe:
            moe = moe_layer_latency_ep(mx, device, stream, world, rank)

        decoder = None
        if not args.no_decoder:
            decoder = decoder_step_latency(mx, device, stream, world, rank)

    status = mx.device_status(device)
    if rank != 0:
        finish(world)
        return

    # Every shape is timed alone (graphs of 5 or 20 launches), so the burst figure is the
    # denominator; kind::mxf8f6f4 runs at the FP8 rate, twice the BF16 rate the file measures.
    fp8_peak = 2.0 * float(peaks["bf16_tflops"])
    line = {
        "metric": "W6A8 GEMM TFLOP/s over the dense M sweep", "value": value, "unit": "TFLOP/s",
        "n_gpus": world, "steps": args.steps, "warmup": warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "mxfp6(e3m2) x mxfp8(e4m3) -> f32 accumulate -> bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "shapes": NK_SHAPES, "m_values": M_VALUES,
                   "parallelism": "single GPU" if world == 1 else
                   f"tp{world}: K=5120 projections column-parallel, 5120x6144 and 5120x17408 "
                   "row-parallel + all-reduce (one peer-memory kernel up to 256 rows; above, "
                   + ("two-phase peer-memory kernels" if big_peer is not None else "NCCL")
                   + " on a side stream beside the following shapes' GEMMs)",
                   "row_sum": args.row_sum,
                   "l2": "inputs larger than L2: shapes run M-major, 270 MB of packed weights "
                         "cycle through the 126 MB L2 between reuses",
                   "graph": "one CUDA graph per step"},
        "clocks": clocks.summary(),
        "gpu_launches": launches_per_step * args.steps,
        "device_status": status,
    }
    if parity is not None:
        line["parity_check"] = parity
    if breakdown is not None and per_shape:
        breakdown["gemm"] = round(gemm_ms, 4)
        breakdown["note"] = ("each part replayed alone (max over ranks); the step overlaps nothing "
                             "across parts, the remainder is launch gaps")
        line["step_breakdown_ms"] = breakdown
    if big_ms > 0:
        achieved = big_flops / (big_ms * 1e-3) / 1e12
        line["roofline"] = {
            "bound": "tensor", "achieved": achieved, "peak": fp8_peak, "unit": "TFLOP/s",
            "frac": achieved / fp8_peak,
            "traffic": 78.1e6,
            "traffic_launch": "M=4096 N=7168 K=5120 (algorithmic bytes of that launch 109.0e6; part "
                              "of the output is still in L2 when the kernel ends)",
            "traffic_source": "profiles/w6a8_gemm_pair_kernel_m4096_n7168_k5120.md "
                              "(dram__bytes_read.sum + dram__bytes_write.sum of one launch)",
            "kernel": "w6a8_gemm_pair_kernel (CTA pairs), M >= 4096 launches of the sweep",
            "peak_note": f"2 x bf16_tflops burst ({peaks['source']}): every shape is timed in "
                         "isolation, and kind::mxf8f6f4 runs at the FP8 rate, twice the BF16 rate "
                         "the peak file measures",
            "frac_of_2x_sustained": achieved / (2.0 * float(peaks["bf16_tflops_sustained"])),
            "frac_of_nominal_4500": achieved / 4500.0,
        }
        if small_ms > 0:
            small = small_bytes / (small_ms * 1e-3) / 1e9
            line["roofline"]["small_m"] = {
                "bound": "hbm", "achieved": small, "peak": float(peaks["hbm_gbs"]), "unit": "GB/s",
                "frac": small / float(peaks["hbm_gbs"]),
                "traffic": SMALL_M_TRAFFIC["traffic"],
                "traffic_launch": SMALL_M_TRAFFIC["launch"],
                "traffic_source": SMALL_M_TRAFFIC["source"],
                "kernel": "w6a8_stream_kernel, M <= 32 launches of the sweep (20 back-to-back "
                          "launches per shape over weight copies that exceed the L2)",
                "peak_note": f"hbm_gbs ({peaks['source']})",
                "per_m": small_per_m,
            }
    if quant is not None:
        line["quantizer"] = quant
    if per_shape:
        line["gemm_only_ms_per_step"] = gemm_ms
    if e2e is not None:
        line["e2e"] = e2e
    if moe is not None:
        line["moe_layer"] = moe
    if decoder is not None:
        line["decoder_step"] = decoder
    if not args.no_cpu_baseline and world == 1:
        base = cpu_reference_sample(os.cpu_count() or 1)
        line["cpu_baseline"] = {key: base[key] for key in ("value", "unit", "cores", "kind", "sample")}
    if per_shape:
        line["sweep"] = per_shape  # last: the longest array
    print(json.dumps(line), flush=True)
    finish(world)


def finish(world: int) -> None:
    """Leave a multi-rank run without tearing NCCL down: communicators that were
    captured into CUDA graphs can block in destroy_process_group, and every rank has
    already synchronised and reported by the time this is called."""
    if world > 1:
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
