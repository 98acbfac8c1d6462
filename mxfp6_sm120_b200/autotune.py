"""First-use tuning of the dense W6A8 GEMM over the library's explicit configurations.

Mirrors the surface of the reference's ``mxfp6.autotune`` (python/mxfp6/autotune.py:
``W6A8Config`` :78-92, ``AutotuneResult`` :95-101, the ``MXFP6_AUTOTUNE*`` switches :110-202,
``ensure_w6a8_tuned`` :772-885, the per-key JSON cache :287-389): for one problem
``(device, M, N, K, output dtype)`` every configuration of ``w6a8_configs()`` that accepts the
problem is timed inside a CUDA graph, the fastest one is checked against the default plan's
output, installed in the library's override registry (``set_w6a8_config``) and written to a
cache file, so later processes install it without timing anything.

Differences from the reference, on purpose.  The default plan here is a table measured on
the B200 for the shapes the benchmark names, so tuning is OFF unless ``MXFP6_AUTOTUNE`` asks
for it (``on`` / ``1``, or ``cache_only`` to install cached winners but never time); the
explicit call ``autotune_w6a8(..., force=True)`` tunes in any mode but ``cache_only``.  The
candidates are this library's 58 configurations, not 30 CUTLASS kernels; ``swizzle`` and
``raster_order`` have no effect on them and are recorded as 1 and 0.
"""

from __future__ import annotations

import fcntl
import hashlib
import json
import os
import statistics
import tempfile
import threading
from contextlib import contextmanager
from dataclasses import asdict, dataclass
from pathlib import Path

import torch

AUTOTUNE_SCHEMA = 1
FALLBACK_CONFIG_ID = -1
TIMING_POLICY = "cuda-graph-events-median-v1"
DEFAULT_AUTOTUNE_WARMUP = 3
DEFAULT_AUTOTUNE_ITERATIONS = 10
DEFAULT_AUTOTUNE_REPEATS = 3
DEFAULT_MIN_IMPROVEMENT = 0.03
VALIDATION_REL_FRO = 1.0e-3


@dataclass(frozen=True)
class W6A8Config:
    """One explicit configuration; ``config_id`` -1 means "keep the default plan"."""

    config_id: int
    swizzle: int = 1
    raster_order: int = 0

    @property
    def kernel(self) -> str:
        if self.config_id == FALLBACK_CONFIG_ID:
            return "builtin_fallback"
        from .ops import w6a8_configs

        c = w6a8_configs()[self.config_id]
        return f"{c['kernel']}_tn{c['tile_tokens']}_ck{c['cluster_k']}_split{c['splits']}"


@dataclass(frozen=True)
class AutotuneResult:
    config: W6A8Config
    latency_us: float
    fallback_us: float
    runner_up_us: float
    samples: int


_STATE_LOCK = threading.Lock()
_DECISIONS: dict[tuple, W6A8Config] = {}


def _env_bool(name: str, default: bool) -> bool:
    raw = os.environ.get(name)
    if raw is None:
        return default
    return raw.strip().lower() not in ("", "0", "false", "no", "off")


def _env_int(name: str, default: int, minimum: int) -> int:
    try:
        return max(minimum, int(os.environ.get(name, default)))
    except ValueError:
        return default


def autotune_mode() -> str:
    """``off`` (default), ``on`` or ``cache_only``, from ``MXFP6_AUTOTUNE``."""
    raw = os.environ.get("MXFP6_AUTOTUNE")
    if raw is None:
        return "off"
    value = raw.strip().lower()
    if value == "cache_only":
        return "cache_only"
    return "off" if value in ("", "0", "false", "no", "off") else "on"


def is_autotune_enabled() -> bool:
    return autotune_mode() != "off"


def is_autotune_cache_only() -> bool:
    return autotune_mode() == "cache_only"


def should_tune_exact_shapes() -> bool:
    """Whether shapes of the measured table are retuned too (``MXFP6_AUTOTUNE_EXACT``)."""
    return _env_bool("MXFP6_AUTOTUNE_EXACT", False)


def _verbose(message: str) -> None:
    if _env_bool("MXFP6_AUTOTUNE_VERBOSE", False):
        print(f"[mxfp6 autotune] {message}", flush=True)


def cache_directory() -> Path:
    root = os.environ.get("MXFP6_AUTOTUNE_CACHE_DIR")
    return Path(root) if root else Path.home() / ".cache" / "mxfp6_b200" / "autotune"


def w6a8_config_abi() -> str:
    from .ops import w6a8_config_abi as abi

    return abi()


def can_autotune_now() -> bool:
    """Timing needs to launch and synchronise: not while a stream is capturing."""
    return torch.cuda.is_available() and not torch.cuda.is_current_stream_capturing()


def _library_fingerprint() -> str:
    from ._loader import load_library

    path = Path(load_library())
    stat = path.stat()
    return f"{path.name}:{stat.st_size}:{int(stat.st_mtime)}"


def _descriptor(device: torch.device, m: int, n: int, k: int, out_dtype: torch.dtype) -> dict:
    props = torch.cuda.get_device_properties(device)
    return {
        "schema": AUTOTUNE_SCHEMA,
        "abi": w6a8_config_abi(),
        "timing": TIMING_POLICY,
        "library": _library_fingerprint(),
        "gpu": props.name,
        "sms": props.multi_processor_count,
        "m": int(m), "n": int(n), "k": int(k),
        "out_dtype": str(out_dtype).replace("torch.", ""),
    }


def _cache_key(descriptor: dict) -> str:
    return hashlib.sha256(json.dumps(descriptor, sort_keys=True).encode()).hexdigest()[:32]


def _entry_path(key: str) -> Path:
    return cache_directory() / f"{key}.json"


@contextmanager
def _file_lock(key: str):
    directory = cache_directory()
    directory.mkdir(parents=True, exist_ok=True)
    with open(directory / f"{key}.lock", "w") as handle:
        fcntl.flock(handle, fcntl.LOCK_EX)
        try:
            yield
        finally:
            fcntl.flock(handle, fcntl.LOCK_UN)


def _read_entry(key: str, descriptor: dict) -> AutotuneResult | None:
    try:
        data = json.loads(_entry_path(key).read_text())
        if data["descriptor"] != descriptor:
            return None
        result = data["result"]
        return AutotuneResult(W6A8Config(**result["config"]), float(result["latency_us"]),
                              float(result["fallback_us"]), float(result["runner_up_us"]),
                              int(result["samples"]))
    except (OSError, KeyError, TypeError, ValueError):
        return None


def _write_entry(key: str, descriptor: dict, result: AutotuneResult) -> None:
    directory = cache_directory()
    directory.mkdir(parents=True, exist_ok=True)
    payload = json.dumps({"descriptor": descriptor, "result": asdict(result)}, indent=1, sort_keys=True)
    with tempfile.NamedTemporaryFile("w", dir=directory, suffix=".tmp", delete=False) as handle:
        handle.write(payload)
        name = handle.name
    os.replace(name, _entry_path(key))


def _measure(run, warmup: int, iterations: int, repeats: int, flush) -> float:
    """Median over ``repeats`` of the mean latency of ``iterations`` captured launches, in us."""
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for _ in range(warmup):
            run()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for _ in range(iterations):
                run()
        graph.replay()
        samples = []
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(repeats):
            if flush is not None:
                flush.fill_(1)
            start.record(stream)
            graph.replay()
            stop.record(stream)
            stream.synchronize()
            samples.append(start.elapsed_time(stop) * 1e3 / iterations)
    return statistics.median(samples)


def _tune(a, b, out_dtype: torch.dtype) -> AutotuneResult:
    from . import ops

    warmup = _env_int("MXFP6_AUTOTUNE_WARMUP", DEFAULT_AUTOTUNE_WARMUP, 1)
    iterations = _env_int("MXFP6_AUTOTUNE_ITERATIONS", DEFAULT_AUTOTUNE_ITERATIONS, 1)
    repeats = _env_int("MXFP6_AUTOTUNE_REPEATS", DEFAULT_AUTOTUNE_REPEATS, 1)
    flush_mb = _env_int("MXFP6_AUTOTUNE_FLUSH_L2_MB", 0, 0)
    try:
        min_gain = float(os.environ.get("MXFP6_AUTOTUNE_MIN_IMPROVEMENT", DEFAULT_MIN_IMPROVEMENT))
    except ValueError:
        min_gain = DEFAULT_MIN_IMPROVEMENT
    flush = torch.empty(flush_mb << 20, dtype=torch.uint8, device=a.device) if flush_mb else None
    out = torch.empty((a.rows, b.rows), dtype=out_dtype, device=a.device)

    # the default plan without any override in the way
    ops.set_w6a8_config(a.values, a.rows, b.rows, a.k, FALLBACK_CONFIG_ID, output_dtype=out_dtype)
    reference = ops.gemm_w6a8(a, b, out_dtype=out_dtype).clone()
    fallback_us = _measure(lambda: ops.gemm_w6a8(a, b, out_dtype=out_dtype, out=out), warmup, iterations,
                           repeats, flush)
    timed: list[tuple[float, int]] = []
    for config in ops.w6a8_configs():
        config_id = int(config["config_id"])
        if int(config["splits"]) > 1:
            continue  # scratch-based splits need caller-owned scratch; clusters cover split-K
        try:
            got = ops.gemm_w6a8_config(a, b, out_dtype=out_dtype, config_id=config_id, out=out)
        except (ValueError, RuntimeError):
            continue  # the configuration does not take this problem
        rel = float((got.float() - reference.float()).norm() / reference.float().norm().clamp_min(1e-30))
        if not rel <= VALIDATION_REL_FRO:
            _verbose(f"config {config_id} rejected: rel-Frobenius {rel:.2e}")
            continue
        latency = _measure(lambda: ops.gemm_w6a8_config(a, b, out_dtype=out_dtype, config_id=config_id, out=out),
                           warmup, iterations, repeats, flush)
        timed.append((latency, config_id))
        _verbose(f"config {config_id}: {latency:.2f} us")
    timed.sort()
    if not timed or timed[0][0] > fallback_us * (1.0 - min_gain):
        best = (fallback_us, FALLBACK_CONFIG_ID)
        runner_up = timed[0][0] if timed else fallback_us
    else:
        best = timed[0]
        runner_up = timed[1][0] if len(timed) > 1 else fallback_us
    return AutotuneResult(W6A8Config(best[1]), round(best[0], 3), round(fallback_us, 3), round(runner_up, 3),
                          repeats)


def _install(a, b, out_dtype: torch.dtype, config: W6A8Config) -> None:
    from . import ops

    ops.set_w6a8_config(a.values, a.rows, b.rows, a.k, config.config_id, config.swizzle,
                        config.raster_order, out_dtype)


def ensure_w6a8_tuned(a, b, *, out_dtype: torch.dtype = torch.float16, force: bool = False) -> W6A8Config | None:
    """Install the cached winner for ``(a.rows, b.rows, a.k, out_dtype)``, tuning once on a miss.

    ``a`` is an ``MXFP8Tensor``, ``b`` a ``PackedMXFP6Tensor``.  Returns ``None`` when tuning
    is off (and not forced), while a stream is capturing, or on a miss in ``cache_only`` mode;
    a decision to keep the default plan is a config with id -1 and is cached like any other.
    """
    if not force and not is_autotune_enabled():
        return None
    if not can_autotune_now():
        return None
    device = a.values.device
    process_key = (device.index, a.rows, b.rows, a.k, out_dtype)
    with _STATE_LOCK:
        known = _DECISIONS.get(process_key)
    if known is not None and not force:
        return known
    descriptor = _descriptor(device, a.rows, b.rows, a.k, out_dtype)
    key = _cache_key(descriptor)
    with torch.cuda.device(device), _file_lock(key):
        result = None if (force and not is_autotune_cache_only()) else _read_entry(key, descriptor)
        if result is None:
            if is_autotune_cache_only():
                return None
            result = _tune(a, b, out_dtype)
            _write_entry(key, descriptor, result)
            _verbose(f"{descriptor['m']}x{descriptor['n']}x{descriptor['k']}: {result.config.kernel} "
                     f"{result.latency_us} us (default {result.fallback_us} us)")
        _install(a, b, out_dtype, result.config)
    with _STATE_LOCK:
        _DECISIONS[process_key] = result.config
    return result.config


def cached_result(a, b, *, out_dtype: torch.dtype = torch.float16) -> AutotuneResult | None:
    """The cache entry of a problem, if there is one (nothing is timed or installed)."""
    descriptor = _descriptor(a.values.device, a.rows, b.rows, a.k, out_dtype)
    return _read_entry(_cache_key(descriptor), descriptor)
