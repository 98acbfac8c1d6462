"""First-use tuner: switches, cache entries, and (on a GPU) one real search.

Follows the reference's contract (python/mxfp6/autotune.py:117-138 modes, :287-389 cache
entries keyed by build / GPU / shape, :772-885 install-or-tune): a decision is timed once,
validated against the default plan, installed in the override registry and read back from
its JSON file by later lookups; ``cache_only`` never times.
"""

from __future__ import annotations

import json

import pytest
import torch

import mxfp6_sm120_b200 as mx
from mxfp6_sm120_b200 import autotune as at


def test_modes_follow_the_environment(monkeypatch):
    monkeypatch.delenv("MXFP6_AUTOTUNE", raising=False)
    assert at.autotune_mode() == "off" and not mx.is_autotune_enabled()
    for raw, mode in (("1", "on"), ("on", "on"), ("cache_only", "cache_only"), ("0", "off"), ("false", "off")):
        monkeypatch.setenv("MXFP6_AUTOTUNE", raw)
        assert at.autotune_mode() == mode
    assert mx.is_autotune_cache_only() is False
    monkeypatch.setenv("MXFP6_AUTOTUNE", "cache_only")
    assert mx.is_autotune_cache_only() and mx.is_autotune_enabled()
    monkeypatch.setenv("MXFP6_AUTOTUNE_CACHE_DIR", "/tmp/somewhere")
    assert str(mx.autotune_cache_directory()) == "/tmp/somewhere"
    assert at.W6A8Config(-1).kernel == "builtin_fallback"
    assert at.W6A8Config(53).kernel == "stream_tn64_ck4_split1"


def test_cache_entries_round_trip_and_reject_foreign_descriptors(tmp_path, monkeypatch):
    monkeypatch.setenv("MXFP6_AUTOTUNE_CACHE_DIR", str(tmp_path))
    descriptor = {"schema": 1, "abi": "b200-w6a8-58-v1", "gpu": "NVIDIA B200", "m": 24, "n": 2048, "k": 1024,
                  "out_dtype": "bfloat16"}
    key = at._cache_key(descriptor)
    assert at._read_entry(key, descriptor) is None
    result = at.AutotuneResult(at.W6A8Config(10), 4.25, 5.0, 4.5, 3)
    at._write_entry(key, descriptor, result)
    assert at._read_entry(key, descriptor) == result
    assert json.loads((tmp_path / f"{key}.json").read_text())["result"]["config"]["config_id"] == 10
    assert at._read_entry(key, dict(descriptor, gpu="another")) is None      # same file, other build or GPU
    (tmp_path / f"{key}.json").write_text("{ truncated")
    assert at._read_entry(key, descriptor) is None
    assert at._cache_key(dict(descriptor, m=25)) != key


@pytest.mark.gpu
def test_search_installs_the_winner_and_the_cache_serves_it_afterwards(tmp_path, monkeypatch):
    dev = "cuda:0"
    monkeypatch.setenv("MXFP6_AUTOTUNE_CACHE_DIR", str(tmp_path))
    monkeypatch.setenv("MXFP6_AUTOTUNE_MIN_IMPROVEMENT", "0.0")
    monkeypatch.delenv("MXFP6_AUTOTUNE", raising=False)
    m, n, k = 24, 2048, 1024
    gen = torch.Generator(device="cpu").manual_seed(61)
    a = torch.randn((m, k), generator=gen).to(torch.bfloat16).to(dev)
    w = mx.quantize_mxfp6((torch.randn((n, k), generator=gen) * 0.02).to(torch.bfloat16).to(dev))
    default = mx.gemm_from_float(a, w, out_dtype=torch.bfloat16).clone()
    assert mx.autotune_w6a8(a, w, out_dtype=torch.bfloat16) is None          # tuning is off by default
    try:
        config = mx.autotune_w6a8(a, w, out_dtype=torch.bfloat16, force=True)
        assert isinstance(config, mx.W6A8Config)
        entry = at.cached_result(mx.quantize_mxfp8(a), w, out_dtype=torch.bfloat16)
        assert entry is not None and entry.config == config
        assert entry.latency_us <= entry.fallback_us and entry.latency_us <= entry.runner_up_us
        if config.config_id >= 0:
            described = mx.w6a8_configs()[config.config_id]
            plan = mx.gemm_w6a8_plan(m, n, k)
            assert plan["kernel"] == described["kernel"] and plan["tile_tokens"] == described["tile_tokens"]
        tuned = mx.gemm_from_float(a, w, out_dtype=torch.bfloat16)
        rel = float((tuned.float() - default.float()).norm() / default.float().norm())
        assert rel <= 1e-3

        # a later process in cache-only mode: installs from the file, times nothing
        at._DECISIONS.clear()
        mx.set_w6a8_config(a, m, n, k, -1, output_dtype=torch.bfloat16)
        monkeypatch.setenv("MXFP6_AUTOTUNE", "cache_only")
        monkeypatch.setattr(at, "_tune", lambda *args, **kwargs: pytest.fail("cache_only must not time"))
        assert mx.autotune_w6a8(a, w, out_dtype=torch.bfloat16) == config
        other = torch.randn((m + 1, k), generator=gen).to(torch.bfloat16).to(dev)
        assert mx.autotune_w6a8(other, w, out_dtype=torch.bfloat16) is None   # a miss stays a miss
    finally:
        mx.set_w6a8_config(a, m, n, k, -1, output_dtype=torch.bfloat16)
    assert mx.device_status() == 0
