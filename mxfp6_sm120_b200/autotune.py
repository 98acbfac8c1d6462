"""Configuration surface kept for callers of the reference's ``mxfp6.autotune``.

The reference times 30 ahead-of-time CUTLASS candidates per shape on first use and
caches the winner (python/mxfp6/autotune.py:552-885).  This library has one kernel
family whose tile and split-K choice is a static function of (M, N, K), so there is
nothing to search: the switches below exist so that code written against the
reference keeps importing and behaves as "autotuning off".
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from pathlib import Path

from .ops import gemm_w6a8_plan, is_stream_k_enabled  # noqa: F401  (re-exported)

CANDIDATE_ABI = "b200-tcgen05-static-table-v1"


@dataclass(frozen=True)
class W6A8Config:
    """One explicit launch configuration of the tcgen05 GEMM."""

    tile_tokens: int = 0   # activation rows per tile (MMA N); 0 = library's choice
    splits: int = 0        # scratch-arena split-K factor; 0 = library's choice

    @property
    def kernel(self) -> str:
        return f"w6a8_tcgen05_tn{self.tile_tokens or 'auto'}_split{self.splits or 'auto'}"


def is_autotune_enabled() -> bool:
    """Always False: the tile/split-K table is static."""
    return False


def is_autotune_cache_only() -> bool:
    return False


def cache_directory() -> Path:
    """Directory the reference would cache decisions in (unused here)."""
    root = os.environ.get("MXFP6_AUTOTUNE_CACHE_DIR")
    return Path(root) if root else Path.home() / ".cache" / "mxfp6"


def w6a8_config_abi() -> str:
    return CANDIDATE_ABI


def config_for(m: int, n: int, k: int) -> W6A8Config:
    """The configuration the static table picks for a dense problem."""
    plan = gemm_w6a8_plan(m, n, k)
    return W6A8Config(plan["tile_tokens"], plan["splits"])
