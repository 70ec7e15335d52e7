"""Evaluation settings and presets (reference: python/cleave/pipeline/config.py:23-91)."""

from __future__ import annotations

import dataclasses
import os
from dataclasses import dataclass

from ..runtime.validate import DEFAULT_TOLERANCE, Tolerance


@dataclass(frozen=True)
class EvalConfig:
    warmup: int = 16
    iters: int = 1000
    tolerance: Tolerance = DEFAULT_TOLERANCE
    timeout_s: float | None = None  # per candidate, when candidates run in worker processes
    max_parallel: int = 1
    pool: str | None = None         # None = in process; "spawn" / "fork" = one worker per candidate

    def replace(self, **kw):
        return dataclasses.replace(self, **kw)


DEFAULT_SPLITS = (4, 8, 16)  # python/cleave/pipeline/compile.py:18

PRESETS = {
    "fast": EvalConfig(warmup=4, iters=100),
    "default": EvalConfig(),
    "exhaustive": EvalConfig(warmup=32, iters=4000),
}


def list_presets():
    return sorted(PRESETS)


def resolve_eval(preset="default", eval=None) -> EvalConfig:  # noqa: A002
    if eval is not None:
        return eval
    if preset not in PRESETS:
        raise ValueError(f"unknown preset {preset!r}; choose from {list_presets()}")
    cfg = PRESETS[preset]
    t = os.environ.get("CLEAVE_COMPILE_AND_RUN_TIMEOUT_SECS")
    return cfg.replace(timeout_s=float(t)) if t else cfg


def cache_root() -> str:
    return os.environ.get("CLEAVE_CACHE_ROOT") or os.path.join(os.path.expanduser("~"), ".cache", "cleave_b200")
