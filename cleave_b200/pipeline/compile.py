"""``compile``: operator -> plans -> built, validated, timed candidates -> the best ``Kernel``
(the call surface of python/cleave/pipeline/compile.py:74-144)."""

from __future__ import annotations

import hashlib
import json
import os
import time

from ..codegen import B200CodeGen
from ..core.errors import CleaveError
from ..frontend import JitFunction, Program, trace
from ..runtime.validate import BenchOptions
from . import plans as _plans
from .build import BuiltKernel
from .config import DEFAULT_SPLITS, cache_root, resolve_eval
from .report import Report, Result


def _lib_digest() -> str:
    from .. import _lib

    try:
        with open(_lib.LIB_PATH, "rb") as f:
            return hashlib.sha256(f.read()).hexdigest()[:16]
    except OSError:
        return "nolib"


def _cache_dir(program: Program, cfg, splits) -> str:
    key = json.dumps({"program": program.fingerprint(), "splits": list(splits), "iters": cfg.iters,
                      "warmup": cfg.warmup, "tol": [cfg.tolerance.rtol, cfg.tolerance.atol], "lib": _lib_digest()},
                     sort_keys=True, default=str)
    return os.path.join(cache_root(), "persistent", "kernels",
                        f"{program.name}-{hashlib.sha256(key.encode()).hexdigest()[:16]}")


def build(planset, cfg, progress=None) -> Report:
    """Codegen in the parent, then validate and time every candidate."""
    from ..runtime import evaluate as _evaluate  # resolved at call time: tests monkeypatch run_candidates
    from ..runtime.validate import publish_reference

    t0 = time.perf_counter()
    plans = list(planset)
    gen = B200CodeGen()
    runs = _evaluate.run_candidates(
        plans, build_fn=lambda plan: gen.gen(plan.spec),
        # fused candidates compute the same function and share one published reference; partial and combine
        # stages compute different things and are each checked against their own spec
        reference_fn=(lambda d: publish_reference(d, plans[0].spec)[0]) if plans and all(p.role == "main" for p in plans) else None,
        pool=cfg.pool, max_parallel=cfg.max_parallel, timeout_s=cfg.timeout_s, tolerance=cfg.tolerance,
        benchmark=BenchOptions(cfg.warmup, cfg.iters), labels=[p.label for p in plans], progress=progress)
    results = [Result(p, r, BuiltKernel.from_plan(p, r.code) if r.code else None) for p, r in zip(plans, runs)]
    return Report(results, planset, {"build": time.perf_counter() - t0})


def compile(fn, shapes=None, dtype=None, *, split=None, preset="default", eval=None, cache_kernels=True,  # noqa: A001,A002
            progress=None, two_stage=False, **attrs):
    """Compile an operator for fixed shapes and return the fastest validated :class:`Kernel`; its
    ``report`` holds every candidate. ``fn`` is a ``@cleave_b200.jit`` function, a traced
    ``Program``, or the name of a paged operator (``"gqa_paged_decode"``, ``"mla_paged_decode"``; these
    go to :func:`cleave_b200.pipeline.dynamic.compile_dynamic`). ``two_stage`` also schedules the reference's
    partial + combine kernel pairs (variant ``split-k=N/two-stage``) beside the fused split kernels."""
    if isinstance(fn, str):
        from .dynamic import compile_dynamic

        return compile_dynamic(fn, dtype=dtype, preset=preset, eval=eval, **attrs)
    if attrs:
        raise TypeError(f"compile(): unexpected options {sorted(attrs)}")
    program = fn if isinstance(fn, Program) else trace(fn, shapes, dtype, split=split)
    if not isinstance(fn, (Program, JitFunction)) and not callable(fn):
        raise TypeError("compile() takes a @jit function, a Program or a paged operator name")
    cfg = resolve_eval(preset, eval)
    splits = program.split if program.split else (DEFAULT_SPLITS if split is None else ())
    if split is False:
        splits = ()
    path = _cache_dir(program, cfg, tuple(splits) + (("two-stage",) if two_stage else ()))
    if cache_kernels and os.path.isfile(os.path.join(path, "kernel.json")):
        from .kernel import load

        kernel = load(path)
        kernel.meta["cache_hit"] = True
        return kernel
    t0 = time.perf_counter()
    planset = _plans.schedule(program, splits, two_stage=two_stage)
    report = build(planset, cfg, progress)
    report.timings["schedule"] = 0.0
    report.timings["total"] = time.perf_counter() - t0
    try:
        kernel = report.best()
    except CleaveError as err:
        err.report = report
        raise
    if cache_kernels:
        kernel.save(path)
    return kernel
