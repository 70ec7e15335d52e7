"""Build, check and time a list of candidates, with failures classified by stage.

Mirrors ``run_candidates`` of the reference (python/cleave/runtime/evaluate.py:136-376): the
parent generates every candidate's kernel text (``build_fn``), then ``check_fn`` loads, validates
and times it - in process, or in worker processes with a per-candidate timeout, where a worker
that hangs is killed (``CandidateTimeout``) and one that dies is reported (``WorkerCrash``)
without taking the other candidates with it. ``build_fn``, ``check_fn``, ``reference_fn`` and
``pool`` are explicit injection points, as in the reference, so the orchestration is testable
without a GPU.
"""

from __future__ import annotations

import multiprocessing as mp
import os
import signal
import tempfile
import time
import traceback
from dataclasses import dataclass

from ..core.errors import (BenchmarkError, CandidateTimeout, CleaveError, CodegenError, CompileError,  # noqa: F401
                           ValidationError, WorkerCrash, for_stage)

_TRACEBACK_LINES = 20


@dataclass
class CandidateResult:
    cand: object
    status: str  # "ok" | "failed"
    stage: str | None = None  # codegen|compile|validate|bench|timeout|crash on failure
    error: CleaveError | None = None
    code: str | None = None
    cuda_src: str | None = None
    latency_ms: float | None = None
    label: str = ""

    @property
    def ok(self) -> bool:
        return self.status == "ok"


def _short_traceback(text):
    lines = text.strip().splitlines()
    if len(lines) > _TRACEBACK_LINES:
        lines = ["..."] + lines[-_TRACEBACK_LINES:]
    return "\n".join(lines)


def _typed_error(stage, label, exc_type, message, tb):
    text = "\n".join(x for x in (f"{label} failed with {exc_type}", message, _short_traceback(tb)) if x)
    cls = for_stage(stage)
    return cls(text)


def _run_check(check_fn, code, kwargs):
    """Runs in the worker (or in process): ``{"ok": True, ...}`` or a failure report."""
    try:
        src, latency_ms = check_fn(code, **kwargs)
        return {"ok": True, "cuda_src": src, "latency_ms": latency_ms}
    except BaseException as exc:  # noqa: BLE001 - everything is reported to the parent
        return {"ok": False, "stage": getattr(exc, "_cleave_stage", None) or "compile",
                "error_type": type(exc).__name__, "error_message": str(exc),
                "traceback": "".join(traceback.format_exception(exc))}


def _worker_main(conn, check_fn, code, kwargs):
    try:
        os.setsid()  # own process group: a timeout kills the worker and everything it started
    except OSError:
        pass
    conn.send(_run_check(check_fn, code, kwargs))
    conn.close()


def _kill_group(proc):
    try:
        os.killpg(proc.pid, signal.SIGKILL)
    except (ProcessLookupError, PermissionError, OSError):
        try:
            proc.kill()
        except Exception:  # noqa: BLE001
            pass


def run_candidates(cands, *, build_fn=None, check_fn=None, reference_fn=None, pool=None, max_parallel: int = 1,
                   timeout_s: float | None = None, tolerance=None, benchmark=None, labels=None,
                   progress=None) -> list:
    """One :class:`CandidateResult` per candidate, in order.

    ``build_fn(cand) -> str`` defaults to the kernel-spec code generator; ``check_fn(code, **kw) ->
    (source, latency_ms)`` defaults to :func:`cleave_b200.runtime.compile.check_code`;
    ``reference_fn(reference_cache_dir) -> out_idx`` publishes the (inputs, reference) file the
    workers read (skipped when None); ``pool`` is a multiprocessing context name
    (``"spawn"``/``"fork"``) or None for in-process execution.
    """
    from .compile import build_candidate_code, check_code

    build_fn = build_fn or build_candidate_code
    check_fn = check_fn or check_code
    labels = list(labels or [getattr(c, "label", f"candidate {i}") for i, c in enumerate(cands)])
    results = [None] * len(cands)

    # ---- codegen in the parent (plans are not picklable in the reference either)
    codes = []
    for i, cand in enumerate(cands):
        try:
            codes.append(build_fn(cand))
        except BaseException as exc:  # noqa: BLE001
            codes.append(None)
            err = _typed_error("codegen", labels[i], type(exc).__name__, str(exc),
                               "".join(traceback.format_exception(exc)))
            results[i] = CandidateResult(cand, "failed", "codegen", err, label=labels[i])

    kwargs = {}
    if tolerance is not None:
        kwargs["tolerance"] = tolerance
    if benchmark is not None:
        kwargs["benchmark"] = benchmark
    tmpdir = None
    if reference_fn is not None:
        tmpdir = tempfile.TemporaryDirectory(prefix="cleave_b200_ref_")
        out_idx = reference_fn(tmpdir.name)
        kwargs.update(reference_cache_dir=tmpdir.name, out_idx=out_idx)

    def finish(i, report):
        if report.get("ok"):
            results[i] = CandidateResult(cands[i], "ok", None, None, codes[i], report.get("cuda_src"),
                                         report.get("latency_ms"), labels[i])
        else:
            stage = report.get("stage") or "compile"
            err = _typed_error(stage, labels[i], report.get("error_type", "RuntimeError"),
                               report.get("error_message", ""), report.get("traceback", ""))
            results[i] = CandidateResult(cands[i], "failed", stage, err, codes[i], label=labels[i])
        if progress:
            progress(i, results[i])

    todo = [i for i in range(len(cands)) if results[i] is None]
    try:
        if pool is None:
            for i in todo:
                finish(i, _run_check(check_fn, codes[i], kwargs))
        else:
            ctx = mp.get_context(pool) if isinstance(pool, str) else pool
            active = {}  # index -> (process, connection, start time)
            queue = list(todo)
            while queue or active:
                while queue and len(active) < max(1, max_parallel):
                    i = queue.pop(0)
                    parent, child = ctx.Pipe(duplex=False)
                    proc = ctx.Process(target=_worker_main, args=(child, check_fn, codes[i], kwargs), daemon=True)
                    proc.start()
                    child.close()
                    active[i] = (proc, parent, time.monotonic())
                for i, (proc, conn, t0) in list(active.items()):
                    if conn.poll(0.02):
                        try:
                            report = conn.recv()
                        except EOFError:
                            report = None
                        proc.join(timeout=5)
                        del active[i]
                        if report is None:
                            err = WorkerCrash(f"{labels[i]}: the worker exited without a result "
                                              f"(exit code {proc.exitcode})")
                            results[i] = CandidateResult(cands[i], "failed", "crash", err, codes[i], label=labels[i])
                        else:
                            finish(i, report)
                    elif not proc.is_alive():
                        proc.join()
                        del active[i]
                        err = WorkerCrash(f"{labels[i]}: the worker died (exit code {proc.exitcode})")
                        results[i] = CandidateResult(cands[i], "failed", "crash", err, codes[i], label=labels[i])
                    elif timeout_s is not None and time.monotonic() - t0 > timeout_s:
                        _kill_group(proc)
                        proc.join(timeout=5)
                        del active[i]
                        err = CandidateTimeout(f"{labels[i]}: no result within {timeout_s} s; worker killed")
                        results[i] = CandidateResult(cands[i], "failed", "timeout", err, codes[i], label=labels[i])
    finally:
        if tmpdir is not None:
            tmpdir.cleanup()
    return results
