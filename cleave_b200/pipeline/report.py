"""Per-candidate results, failure histograms, the split-K pairing rule and ``best()``
(reference: python/cleave/pipeline/report.py)."""

from __future__ import annotations

from collections import Counter
from dataclasses import dataclass, field
from typing import Any, Sequence

from ..core.errors import CleaveError


@dataclass(eq=False)
class Result:
    plan: Any
    run: Any      # runtime.evaluate.CandidateResult
    kernel: Any = None  # pipeline.build.BuiltKernel

    ok = property(lambda self: self.run.ok)
    latency_ms = property(lambda self: self.run.latency_ms)
    latency_us = property(lambda self: None if self.run.latency_ms is None else self.run.latency_ms * 1e3)
    error = property(lambda self: self.run.error)
    stage = property(lambda self: self.run.stage)
    variant = property(lambda self: self.plan.variant)
    role = property(lambda self: self.plan.role)
    label = property(lambda self: self.plan.label)
    cuda_src = property(lambda self: self.run.cuda_src)

    @property
    def error_type(self):
        if self.ok:
            return None
        return type(self.run.error).__name__ if self.run.error is not None else str(self.run.stage)

    @property
    def source(self):
        return self.kernel.source if self.kernel is not None else self.run.code

    def __repr__(self):
        state = f"{self.latency_us:.2f} us" if self.latency_us is not None else (
            "ok" if self.ok else f"{self.error_type} at {self.stage}")
        return f"Result({self.label}: {state})"


class Failures(list):
    def histogram(self) -> dict:
        return dict(Counter(r.error_type for r in self).most_common())

    def by_stage(self) -> dict:
        return dict(Counter(r.stage for r in self).most_common())

    def __str__(self):
        return ", ".join(f"{n}x {k}" for k, n in self.histogram().items()) or "none"


@dataclass
class VariantResult:
    variant: str
    latency_us: float
    members: list = field(default_factory=list)  # [main] or [partial, combine]


class Report(Sequence):
    def __init__(self, results, plans=None, timings=None):
        self.results, self.plans = list(results), plans
        self.timings = dict(timings or {})
        self._best = None

    def __len__(self):
        return len(self.results)

    def __getitem__(self, i):
        return self.results[i]

    @property
    def correct(self):
        return [r for r in self.results if r.ok]

    @property
    def failures(self) -> Failures:
        return Failures(r for r in self.results if not r.ok)

    def histogram(self) -> dict:
        return self.failures.histogram()

    @property
    def program(self):
        return None if self.plans is None else self.plans.program

    @property
    def timed(self):
        return [r for r in self.results if r.ok and r.latency_ms is not None]

    def variants(self) -> dict:
        """Best latency per variant: solo = best main; split-k=N = best main (the fused kernel, one launch);
        split-k=N/two-stage = best partial + best combine (the reference's pairing rule,
        python/cleave/pipeline/report.py:123-136)."""
        best = {}
        for r in self.timed:
            key = (r.variant, r.role)
            if key not in best or r.latency_ms < best[key].latency_ms:
                best[key] = r
        out = {}
        for variant in dict.fromkeys(v for v, _ in best):
            roles = ("main",) if (variant, "main") in best else ("partial", "combine")
            if all((variant, role) in best for role in roles):
                members = [best[(variant, role)] for role in roles]
                out[variant] = VariantResult(variant, sum(m.latency_us for m in members), members)
        return out

    def best(self, variant=None):
        """The fastest Kernel overall, or of one ``variant`` (``"solo"``, ``"split-k=8"``)."""
        if variant is not None or self._best is None:
            variants = self.variants()
            if variant is not None:
                variants = {k: v for k, v in variants.items() if k == variant}
            if not variants:
                raise CleaveError(f"no {variant or 'kernel'} compiled, validated and timed "
                                  f"({len(self)} candidates; failures: {self.failures})")
            win = min(variants.values(), key=lambda v: v.latency_us)
            kernel = _make_kernel(win, self)
            if variant is not None:
                return kernel
            self._best = kernel
        return self._best

    def summary(self) -> str:
        rows = [f"candidates   {len(self)} built, {len(self.correct)} correct, {len(self.timed)} timed"]
        rows += [f"  {n}x {k}" for k, n in self.histogram().items()]
        for v in sorted(self.variants().values(), key=lambda v: v.latency_us):
            rows.append(f"  {v.variant:<12}{v.latency_us:10.2f} us  " + " + ".join(m.label for m in v.members))
        rows += [f"{k:<13}{t:.2f} s" for k, t in self.timings.items()]
        return "\n".join(rows)

    def table(self, top: int = 10, by=None) -> str:
        rows = sorted(self.timed, key=lambda r: r.latency_ms)[:top]
        return "\n".join(f"{r.latency_us:10.2f} us  {r.variant:<12}{r.label}" for r in rows)

    def to_dict(self) -> dict:
        return {"candidates": len(self), "correct": len(self.correct), "failures": self.histogram(),
                "timings_s": self.timings,
                "variants": {v.variant: v.latency_us for v in self.variants().values()},
                "latency_us": {r.label: r.latency_us for r in self.timed}}

    def __str__(self):
        return self.summary()


def _make_kernel(win: VariantResult, report: Report):
    from .kernel import Kernel, stages_for

    program = report.program
    stages, problem = stages_for([(r.plan, r.run, r.kernel) for r in win.members], program)
    return Kernel(stages, name=program.name, input_names=program.input_names, input_shapes=program.input_shapes,
                  output_shapes=program.output_shapes, variant=win.variant,
                  label=" + ".join(m.label for m in win.members), latency_us=win.latency_us, report=report,
                  plans=[m.plan for m in win.members], unrunnable=problem)
