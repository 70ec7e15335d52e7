"""The compiled result of ``compile``: a callable ``Kernel`` of one stage, or of a partial stage feeding a
combine stage, that can be saved and loaded without searching again.

What is fixed by the reference's API and on-disk format (python/cleave/pipeline/kernel.py:11-203) and kept:
the class names ``Param`` / ``Stage`` / ``Kernel``, their fields, ``Kernel(*inputs)`` / ``Kernel(name=tensor)``
with ``TypeError`` for arity and ``ValueError`` for shapes, ``kernel.json`` with ``"format": 1`` beside one
``kernel*.py`` per stage, ``load``, and ``stages_for`` which turns validated plans into call stages. How the
stages are bound and run is this library's own: a stage's text is a kernel spec bound to ``libcleave_b200.so``.
"""

from __future__ import annotations

import json
import math
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any

FORMAT = 1
MANIFEST = "kernel.json"


@dataclass
class Param:
    """Where one tensor argument of a stage comes from: Program input ``index`` (``source == "input"``) or
    output ``index`` of the stage before (``source == "stage"``); ``shape`` is what the kernel expects."""

    name: str
    source: str
    index: int
    shape: tuple


@dataclass
class Stage:
    role: str  # "main" | "partial" | "combine"
    source: str = field(repr=False)
    out_idx: list
    params: list
    label: str = ""
    latency_us: float | None = None
    built: Any = field(default=None, repr=False, compare=False)

    def file_name(self, position: int, alone: bool) -> str:
        return "kernel.py" if alone else f"kernel_{position}_{self.role}.py"

    def manifest(self, file_name: str) -> dict:
        entry = {"role": self.role, "out_idx": list(self.out_idx), "params": [asdict(p) for p in self.params],
                 "label": self.label, "latency_us": self.latency_us, "file": file_name}
        if self.built is not None:
            entry["kernel"] = self.built.to_dict()
        return entry

    @classmethod
    def from_manifest(cls, entry: dict, directory: Path) -> "Stage":
        from .build import BuiltKernel

        text = (directory / entry["file"]).read_text()
        params = [Param(p["name"], p["source"], int(p["index"]), tuple(p["shape"])) for p in entry["params"]]
        built = BuiltKernel.from_dict(entry["kernel"], text) if "kernel" in entry else None
        return cls(entry["role"], text, list(entry["out_idx"]), params, entry.get("label", ""),
                   entry.get("latency_us"), built)


def _as_shape(x, shape):
    """``x`` viewed as ``shape`` when the element counts agree (unit and batch axes may be laid out
    differently between a Program tensor and a kernel buffer); otherwise ``x`` itself."""
    shape = tuple(shape)
    if tuple(x.shape) == shape or math.prod(x.shape) != math.prod(shape):
        return x
    return x.reshape(shape)


class Kernel:
    def __init__(self, stages, *, name, input_names, input_shapes, output_shapes=None, variant="solo", label="",
                 latency_us=None, report=None, plans=(), unrunnable=None, meta=None):
        self.stages = list(stages)
        self.name, self.variant, self.label, self.latency_us = name, variant, label, latency_us
        self.input_names = list(input_names)
        self.input_shapes = [tuple(s) for s in input_shapes]
        self.output_shapes = None if output_shapes is None else [tuple(s) for s in output_shapes]
        self.report, self.plans = report, list(plans)
        self.unrunnable, self.meta = unrunnable, dict(meta or {})
        self._bound = None  # one library-bound callable per stage, made on first use

    # ---- what callers read
    @property
    def source(self) -> str:
        if len(self.stages) == 1:
            return self.stages[0].source
        return "\n\n".join(f"# ---- stage {i}: {st.role} ----\n{st.source}" for i, st in enumerate(self.stages))

    @property
    def plan(self):
        return self.plans[0] if len(self.plans) == 1 else tuple(self.plans)

    @property
    def kernels(self) -> list:
        return [st.built for st in self.stages]

    def __repr__(self):
        took = "?" if self.latency_us is None else f"{self.latency_us:.2f} us"
        return f"Kernel({self.name!r}, {self.variant}, {took}, {self.label!r})"

    # ---- calling
    def _arguments(self, positional, named) -> list:
        want = self.input_names
        if positional and named:
            raise TypeError("pass inputs either positionally or by name, not both")
        if named:
            unknown = sorted(k for k in named if k not in want)
            absent = [k for k in want if k not in named]
            if unknown or absent:
                raise TypeError(f"{self.name}: missing inputs {absent}, unexpected {unknown}")
            positional = tuple(named[k] for k in want)
        if len(positional) != len(want):
            raise TypeError(f"{self.name}: expected {len(want)} inputs ({', '.join(want)}), got {len(positional)}")
        for label, shape, tensor in zip(want, self.input_shapes, positional):
            if tuple(tensor.shape) != shape:
                raise ValueError(f"{self.name}: input {label!r} has shape {tuple(tensor.shape)}, expected {shape}")
        return list(positional)

    def compile(self) -> "Kernel":
        """Bind every stage's text to the sm_100a library (nothing is searched); ``__call__`` does it lazily."""
        if self.unrunnable:
            raise NotImplementedError(self.unrunnable)
        if self._bound is None:
            from ..runtime.compile import _compile, _load_main_kernel_from_code

            self._bound = [_compile(_load_main_kernel_from_code(st.source), st.out_idx) for st in self.stages]
        return self

    def __call__(self, *args, **named):
        from ..runtime.reference import order_inputs_for_kernel

        program_inputs = self._arguments(args, named)
        self.compile()
        previous: list = []
        for stage, run in zip(self.stages, self._bound):
            pool = {"input": program_inputs, "stage": previous}
            by_name = {p.name: _as_shape(pool[p.source][p.index], p.shape) for p in stage.params}
            produced = run(*order_inputs_for_kernel(by_name, run))
            previous = list(produced) if isinstance(produced, (list, tuple)) else [produced]
        if self.output_shapes is not None:
            previous = [_as_shape(t, s) for t, s in zip(previous, self.output_shapes)]
        return previous[0] if len(previous) == 1 else tuple(previous)

    # ---- persistence
    def save(self, path) -> Path:
        directory = Path(path).expanduser()
        directory.mkdir(parents=True, exist_ok=True)
        alone = len(self.stages) == 1
        entries = []
        for i, stage in enumerate(self.stages):
            file_name = stage.file_name(i, alone)
            (directory / file_name).write_text(stage.source)
            entries.append(stage.manifest(file_name))
        manifest = {"format": FORMAT, "name": self.name, "variant": self.variant, "label": self.label,
                    "latency_us": self.latency_us, "input_names": self.input_names,
                    "input_shapes": self.input_shapes, "output_shapes": self.output_shapes,
                    "unrunnable": self.unrunnable, "stages": entries, "meta": self.meta}
        (directory / MANIFEST).write_text(json.dumps(manifest, indent=1, default=str))
        if hasattr(self.report, "to_dict"):
            (directory / "report.json").write_text(json.dumps(self.report.to_dict(), indent=1, default=str))
        return directory


def load(path) -> Kernel:
    """A saved ``Kernel`` (or ``PagedKernel``) read back; nothing is searched or rebuilt."""
    directory = Path(path).expanduser()
    manifest = json.loads((directory / MANIFEST).read_text())
    if manifest.get("format") != FORMAT:
        raise ValueError(f"{directory}: unsupported kernel format {manifest.get('format')!r}")
    if manifest.get("paged"):
        from .dynamic import PagedKernel

        return PagedKernel._load(directory, manifest)
    stages = [Stage.from_manifest(entry, directory) for entry in manifest["stages"]]
    return Kernel(stages, name=manifest["name"], input_names=manifest["input_names"],
                  input_shapes=manifest["input_shapes"], output_shapes=manifest.get("output_shapes"),
                  variant=manifest["variant"], label=manifest["label"], latency_us=manifest["latency_us"],
                  unrunnable=manifest.get("unrunnable"),
                  meta=dict(manifest.get("meta") or {}, loaded_from=str(directory)))


def stages_for(plans_and_results, program=None):
    """``(stages, problem)`` from ``[(plan, result[, BuiltKernel])]``: one solo / fused plan, or a partial plan
    followed by its combine plan (reference: python/cleave/pipeline/kernel.py:168-203). A main or partial
    stage takes the Program's inputs, bound through ``plan.inputs`` (the kernel's placeholder name for each
    Program input, in order); a combine stage takes the outputs of the stage before, in order. ``problem`` is
    a sentence when the stages cannot be chained (the kernel is then kept as a record but marked unrunnable),
    else None."""
    stages, problem = [], None
    handed_on: list = []   # shapes of the outputs of the stage before
    for plan, result, *rest in plans_and_results:
        built = rest[0] if rest else None
        spec = plan.spec
        params = []
        if plan.role == "combine":
            for position, p in enumerate(spec.inputs):
                fits = position < len(handed_on) and math.prod(handed_on[position]) == math.prod(int(d) for d in p.dims)
                if not fits:
                    problem = problem or f"{plan.label}: combine inputs do not line up with the partial kernel's outputs"
                params.append(Param(p.name, "stage", position, tuple(p.dims)))
        else:
            if plan.inputs is None:
                problem = problem or f"{plan.label}: could not bind kernel placeholders to the Program inputs"
            position_of = {placeholder: i for i, placeholder in enumerate(plan.inputs or ())}
            for p in spec.inputs:
                params.append(Param(p.name, "input", position_of.get(p.name, -1), tuple(p.dims)))
        handed_on = [tuple(int(d) for d in o.dims) for o in spec.outputs]
        took = None if result is None or result.latency_ms is None else result.latency_ms * 1e3
        text = built.source if built is not None else (result.code if result is not None else "")
        n_out = len(spec.outputs)
        stages.append(Stage(plan.role, text, list(range(-n_out, 0)), params, plan.label, took, built))
    return stages, problem
