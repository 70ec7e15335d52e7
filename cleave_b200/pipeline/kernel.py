"""The compiled result: a callable ``Kernel`` (reference: python/cleave/pipeline/kernel.py)."""

from __future__ import annotations

import json
import math
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any

FORMAT = 1


@dataclass
class Param:
    """One kernel input: placeholder ``name`` fed from Program input / previous-stage output ``index``."""

    name: str
    source: str  # "input" | "stage"
    index: int
    shape: tuple


@dataclass
class Stage:
    role: str  # "main" (a fused split-K kernel is one "main" stage)
    source: str = field(repr=False)
    out_idx: list
    params: list
    label: str = ""
    latency_us: float | None = None
    built: Any = field(default=None, repr=False, compare=False)


class Kernel:
    def __init__(self, stages, *, name, input_names, input_shapes, output_shapes=None, variant="solo", label="",
                 latency_us=None, report=None, plans=(), unrunnable=None, meta=None):
        self.stages, self.name, self.variant, self.label = stages, name, variant, label
        self.input_names, self.input_shapes = list(input_names), [tuple(s) for s in input_shapes]
        self.output_shapes = None if output_shapes is None else [tuple(s) for s in output_shapes]
        self.latency_us, self.report, self.plans = latency_us, report, list(plans)
        self.unrunnable, self.meta = unrunnable, dict(meta or {})
        self._compiled = None

    @property
    def source(self) -> str:
        if len(self.stages) == 1:
            return self.stages[0].source
        return "\n\n".join(f"# ---- stage {i}: {s.role} ----\n{s.source}" for i, s in enumerate(self.stages))

    @property
    def plan(self):
        return self.plans[0] if len(self.plans) == 1 else tuple(self.plans)

    @property
    def kernels(self) -> list:
        return [s.built for s in self.stages]

    def __repr__(self):
        lat = "?" if self.latency_us is None else f"{self.latency_us:.2f} us"
        return f"Kernel({self.name!r}, {self.variant}, {lat}, {self.label!r})"

    def _bind(self, args, named) -> list:
        if args and named:
            raise TypeError("pass inputs either positionally or by name, not both")
        if named:
            missing = [n for n in self.input_names if n not in named]
            extra = sorted(set(named) - set(self.input_names))
            if missing or extra:
                raise TypeError(f"{self.name}: missing inputs {missing}, unexpected {extra}")
            args = [named[n] for n in self.input_names]
        if len(args) != len(self.input_names):
            raise TypeError(f"{self.name}: expected {len(self.input_names)} inputs "
                            f"({', '.join(self.input_names)}), got {len(args)}")
        for n, s, x in zip(self.input_names, self.input_shapes, args):
            if tuple(x.shape) != s:
                raise ValueError(f"{self.name}: input {n!r} has shape {tuple(x.shape)}, expected {s}")
        return list(args)

    def compile(self) -> "Kernel":
        """Bind the stage sources to the sm_100a library (no search); done lazily by ``__call__``."""
        if self.unrunnable:
            raise NotImplementedError(self.unrunnable)
        if self._compiled is None:
            from ..runtime.compile import _compile, _load_main_kernel_from_code

            self._compiled = [_compile(_load_main_kernel_from_code(s.source), s.out_idx) for s in self.stages]
        return self

    def __call__(self, *args, **named):
        from ..runtime.reference import order_inputs_for_kernel

        inputs = self._bind(args, named)
        self.compile()
        outs: list = []
        for stage, kernel in zip(self.stages, self._compiled):
            feed = {}
            for p in stage.params:
                x = inputs[p.index] if p.source == "input" else outs[p.index]
                feed[p.name] = _fit(x, p.shape)
            res = kernel(*order_inputs_for_kernel(feed, kernel))
            outs = list(res) if isinstance(res, (list, tuple)) else [res]
        if self.output_shapes is not None:
            outs = [_fit(o, s) for o, s in zip(outs, self.output_shapes)]
        return outs[0] if len(outs) == 1 else tuple(outs)

    def save(self, path) -> Path:
        p = Path(path).expanduser()
        p.mkdir(parents=True, exist_ok=True)
        stages = []
        for i, s in enumerate(self.stages):
            fname = f"kernel_{i}_{s.role}.py" if len(self.stages) > 1 else "kernel.py"
            (p / fname).write_text(s.source)
            d = {"role": s.role, "out_idx": s.out_idx, "params": [asdict(q) for q in s.params],
                 "label": s.label, "latency_us": s.latency_us, "file": fname}
            if s.built is not None:
                d["kernel"] = s.built.to_dict()
            stages.append(d)
        meta = {"format": FORMAT, "name": self.name, "variant": self.variant, "label": self.label,
                "latency_us": self.latency_us, "input_names": self.input_names,
                "input_shapes": self.input_shapes, "output_shapes": self.output_shapes,
                "unrunnable": self.unrunnable, "stages": stages, "meta": self.meta}
        (p / "kernel.json").write_text(json.dumps(meta, indent=1, default=str))
        if self.report is not None and hasattr(self.report, "to_dict"):
            (p / "report.json").write_text(json.dumps(self.report.to_dict(), indent=1, default=str))
        return p


def load(path) -> Kernel:
    """Read a saved Kernel back; nothing is searched or rebuilt."""
    p = Path(path).expanduser()
    m = json.loads((p / "kernel.json").read_text())
    if m.get("format") != FORMAT:
        raise ValueError(f"{p}: unsupported kernel format {m.get('format')!r}")
    if m.get("paged"):
        from .dynamic import PagedKernel

        return PagedKernel._load(p, m)
    from .build import BuiltKernel

    stages = []
    for d in m["stages"]:
        params = [Param(q["name"], q["source"], q["index"], tuple(q["shape"])) for q in d["params"]]
        source = (p / d["file"]).read_text()
        built = None if "kernel" not in d else BuiltKernel.from_dict(d["kernel"], source)
        stages.append(Stage(d["role"], source, list(d["out_idx"]), params, d.get("label", ""), d.get("latency_us"), built))
    return Kernel(stages, name=m["name"], input_names=m["input_names"], input_shapes=m["input_shapes"],
                  output_shapes=m.get("output_shapes"), variant=m["variant"], label=m["label"],
                  latency_us=m["latency_us"], unrunnable=m.get("unrunnable"),
                  meta=dict(m.get("meta") or {}, loaded_from=str(p)))


def _fit(x, shape):
    shape = tuple(shape)
    if tuple(x.shape) == shape or math.prod(x.shape) != math.prod(shape):
        return x
    return x.reshape(shape)
