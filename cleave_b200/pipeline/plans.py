"""Plans: one kernel candidate each (reference: python/cleave/pipeline/plans.py:17-38, 203-234).

The reference's scheduler proposes many tilings per graph, scored by a Hopper cost model; here
a plan keeps what the backend honours - the structure (solo or split, split factor) - and leaves
tile shapes to the hand-written kernels. A split variant is ONE fused kernel (role "main"); with
``two_stage`` the reference's partial + combine pair is scheduled beside it as variant
``split-k=N/two-stage`` (two launches meeting in a partial buffer: the compatibility form).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from ..codegen import make_spec, make_two_stage_specs

GEMM_FAMILIES = ("matmul", "rmsnorm_matmul", "swiglu")


@dataclass(eq=False)
class Plan:
    graph_index: int
    variant: str        # "solo" | "split-k=N"
    role: str           # "main" | "partial" | "combine"
    spec: Any           # codegen.KernelSpec
    inputs: list        # kernel placeholder names, in the Program's input order
    split_factor: int = 1
    label: str = ""
    tile: Any = None    # the reference's TileDict slot; unused (tile shapes are the kernels' own)


@dataclass
class PlanSet:
    program: Any
    plans: list = field(default_factory=list)
    refused: list = field(default_factory=list)

    def __iter__(self):
        return iter(self.plans)

    def __len__(self):
        return len(self.plans)

    def summary(self) -> str:
        return f"{len(self.plans)} plan(s): " + ", ".join(p.variant for p in self.plans)


def schedule(program, splits=None, two_stage: bool = False) -> PlanSet:
    """Solo plus one fused split plan per factor for the GEMM family (the decode families split their KV
    stream inside the kernel and have a single fused plan). ``two_stage`` adds, per factor, the partial and
    combine plans of the two-kernel form where one exists: split-K matmul, split-KV decode attention."""
    by_input = {v: k for k, v in program.bind.items()}  # Program input name -> placeholder name
    inputs = [by_input[n] for n in program.input_names]
    out = PlanSet(program)
    shape = "x".join(str(v) for v in program.dims.values())

    def add(variant, split):
        spec = make_spec(program.family, program.dtype, program.dims, split=split, attrs=program.attrs)
        out.plans.append(Plan(0, variant, "main", spec, inputs, split, f"{program.family} {variant} {shape}"))

    def add_pair(split):
        variant = f"split-k={split}/two-stage"
        try:
            partial, combine = make_two_stage_specs(program.family, program.dtype, program.dims, split, program.attrs)
        except Exception as exc:  # noqa: BLE001 - no two-stage form of this operator
            out.refused.append((variant, exc))
            return
        out.plans.append(Plan(1, variant, "partial", partial, inputs, split, f"{program.family} {variant} partial {shape}"))
        out.plans.append(Plan(1, variant, "combine", combine, None, split, f"{program.family} {variant} combine {shape}"))

    add("solo", 1)
    factors = [int(s) for s in (splits if splits is not None else program.split)]
    if program.family in GEMM_FAMILIES:
        kblocks = -(-program.dims["K"] // 64)
        for s in factors:
            if 1 < s <= kblocks:
                add(f"split-k={s}", s)
                if two_stage and program.dims["K"] % (8 * s) == 0:
                    add_pair(s)
    elif two_stage and program.family == "attention_decode":
        for s in factors:
            if s > 1 and program.dims["SKV"] % s == 0:
                add_pair(s)
    return out
