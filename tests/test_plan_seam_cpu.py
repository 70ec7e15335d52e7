"""The plan -> kernel-text seam on REAL plans of the reference.

``tests/golden/plans.json`` holds structural records of the plans the reference's own search and scheduler
produce for the benchmark configurations and the demo operators (``tests/golden/make_plans.py``; every plan,
deduplicated by structure: the search emits the same operator re-associated and transposed in several ways).
Every one of them must yield the kernel the repo's own ``trace`` yields for the same program - same family,
extents, eps, score scale and split factor, each input bound to the placeholder that plays its part - and
equal plans must give byte-equal text (the reference deduplicates and hashes generated source,
python/cleave/pipeline/dynamic.py:59-63). Where a reference checkout is present the same check runs live on
every plan of a fresh search.
"""

import os

import pytest

import plans as plan_fixtures
import reference_env
from cleave_b200 import lang as cl
from cleave_b200.codegen import B200CodeGen, recognise
from cleave_b200.frontend import Program, jit, trace
from cleave_b200.pipeline.build import pass_configs_of
from cleave_b200.runtime.compile import _load_main_kernel_from_code

DATA = plan_fixtures.load()


# ---- the same programs, traced by this repo's front door ------------------------------------------------
def _attention(q, k, v):
    n = q.shape[-1] ** 0.5
    return cl.softmax((q @ k.mT) / n, dim=-1, shift=-50 / n) @ v


@jit
def matmul(x: cl.Tensor["M", "K"], w: cl.Tensor["K", "N"]):
    return x @ w


@jit
def rmsnorm_matmul(x: cl.Tensor["M", "K"], w: cl.Tensor["K", "N"]):
    return cl.rms_norm(x, dim=-1, eps=1e-6) @ w


@jit
def swiglu(x: cl.Tensor["M", "K"], w0: cl.Tensor["K", "N"], w1: cl.Tensor["K", "N"]):
    gate, up = x @ w0, x @ w1
    return cl.silu(gate) * up


@jit
def gqa_decode(q: cl.Tensor["HQ", "SQ", "D"], k: cl.Tensor["HKV", "SKV", "D"], v: cl.Tensor["HKV", "SKV", "D"]):
    return _attention(q, k, v)


@jit
def mla_decode(q: cl.Tensor["B", "H", "D"], kv: cl.Tensor["B", "SKV", "D"], q_pe: cl.Tensor["B", "H", "PE"],
               k_pe: cl.Tensor["B", "SKV", "PE"]):
    n = 192 ** 0.5
    s = (q @ kv.mT + q_pe @ k_pe.mT) / n
    return cl.softmax(s, dim=-1, shift=-50 / n) @ kv


@jit
def matmul_matmul(q: cl.Tensor["BH", "SQ", "D"], k: cl.Tensor["BH", "SKV", "D"], v: cl.Tensor["BH", "SKV", "D"]):
    return (q @ k.mT) @ v


@jit
def matmul_rowsum(x: cl.Tensor["M", "K"], w: cl.Tensor["K", "N"]):
    return (x @ w).sum(-1, keepdim=True)


@jit
def mha_decode_exact(q: cl.Tensor["H", "SQ", "D"], k: cl.Tensor["H", "SKV", "D"], v: cl.Tensor["H", "SKV", "D"]):
    return cl.softmax((q @ k.mT) / q.shape[-1] ** 0.5, dim=-1) @ v


def _lora():
    p = Program("lora", dtype=cl.f16)
    M, K, N, R = p.dims(M=16, K=4096, N=4096, R=16)
    x, w = p.input("x", (M, K)), p.input("w", (K, N))
    a, b = p.input("a", (K, R)), p.input("b", (R, N))
    p.output(x @ w + (x @ a) @ b, name="y")
    return p


TRACED = {
    "cfg1_matmul": lambda: trace(matmul, dict(M=128, N=128, K=4096), cl.f16),
    "cfg2_rmsnorm_matmul_eps": lambda: trace(rmsnorm_matmul, dict(M=64, N=11008, K=4096), cl.f16),
    "swiglu": lambda: trace(swiglu, dict(M=64, N=11008, K=4096), cl.f16),
    "cfg3_gqa_decode": lambda: trace(gqa_decode, dict(HQ=256, HKV=64, SQ=1, SKV=8192, D=128), cl.f16),
    "cfg4_mla_decode": lambda: trace(mla_decode, dict(B=16, H=128, SKV=4096, D=512, PE=64), cl.bf16),
    "demo_matmul_matmul": lambda: trace(matmul_matmul, dict(BH=32, SQ=4096, SKV=4096, D=64), cl.f16),
    "demo_matmul_rowsum": lambda: trace(matmul_rowsum, dict(M=4096, N=4096, K=64), cl.f16),
    "demo_mha_decode_exact": lambda: trace(mha_decode_exact, dict(H=32, SQ=64, SKV=256, D=64), cl.f16),
    "demo_lora": _lora,
}


def _check_plan(plan, program, program_inputs):
    """One real plan against the traced program."""
    spec = recognise(plan)
    if plan.role == "combine":
        assert spec.family == "split_combine" and spec.role == "combine" and spec.split == plan.split_factor
        return spec
    assert spec.family == program.family, (plan.label, spec.family)
    assert spec.dims == program.dims and spec.dtype == program.dtype
    assert spec.split == (plan.split_factor or 1)
    assert spec.role == ("main" if plan.role == "main" else "partial")
    for key in ("eps", "scale"):
        if key in program.attrs or key in spec.attrs:
            want = program.attrs.get(key, spec.dims.get("D", 1) ** -0.5 if key == "scale" else 0.0)
            assert spec.attrs[key] == pytest.approx(want, rel=1e-5, abs=1e-9), (plan.label, key)
    # every part is played by a placeholder of the right shape; where the plan binds its placeholders to the
    # Program's arguments, the part has the argument's name
    bind = spec.attrs["bind"]
    shapes = {p.name: tuple(p.dims) for p in spec.inputs}
    by_name = dict(program_inputs)
    assert sorted(bind) == sorted(by_name)
    # the reference binds placeholders to arguments by position when shapes repeat (q, k and v of one shape:
    # python/cleave/pipeline/plans.py:116-136), which says nothing about the part a placeholder plays
    unique_shapes = len({s for _, s in program_inputs}) == len(program_inputs)
    for part, placeholder in bind.items():
        assert shapes[placeholder] == by_name[part], (plan.label, part)
        if plan.inputs is not None and unique_shapes:
            assert program_inputs[plan.inputs.index(placeholder)][0] == part
    assert spec.input_roles() == [{v: k for k, v in bind.items()}[p.name] for p in spec.inputs]
    return spec


@pytest.mark.parametrize("case", sorted(DATA))
def test_every_recorded_plan_gives_the_traced_kernel(case):
    c = DATA[case]
    program = TRACED[case]()
    assert [tuple(s) for s in program.input_shapes] == [s for _, s in c["program_inputs"]]
    gen = B200CodeGen()
    covered = 0
    for plan in c["plans"]:
        spec = _check_plan(plan, program, c["program_inputs"])
        text = gen.gen(plan)
        assert "main_kernel" in text and pass_configs_of(text) == {}
        assert _load_main_kernel_from_code(text) == spec
        assert gen.gen(plan) == text == B200CodeGen(apply_rasterization=16).gen(plan_fixtures.plan_from_record(
            {"variant": plan.variant, "role": plan.role, "split_factor": plan.split_factor, "inputs": plan.inputs,
             "nodes": _records(case)[c["plans"].index(plan)]["nodes"]}))      # an equal plan, built afresh
        covered += plan.count
    assert covered == c["n_plans"]


def _records(case):
    import json

    with open(plan_fixtures.PATH) as f:
        return json.load(f)[case]["records"]


def test_a_partial_combine_pair_becomes_one_fused_kernel():
    c = DATA["cfg1_matmul"]
    for s in (4, 8, 16):
        partial = next(p for p in c["plans"] if p.role == "partial" and p.split_factor == s)
        combine = next(p for p in c["plans"] if p.role == "combine" and p.split_factor == s)
        fused = recognise([partial, combine])
        assert (fused.family, fused.role, fused.split) == ("matmul", "main", s)
        assert [tuple(p.dims) for p in fused.outputs] == [(128, 128)]
        lone = recognise(partial)
        assert lone.role == "partial" and [tuple(p.dims) for p in lone.outputs] == [(s, 128, 128)]
        comb = recognise(combine)
        assert [tuple(p.dims) for p in comb.inputs] == [(s, 128, 128)] and comb.attrs == {"axes": [0], "divide": False}


def test_attention_split_pairs_keep_both_partial_outputs():
    c = DATA.get("cfg3_gqa_decode")
    if c is None:
        pytest.skip("no cfg3 records")
    partial = next(p for p in c["plans"] if p.role == "partial" and p.split_factor == 8)
    combine = next(p for p in c["plans"] if p.role == "combine" and p.split_factor == 8)
    lone = recognise(partial)
    assert lone.family == "attention_decode" and len(lone.outputs) == 2
    assert sorted(tuple(d for d in p.dims if d != 1) for p in lone.outputs) == [(256, 8), (256, 8, 128)]
    comb = recognise(combine)
    assert comb.attrs["divide"] and len(comb.inputs) == 2
    fused = recognise([partial, combine])
    assert fused.role == "main" and fused.split == 8 and [tuple(p.dims) for p in fused.outputs] == [(256, 1, 128)]


def test_plans_this_library_has_no_kernel_for_are_refused():
    from types import SimpleNamespace as NS

    from cleave_b200.core.errors import CodegenError

    c = DATA["cfg1_matmul"]
    with pytest.raises(CodegenError):
        recognise([])
    with pytest.raises(CodegenError):
        recognise(NS(tile=NS(flat_graph=NS(nodes=[]))))
    # x @ w with w stored (N, K): the kernels read W as (K, N), so the plan is refused, not mis-bound
    rec = _records("cfg1_matmul")[0]
    nodes = [dict(n) for n in rec["nodes"]]
    mm = next(n for n in nodes if n["type"] == "Matmul")
    mm["transpose_B"] = True
    with pytest.raises(CodegenError):
        recognise(plan_fixtures.plan_from_record(dict(rec, nodes=nodes)))
    del c


LIVE = {"cfg1_matmul"} | ({"swiglu", "demo_matmul_rowsum", "demo_matmul_matmul", "demo_lora"}
                          if os.environ.get("CLEAVE_B200_LIVE_PLANS") else set())


@pytest.mark.skipif(not reference_env.available(), reason="no reference checkout on this machine")
@pytest.mark.parametrize("case", sorted(LIVE))
def test_live_plans_of_the_reference(case):
    """Runs the reference's own ``superoptimize`` -> ``schedule`` now and feeds EVERY plan to the code
    generator. Configuration 1 (solo and split-K 4 / 8 / 16: seconds) always; the slower searches when
    CLEAVE_B200_LIVE_PLANS is set (the recorded fixtures cover them otherwise)."""
    import make_plans

    try:
        cleave = reference_env.activate()
    except Exception as exc:  # noqa: BLE001 - a machine without the reference's build dependencies
        pytest.skip(f"the reference's plan producer does not build here: {exc}")
    import cleave.lang as rcl
    from cleave.pipeline.compile import as_program, resolve_configs
    from cleave.pipeline.config import SuperoptConfig
    from cleave.pipeline.plans import schedule
    from cleave.pipeline.superopt import superoptimize

    fn, shapes, dtype, split, so_kw, _ = make_plans.programs(cleave, rcl)[case]
    program = as_program(fn, shapes, dtype)
    so, sc, _ = resolve_configs(program, preset="default", superopt=SuperoptConfig(**so_kw) if so_kw else None,
                                schedule=None, eval=None, split=split)
    plans = schedule(superoptimize(program, so.replace(cache=False)), sc)
    assert len(plans) > 0
    traced = TRACED[case]()
    program_inputs = [(s.name, tuple(int(d) for d in s.shape)) for s in program.inputs]
    gen, texts = B200CodeGen(), {}
    for plan in plans:
        _check_plan(plan, traced, program_inputs)
        key = make_plans.json.dumps(make_plans.plan_record(plan), sort_keys=True)
        text = gen.gen(plan)
        assert texts.setdefault(key, text) == text          # equal plans, byte-equal text
    pairs = {}
    for plan in plans:
        if plan.role in ("partial", "combine"):
            pairs.setdefault(plan.variant, {}).setdefault(plan.role, plan)
    for variant, pair in pairs.items():
        fused = recognise([pair["partial"], pair["combine"]])
        assert fused.role == "main" and f"split-k={fused.split}" == variant
