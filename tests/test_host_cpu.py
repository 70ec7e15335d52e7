"""Host-side logic that needs no GPU: the C ABI exports, kernel-spec text, plan recognition,
tracing, the split-K pairing rule, and candidate orchestration with injected failures."""

import ctypes
import os
import re
import time
from types import SimpleNamespace

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_loads_and_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "cleave_b200.h")).read()
    declared = set(re.findall(r"^(?:int|size_t|const char\*)\s+(cb200_[a-z0-9_]+)\s*\(", header, re.M))
    assert len(declared) >= 14
    lib = ctypes.CDLL(os.path.join(ROOT, "cleave_b200", "libcleave_b200.so"))
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    lib.cb200_strerror.restype = ctypes.c_char_p
    assert lib.cb200_version() == 5
    assert b"workspace" in lib.cb200_strerror(4)


def test_kernel_text_is_deterministic_and_round_trips():
    from cleave_b200.codegen import B200CodeGen, make_spec
    from cleave_b200.pipeline.build import pass_configs_of
    from cleave_b200.runtime.compile import _load_main_kernel_from_code

    a = make_spec("matmul", "float16", {"M": 128, "N": 128, "K": 4096}, split=4)
    b = make_spec("matmul", "float16", {"K": 4096, "N": 128, "M": 128}, split=4)  # other key order
    ta, tb = B200CodeGen().gen(a), B200CodeGen(apply_rasterization=16).gen(b)
    assert ta == tb and "main_kernel" in ta
    back = _load_main_kernel_from_code(ta)
    assert back == a and back._cache_source_hint == ta
    assert B200CodeGen().gen(make_spec("matmul", "float16", {"M": 128, "N": 128, "K": 4096}, split=8)) != ta
    assert pass_configs_of(ta) == {}
    assert pass_configs_of("PASS_CONFIGS = {'tl.x': 1}\nmain_kernel = 0\n") == {"tl.x": 1}
    assert [p.name for p in a.params] == ["PlaceHolder_x", "PlaceHolder_w", "OutputNode"]


def test_trace_matches_the_demo_operators():
    import cleave_b200.lang as cl
    from cleave_b200.core.errors import SpecError
    from cleave_b200.frontend import jit, trace

    @jit
    def rmsnorm_matmul(x: cl.Tensor["M", "K"], w: cl.Tensor["K", "N"]):
        return cl.rms_norm(x, dim=-1) @ w

    p = trace(rmsnorm_matmul, dict(M=64, N=11008, K=4096), split=cl.Split("K", (4, 8)))
    assert (p.family, p.split, p.input_names) == ("rmsnorm_matmul", (4, 8), ["x", "w"])

    @jit
    def attention(q: cl.Tensor["HQ", "SQ", "D"], k: cl.Tensor["HKV", "SKV", "D"], v: cl.Tensor["HKV", "SKV", "D"]):
        n = q.shape[-1] ** 0.5
        return cl.softmax((q @ k.mT) / n, dim=-1, shift=-50 / n) @ v

    p = trace(attention, dict(HQ=32, HKV=8, SQ=1, SKV=4096, D=128))
    assert p.family == "attention_decode" and abs(p.attrs["scale"] - 128 ** -0.5) < 1e-9

    # the remaining demo operators (demo/matmul_matmul.py, matmul_rowsum.py, qknorm.py, mha_decode_exact.py, lora.py)
    @jit
    def matmul_matmul(q: cl.Tensor["BH", "SQ", "D"], k: cl.Tensor["BH", "SKV", "D"], v: cl.Tensor["BH", "SKV", "D"]):
        return (q @ k.mT) @ v

    p = trace(matmul_matmul, dict(BH=32, SQ=4096, SKV=4096, D=64))
    assert p.family == "matmul_matmul" and p.output_shapes == [(32, 4096, 64)]

    @jit
    def matmul_rowsum(x: cl.Tensor["M", "K"], w: cl.Tensor["K", "N"]):
        return (x @ w).sum(-1, keepdim=True)

    p = trace(matmul_rowsum, dict(M=4096, N=4096, K=64))
    assert p.family == "matmul_rowsum" and p.output_shapes == [(4096, 1)]

    @jit
    def qknorm(q: cl.Tensor["HQ", "SQ", "D"], k: cl.Tensor["HKV", "SKV", "D"], v: cl.Tensor["HKV", "SKV", "D"]):
        q_sq, k_sq = q * q, k * k
        q_ms, k_ms = q_sq.mean(-1, keepdim=True), k_sq.mean(-1, keepdim=True)
        qn = q * cl.rsqrt(q_ms + 1e-6)
        kn = k * cl.rsqrt(k_ms + 1e-6)
        n = qn.shape[-1] ** 0.5
        return cl.softmax((qn @ kn.mT) / n, dim=-1, shift=-50 / n) @ v

    p = trace(qknorm, dict(HQ=64, HKV=8, SQ=4096, SKV=4096, D=128))
    assert p.family == "qknorm_attention" and p.attrs["eps"] == 1e-6 and abs(p.attrs["scale"] - 128 ** -0.5) < 1e-9

    @jit
    def mha_decode_exact(q: cl.Tensor["H", "SQ", "D"], k: cl.Tensor["H", "SKV", "D"], v: cl.Tensor["H", "SKV", "D"]):
        return cl.softmax((q @ k.mT) / q.shape[-1] ** 0.5, dim=-1) @ v

    assert trace(mha_decode_exact, dict(H=32, SQ=64, SKV=256, D=64)).family == "attention_decode"

    from cleave_b200.frontend import Program

    prog = Program("lora", dtype=cl.f16)
    M, K, N, R = prog.dims(M=16, K=4096, N=4096, R=16)
    x, w = prog.input("x", (M, K)), prog.input("w", (K, N))
    a, b = prog.input("a", (K, R)), prog.input("b", (R, N))
    prog.output(x @ w + (x @ a) @ b, name="y")
    assert (prog.family, prog.dims, prog.input_names) == ("lora", {"M": 16, "N": 4096, "K": 4096, "R": 16},
                                                         ["x", "w", "a", "b"])
    assert prog.dtype == "float16" and prog.output_shapes == [(16, 4096)]
    with pytest.raises(SpecError):
        prog.input("late", (1, 1))

    @jit
    def unknown(x: cl.Tensor["M", "K"]):
        return x * 2.0

    with pytest.raises(SpecError):
        trace(unknown, dict(M=4, K=4))
    with pytest.raises(SpecError):
        trace(rmsnorm_matmul, dict(M=4))


def _result(variant, role, ms, label=""):
    from cleave_b200.pipeline.report import Result
    from cleave_b200.runtime.evaluate import CandidateResult

    plan = SimpleNamespace(variant=variant, role=role, label=label or f"{variant}/{role}")
    run = CandidateResult(plan, "ok" if ms is not None else "failed", None if ms is not None else "validate",
                          None, "code", "src", ms, plan.label)
    return Result(plan, run)


def test_split_k_pairing_rule():
    """Reference: python/cleave/pipeline/report.py:123-153 - solo = best main; a split variant is a single
    fused main, or partial + combine summed; a variant with a missing member is dropped."""
    from cleave_b200.pipeline.report import Report

    rep = Report([_result("solo", "main", 0.010), _result("solo", "main", 0.008),
                  _result("split-k=4", "main", 0.006), _result("split-k=8", "partial", 0.003),
                  _result("split-k=8", "combine", 0.002), _result("split-k=16", "partial", 0.001),
                  _result("split-k=2", "main", None)])
    v = rep.variants()
    assert set(v) == {"solo", "split-k=4", "split-k=8"}
    assert abs(v["solo"].latency_us - 8.0) < 1e-9 and abs(v["split-k=8"].latency_us - 5.0) < 1e-9
    assert min(v.values(), key=lambda x: x.latency_us).variant == "split-k=8"
    assert rep.histogram() == {"validate": 1}


def _fake_check(code, **kw):
    if code == "slow":
        time.sleep(30)
    if code == "crash":
        os._exit(3)
    if code == "wrong":
        err = AssertionError("mismatch")
        err._cleave_stage = "validate"
        raise err
    return "src:" + code, 0.001


def test_run_candidates_classifies_timeout_crash_and_wrong_answers():
    """Reference: tests/test_runtime_parallel.py:18-56 - failures are injected on the host."""
    from cleave_b200.core.errors import CandidateTimeout, CodegenError, ValidationError, WorkerCrash
    from cleave_b200.runtime.evaluate import run_candidates

    def build(c):
        if c == "nogen":
            raise ValueError("cannot generate")
        return c

    cands = ["good", "slow", "crash", "wrong", "nogen", "good2"]
    t0 = time.monotonic()
    res = run_candidates(cands, build_fn=build, check_fn=_fake_check, pool="fork", max_parallel=3, timeout_s=1.5)
    assert time.monotonic() - t0 < 20
    assert [r.status for r in res] == ["ok", "failed", "failed", "failed", "failed", "ok"]
    assert [r.stage for r in res] == [None, "timeout", "crash", "validate", "codegen", None]
    assert isinstance(res[1].error, CandidateTimeout) and isinstance(res[2].error, WorkerCrash)
    assert isinstance(res[3].error, ValidationError) and isinstance(res[4].error, CodegenError)
    assert res[0].cuda_src == "src:good" and res[0].latency_ms == 0.001
    # in process, without a pool
    res = run_candidates(["good", "wrong"], build_fn=build, check_fn=_fake_check)
    assert [r.stage for r in res] == [None, "validate"]


def test_kernel_binding_errors_and_save_load_roundtrip(tmp_path):
    from cleave_b200.codegen import B200CodeGen, make_spec
    from cleave_b200.pipeline.kernel import Kernel, Param, Stage, load

    src = B200CodeGen().gen(make_spec("matmul", "float16", {"M": 4, "N": 8, "K": 64}))
    k = Kernel([Stage("main", src, [-1], [Param("PlaceHolder_x", "input", 0, (4, 64)),
                                          Param("PlaceHolder_w", "input", 1, (64, 8))], "lbl", 1.5)],
               name="mm", input_names=["x", "w"], input_shapes=[(4, 64), (64, 8)], output_shapes=[(4, 8)],
               variant="solo", latency_us=1.5)
    x, w = SimpleNamespace(shape=(4, 64)), SimpleNamespace(shape=(64, 8))
    with pytest.raises(TypeError):
        k._arguments((x,), {})
    with pytest.raises(TypeError):
        k._arguments((x,), {"w": w})
    with pytest.raises(ValueError):
        k._arguments((w, x), {})
    assert k._arguments((), {"w": w, "x": x}) == [x, w]
    back = load(k.save(tmp_path / "k"))
    assert back.source == k.source and back.variant == "solo" and back.stages[0].params[1].shape == (64, 8)
    assert (tmp_path / "k" / "kernel.json").exists() and (tmp_path / "k" / "kernel.py").read_text() == src


def test_paged_workload_generator_is_seeded_and_ragged():
    from cleave_b200.pipeline.dynamic import paged_decode_workloads

    a, b = paged_decode_workloads(), paged_decode_workloads()
    assert a == b and len(a) == 18
    assert min(min(l) for _, l in a) >= 1 and max(max(l) for _, l in a) == 8192
    assert any(len(set(l)) > 1 for _, l in a)


def test_prefill_operators_in_the_dynamic_registry_and_kernel_text():
    """The ragged and paged causal prefill operators carry the reference's argument order
    (python/cleave/dynamic/reference.py:204-258), their kernel text round-trips, and their workload
    generator is seeded, causal (q_len <= kv_len) and includes a request without queries."""
    from cleave_b200.codegen import B200CodeGen, make_spec
    from cleave_b200.pipeline.dynamic import OPERATORS, paged_prefill_workloads
    from cleave_b200.runtime.compile import _load_main_kernel_from_code

    assert OPERATORS["gqa_ragged_prefill_causal"][1] == ("q", "k", "v", "qo_indptr", "kv_indptr", "sm_scale")
    assert OPERATORS["gqa_paged_prefill_causal"][1] == ("q", "k_cache", "v_cache", "qo_indptr", "kv_indptr", "kv_indices",
                                                        "sm_scale")
    for family in ("gqa_ragged_prefill", "gqa_paged_prefill"):
        spec = make_spec(family, "bfloat16", dict(num_qo_heads=32, num_kv_heads=8, head_dim=128))
        text = B200CodeGen().gen(spec)
        assert text == B200CodeGen().gen(spec)
        again = _load_main_kernel_from_code(text)
        assert again.family == family and [p.name for p in again.outputs] == ["OutputNode", "OutputNode_1"]
        assert again.outputs[1].dtype == "float32" and again.outputs[0].dims == ("total_q", 32, 128)
    a, b = paged_prefill_workloads(), paged_prefill_workloads()
    assert a == b and len(a) == 8
    assert all(q <= k for _, (ql, kl) in a for q, k in zip(ql, kl))
    assert any(0 in ql for _, (ql, _) in a)


def test_oracle_causal_mask_is_end_aligned():
    """python/cleave/dynamic/reference.py:129-133: query row r of q_len rows sees keys <= kv_len - q_len + r;
    with one query row the result equals unmasked attention over all keys."""
    import numpy as np

    from oracle import cleave_oracle as orc

    rng = np.random.default_rng(0)
    q = rng.standard_normal((2, 3, 16), dtype=np.float32)
    k = rng.standard_normal((2, 7, 16), dtype=np.float32)
    v = rng.standard_normal((2, 7, 16), dtype=np.float32)
    out, lse = orc.attention_masked(q, k, v, 0.25, True, "f16")
    for r in range(3):
        want, want_lse = orc.attention_masked(q[:, r:r + 1], k[:, :5 + r], v[:, :5 + r], 0.25, False, "f16")
        np.testing.assert_allclose(out[:, r:r + 1], want, rtol=1e-3, atol=1e-3)
        np.testing.assert_allclose(lse[:, r:r + 1], want_lse, rtol=1e-5, atol=1e-5)


def test_arch_description_and_tile_snapping():
    """The sm_100 row in the reference's format (python/cleave/arch/cuda.py:120-186) and the mapping of a
    scheduler's tile hints onto the kernels' tiles."""
    from cleave_b200 import arch

    dev = arch.B200()
    for name in ("reg_cap", "smem_cap", "compute_max_core", "warp_size", "sm_partition", "transaction_size",
                 "max_smem_usage", "bandwidth", "platform", "compute_capability", "l2_cache_size_bytes"):
        assert getattr(dev, name)  # every field of the reference's Arch is present and filled in
    assert dev.compute_max_core == arch.OFFLINE_DEVICES[100]["sms"] == 148
    assert [128, 256] in dev.get_avaliable_tensorintrin_shapes()
    assert dev.is_tensorcore_supported_precision("bfloat16", "float32")
    assert not dev.is_tensorcore_supported_precision("int8", "int32")
    assert arch.snap_tile(64, 32) == (128, 128)            # the split-K matmul partial's Hopper hint
    assert arch.snap_tile(128, 256) == (128, 256)
    assert arch.snap_tile(256, 128, m=4096) == (256, 256)
    assert arch.snap_tile(256, 128, m=64) == (128, 256)    # no pair tile for a 64-row problem
    assert arch.snap_tile(64, 512, n=128) == (128, 128)    # the problem has 128 columns only
    assert arch.tmem_columns_needed((128, 256)) == dev.tmem_columns
    with pytest.raises(ValueError):
        arch.snap_tile(0, 8)


def test_new_operators_refuse_cpu_tensors_and_bad_shapes():
    """There is no CPU path: every operator refuses host tensors before anything is launched, and shape
    errors are reported as ValueError like the reference's kernel binding does (python/cleave/pipeline/kernel.py:67-82)."""
    import torch

    from cleave_b200 import ops

    h = lambda *s: torch.zeros(*s, dtype=torch.float16)  # noqa: E731
    with pytest.raises(ValueError, match="CUDA"):
        ops.matmul_matmul(h(2, 8, 64), h(2, 8, 64), h(2, 8, 64))
    with pytest.raises(ValueError, match="CUDA"):
        ops.qknorm_attention(h(2, 8, 64), h(2, 8, 64), h(2, 8, 64))
    with pytest.raises(ValueError, match="CUDA"):
        ops.matmul_rowsum(h(8, 16), h(16, 8))
    with pytest.raises(ValueError, match="CUDA"):
        ops.lora(h(8, 16), h(16, 8), h(16, 8), h(8, 8))


def test_kernel_text_of_the_remaining_demo_operators_round_trips():
    from cleave_b200.codegen import B200CodeGen, make_spec
    from cleave_b200.runtime.compile import _load_main_kernel_from_code

    for family, dims, attrs in (("matmul_matmul", {"HQ": 32, "HKV": 32, "SQ": 4096, "SKV": 4096, "D": 64}, {}),
                                ("qknorm_attention", {"HQ": 64, "HKV": 8, "SQ": 4096, "SKV": 4096, "D": 128}, {"eps": 1e-6}),
                                ("matmul_rowsum", {"M": 4096, "N": 4096, "K": 64}, {}),
                                ("lora", {"M": 16, "N": 4096, "K": 4096, "R": 16}, {})):
        spec = make_spec(family, "float16", dims, attrs=attrs)
        text = B200CodeGen().gen(spec)
        assert "main_kernel" in text and text == B200CodeGen().gen(make_spec(family, "float16", dims, attrs=attrs))
        back = _load_main_kernel_from_code(text)
        assert back.family == family and back.dims == dims and [p.name for p in back.params] == [p.name for p in spec.params]
    assert [p.name for p in make_spec("lora", "float16", {"M": 16, "N": 4096, "K": 4096, "R": 16}).params] == [
        "PlaceHolder_x", "PlaceHolder_w", "PlaceHolder_a", "PlaceHolder_b", "OutputNode"]


def test_calibrate_dispatch_threshold_rule():
    """The reference's rule (python/cleave/pipeline/dynamic.py:209-242): the threshold with the best hybrid
    geomean over the observed tile counts, the smallest one on a tie, result fields kept."""
    from cleave_b200.core.errors import CleaveError
    from cleave_b200.pipeline.dynamic import WorkloadCandidate, calibrate_dispatch

    tiles = {"a": 1, "b": 4, "c": 32, "d": 128}
    pair = WorkloadCandidate("full grid", "", latency_us={"a": 9.0, "b": 9.0, "c": 10.0, "d": 20.0})
    solo = WorkloadCandidate("small grid", "", latency_us={"a": 5.0, "b": 6.0, "c": 30.0, "d": 200.0})
    d = calibrate_dispatch(pair, solo, tiles, kv_tile=64, page_size=16, indptr_index=3)
    assert d["min_tiles"] == 32 and d["split_runs"] == 2 and d["n_workloads"] == 4 and d["applied"]
    assert d["geomean_us"]["hybrid"] == pytest.approx((5.0 * 6.0 * 10.0 * 20.0) ** 0.25)
    assert (d["split_label"], d["single_label"], d["page_size"], d["kv_tile"]) == ("full grid", "small grid", 16, 64)
    # the full grid wins everywhere: threshold 1 (ties go to the smallest), nothing to apply
    never = WorkloadCandidate("small grid", "", latency_us={k: 50.0 for k in tiles})
    d2 = calibrate_dispatch(pair, never, tiles)
    assert d2["min_tiles"] == 1 and d2["split_runs"] == 4 and not d2["applied"]
    with pytest.raises(CleaveError):
        calibrate_dispatch(pair, WorkloadCandidate("x", ""), tiles)


def test_ctypes_structs_match_the_c_header(tmp_path):
    """Every argument struct of include/cleave_b200.h has the same size and the same field offsets in the ctypes
    mirror the package calls through (cleave_b200/_lib.py): a C program compiled from the header prints them."""
    import ctypes
    import shutil
    import subprocess

    from cleave_b200 import _lib

    if shutil.which("gcc") is None:
        pytest.skip("no C compiler")
    pairs = {"cb200_attn_decode_args": _lib.AttnDecodeArgs, "cb200_gemm_args": _lib.GemmArgs,
             "cb200_gemm_plan_info": _lib.GemmPlanInfo, "cb200_mla_prefill_args": _lib.MlaPrefillArgs,
             "cb200_split_combine_args": _lib.SplitCombineArgs, "cb200_attn_unnormalise_args": _lib.AttnUnnormaliseArgs,
             "cb200_matmul_rowsum_args": _lib.MatmulRowsumArgs, "cb200_matmul_matmul_args": _lib.MatmulMatmulArgs,
             "cb200_lora_args": _lib.LoraArgs, "cb200_mla_decode_args": _lib.MlaDecodeArgs,
             "cb200_attn_prefill_args": _lib.AttnPrefillArgs, "cb200_attn_prefill_ragged_args": _lib.AttnPrefillRaggedArgs}
    lines = ["#include <stdio.h>", "#include <stddef.h>", '#include "cleave_b200.h"', "int main(void) {"]
    for cname, cls in pairs.items():
        lines.append(f'  printf("{cname} size %zu\\n", sizeof({cname}));')
        for field, _ in cls._fields_:
            lines.append(f'  printf("{cname} {field} %zu\\n", offsetof({cname}, {field}));')
    lines += ["  return 0;", "}"]
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    include = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include")
    subprocess.run(["gcc", "-I", include, str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout
    got = {(a, b): int(c) for a, b, c in (ln.split() for ln in out.splitlines())}
    for cname, cls in pairs.items():
        assert got[(cname, "size")] == ctypes.sizeof(cls), cname
        for field, _ in cls._fields_:
            assert got[(cname, field)] == getattr(cls, field).offset, (cname, field)


def test_peer_fields_are_checked_before_any_device_call():
    """The multi-GPU fields of cb200_gemm_args and cb200_peer_scatter_cols are caller data: counts, pitches and
    alignments are refused with a status before the library touches CUDA (so this runs without a GPU)."""
    import ctypes as C

    from cleave_b200 import _lib

    L = _lib.lib()

    def gemm(**kw):
        a = _lib.GemmArgs()
        a.m, a.n, a.k, a.op, a.dtype = 512, 512, 512, 0, _lib.F16
        for k, v in kw.items():
            setattr(a, k, v)
        return L.cb200_gemm(C.byref(a), None)

    assert gemm(n_peers=8) == 1 and gemm(n_peers=-1) == 1          # at most seven peer copies
    assert gemm(ldy=504) == 1 and gemm(ldy=516) == 1               # the pitch covers the slice and is a multiple of 8
    a = _lib.GemmArgs()
    a.m, a.n, a.k, a.op, a.dtype, a.n_peers = 512, 512, 512, 0, _lib.F16, 2
    a.y_peers[0] = 4096
    assert L.cb200_gemm(C.byref(a), None) == 1                     # a peer pointer is missing
    a.y_peers[1] = 4104
    assert L.cb200_gemm(C.byref(a), None) == 1                     # ... or not 16-byte aligned

    dsts = (C.c_void_p * 2)(4096, 8192)
    scatter = lambda src, m, n, ld, d, nd, dt: L.cb200_peer_scatter_cols(src, m, n, ld, d, nd, dt, None)  # noqa: E731
    assert scatter(None, 8, 64, 128, dsts, 2, _lib.F16) == 1
    assert scatter(4096, 8, 60, 128, dsts, 2, _lib.F16) == 1       # 16-byte pieces
    assert scatter(4096, 8, 64, 56, dsts, 2, _lib.F16) == 1        # pitch shorter than the block
    assert scatter(4096, 8, 64, 128, dsts, 9, _lib.F16) == 1
    assert scatter(4096, 8, 64, 128, dsts, 2, 7) == 2              # dtype
    assert scatter(4100, 8, 64, 128, dsts, 2, _lib.F16) == 3       # alignment
    bad = (C.c_void_p * 2)(4096, 8200)
    assert scatter(4096, 8, 64, 128, bad, 2, _lib.F16) == 1
