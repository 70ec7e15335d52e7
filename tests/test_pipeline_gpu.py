"""End-to-end ``compile`` on the GPU: candidates are validated and timed, the best becomes a
callable Kernel that can be saved, loaded and cached; paged operators return a PagedKernel."""

import json

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _fast():
    from cleave_b200.pipeline import EvalConfig

    return EvalConfig(warmup=2, iters=20)


def test_compile_matmul_split_k_save_load_cache(tmp_path, monkeypatch):
    """Reference: tests/pipeline_api/test_e2e.py:32-99 (matmul e2e, split-K chain == x.float() @ w.float(),
    save/load, cache hit)."""
    import cleave_b200 as cleave
    import cleave_b200.lang as cl

    monkeypatch.setenv("CLEAVE_CACHE_ROOT", str(tmp_path / "cache"))

    @cleave.jit
    def matmul(x: cl.Tensor["M", "K"], w: cl.Tensor["K", "N"]):
        return x @ w

    k = cleave.compile(matmul, shapes=dict(M=128, N=128, K=4096), dtype=cl.f16, split=cl.Split("K", (4, 8)),
                       eval=_fast())
    assert "main_kernel" in k.source
    rep = k.report
    assert set(rep.variants()) == {"solo", "split-k=4", "split-k=8"} and len(rep.correct) == 3
    assert k.latency_us == min(v.latency_us for v in rep.variants().values())
    x = torch.randn(128, 4096, device="cuda").half()
    w = (torch.randn(4096, 128, device="cuda") / 64).half()
    y = k(x, w)
    torch.testing.assert_close(y.float(), x.float() @ w.float(), rtol=2e-2, atol=5e-2)
    assert torch.equal(k(x=x, w=w), y)
    for variant in ("solo", "split-k=8"):
        torch.testing.assert_close(rep.best(variant)(x, w).float(), x.float() @ w.float(), rtol=2e-2, atol=5e-2)
    with pytest.raises(ValueError):
        k(w, x)
    loaded = cleave.load(k.save(tmp_path / "saved"))
    assert torch.equal(loaded(x, w), y) and loaded.variant == k.variant
    again = cleave.compile(matmul, shapes=dict(M=128, N=128, K=4096), dtype=cl.f16, split=cl.Split("K", (4, 8)),
                           eval=_fast())
    assert again.meta.get("cache_hit") and torch.equal(again(x, w), y)


def test_compile_rmsnorm_gamma_swiglu_attention_and_mla():
    import cleave_b200 as cleave
    import cleave_b200.lang as cl
    from cleave_b200.runtime import reference as R

    @cleave.jit
    def rn(x: cl.Tensor["M", "K"], g: cl.Tensor["K"], w: cl.Tensor["K", "N"]):
        return (cl.rms_norm(x, eps=1e-6) * g) @ w

    @cleave.jit
    def sw(x: cl.Tensor["M", "K"], w0: cl.Tensor["K", "N"], w1: cl.Tensor["K", "N"]):
        return cl.silu(x @ w0) * (x @ w1)

    @cleave.jit
    def att(q: cl.Tensor["HQ", "SQ", "D"], k: cl.Tensor["HKV", "SKV", "D"], v: cl.Tensor["HKV", "SKV", "D"]):
        n = q.shape[-1] ** 0.5
        return cl.softmax((q @ k.mT) / n, dim=-1, shift=-50 / n) @ v

    @cleave.jit
    def mla(q: cl.Tensor["B", "H", "D"], kv: cl.Tensor["B", "SKV", "D"], q_pe: cl.Tensor["B", "H", "PE"],
            k_pe: cl.Tensor["B", "SKV", "PE"]):
        s = (q @ kv.mT + q_pe @ k_pe.mT) * 0.07
        return cl.softmax(s, dim=-1) @ kv

    g = torch.Generator(device="cuda").manual_seed(1)
    rnd = lambda *s, dt=torch.float16: torch.randn(*s, device="cuda", generator=g).to(dt)  # noqa: E731
    k1 = cleave.compile(rn, shapes=dict(M=64, N=512, K=1024), eval=_fast(), cache_kernels=False)
    x, gm, w = rnd(64, 1024), 1 + 0.1 * rnd(1024), rnd(1024, 512) / 32
    torch.testing.assert_close(k1(x, gm, w).float(), R.rmsnorm_matmul(x, w, 1e-6, gm), rtol=2e-2, atol=2e-2)
    k2 = cleave.compile(sw, shapes=dict(M=128, N=256, K=512), eval=_fast(), cache_kernels=False)
    x, w0, w1 = rnd(128, 512), rnd(512, 256) / 22, rnd(512, 256) / 22
    torch.testing.assert_close(k2(x, w0, w1).float(), R.swiglu(x, w0, w1), rtol=2e-2, atol=2e-2)
    k3 = cleave.compile(att, shapes=dict(HQ=32, HKV=8, SQ=1, SKV=777, D=128), eval=_fast(), cache_kernels=False)
    q, kk, v = rnd(32, 1, 128), rnd(8, 777, 128), rnd(8, 777, 128)
    torch.testing.assert_close(k3(q, kk, v).float(), R.attention(q, kk, v), rtol=2e-2, atol=2e-2)
    assert set(k3.report.variants()) == {"solo"}
    # the same program at a prefill shape (demo/gqa_prefill.py) runs on the tcgen05 attention kernel
    k3p = cleave.compile(att, shapes=dict(HQ=8, HKV=2, SQ=300, SKV=300, D=64), eval=_fast(), cache_kernels=False)
    q, kk, v = rnd(8, 300, 64), rnd(2, 300, 64), rnd(2, 300, 64)
    torch.testing.assert_close(k3p(q, kk, v).float(), R.attention(q, kk, v), rtol=2e-2, atol=2e-2)
    k4 = cleave.compile(mla, shapes=dict(B=2, H=32, SKV=300, D=512, PE=64), dtype=cl.bf16, eval=_fast(),
                        cache_kernels=False)
    bf = torch.bfloat16
    q, kv, qp, kp = rnd(2, 32, 512, dt=bf), rnd(2, 300, 512, dt=bf), rnd(2, 32, 64, dt=bf), rnd(2, 300, 64, dt=bf)
    torch.testing.assert_close(k4(q, kv, qp, kp).float(), R.mla_decode(q, kv, qp, kp, 0.07), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("page_size", [64, 1])
def test_compile_paged_gqa_decode(tmp_path, page_size):
    """Reference: tests/frontend_dynamic/test_paged_pipeline.py:63-92 - lens [700, 1, 129, 64], a pool three
    pages larger than needed, out and lse at 1e-2, named call bit-identical, page size 1 takes None for
    the unread kv_last_page_len, a saved and loaded kernel reproduces the same bits."""
    import cleave_b200 as cleave
    from cleave_b200.pipeline.dynamic import make_inputs, reference

    dims = dict(num_qo_heads=32, num_kv_heads=8, head_dim=128, page_size=page_size)
    wl = [("a", [700, 1, 129, 64]), ("b", [5, 0, 7]), ("c", [3000] * 3)]
    k = cleave.compile("gqa_paged_decode", dtype="bfloat16", workloads=wl, **dims)
    assert k.report.n_workloads == 3 and k.report.best() is not None
    # the split / single question of the reference's calibrate_dispatch, measured on the persistent kernel
    # (reference: python/cleave/pipeline/dynamic.py:209-242; persisted as in tests/frontend_dynamic/test_paged_trace.py:281-328)
    d = k.dispatch
    assert d is k.report.dispatch and d["n_workloads"] == 3 and 1 <= d["min_tiles"] <= 48
    assert set(d["geomean_us"]) == {"hybrid", "split", "single"} and d["geomean_us"]["hybrid"] <= d["geomean_us"]["split"] + 1e-9
    assert d["page_size"] == page_size and d["kv_tile"] == 64 and d["indptr_index"] == 3 and isinstance(d["applied"], bool)
    assert "dispatch" in k.report.summary()
    args = make_inputs("gqa_paged_decode", dims, [700, 1, 129, 64], "bfloat16", seed=5)
    want_out, want_lse = reference("gqa_paged_decode", args)
    out, lse = k(*args)
    torch.testing.assert_close(out.float(), want_out.float(), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(lse, want_lse, rtol=1e-2, atol=1e-2)
    names = ["q", "k_cache", "v_cache", "kv_indptr", "kv_indices", "kv_last_page_len", "sm_scale"]
    out2, lse2 = k(**dict(zip(names, args)))
    assert torch.equal(out, out2) and torch.equal(lse, lse2)
    if page_size == 1:
        assert args[5] is None
        with pytest.raises(ValueError):
            k(*args[:5], torch.zeros(4, dtype=torch.int32, device="cuda"), args[6])
    else:
        with pytest.raises(TypeError):
            k(*args[:5], None, args[6])
    loaded = cleave.load(k.save(tmp_path / "paged"))
    out3, lse3 = loaded(*args)
    assert torch.equal(out, out3) and torch.equal(lse, lse3)
    assert (tmp_path / "paged" / "dispatch.json").exists() and loaded.dispatch == json.loads(json.dumps(d))
    # scratch is owned by the compiled kernel's wrapper and allocated once: a further call allocates nothing
    # (reference: tests/graph/handwritten/test_splitkv_decode.py:85-111)
    owner = k.compile()._compiled
    assert owner.scratch_bytes > 0 and len(owner.workspaces) >= 1
    outs = [torch.empty_like(out), torch.empty_like(lse)]
    kept = [a for a in args if a is not None]
    owner(*kept, *outs)
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    owner(*kept, *outs)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before and torch.equal(outs[0], out)


def test_compile_paged_mla_decode_and_refusals():
    import cleave_b200 as cleave
    from cleave_b200.core.errors import PagingRefusal
    from cleave_b200.pipeline.dynamic import make_inputs, reference

    dims = dict(num_qo_heads=16, head_dim_ckv=512, head_dim_kpe=64)
    k = cleave.compile("mla_paged_decode", dtype="bfloat16", workloads=[("a", [5, 0, 7, 300])], **dims)
    args = make_inputs("mla_paged_decode", dims, [64, 2000, 1], "bfloat16", seed=2)
    want_out, want_lse = reference("mla_paged_decode", args)
    out, lse = k(*args)
    torch.testing.assert_close(out.float(), want_out.float(), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(lse, want_lse, rtol=1e-2, atol=1e-2)
    with pytest.raises(PagingRefusal):
        cleave.compile("gqa_paged_decode", num_qo_heads=32, num_kv_heads=8, head_dim=96, page_size=16)
    with pytest.raises(PagingRefusal):
        cleave.compile("mla_paged_decode", num_qo_heads=16, head_dim_ckv=256, head_dim_kpe=64)


@pytest.mark.parametrize("op", ["gqa_ragged_prefill_causal", "gqa_paged_prefill_causal", "mla_paged_prefill_causal"])
def test_compile_causal_prefill_operators(tmp_path, op):
    """The ragged and paged causal prefill operators of the reference's registry
    (python/cleave/dynamic/registry.py) through the same compile / call / save / load path."""
    import cleave_b200 as cleave
    from cleave_b200.pipeline.dynamic import OPERATORS, make_inputs, reference

    family = OPERATORS[op][0]
    dims = dict(num_qo_heads=8, num_kv_heads=2, head_dim=64)
    if family == "mla_paged_prefill":
        dims = dict(num_qo_heads=16, head_dim_ckv=512, head_dim_kpe=64)
    wl = [("a", ([100, 0, 300], [300, 50, 300])), ("b", ([1], [129])), ("c", ([257, 5], [600, 5]))]
    k = cleave.compile(op, dtype="bfloat16", workloads=wl, **dims)
    assert k.report.n_workloads == 3 and k.report.best() is not None
    args = make_inputs(family, dims, ([200, 17, 0, 128], [333, 17, 9, 128]), "bfloat16", seed=3)
    want_out, want_lse = reference(family, args)
    out, lse = k(*args)
    torch.testing.assert_close(out.float(), want_out.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(lse, want_lse, rtol=1e-2, atol=1e-2)
    out2, lse2 = k(**dict(zip(OPERATORS[op][1], args)))
    assert torch.equal(out, out2) and torch.equal(lse, lse2)
    loaded = cleave.load(k.save(tmp_path / op))
    out3, lse3 = loaded(*args)
    assert torch.equal(out, out3) and torch.equal(lse, lse3)


SHIPPED = [  # the nine operators of the reference's registry (python/cleave/dynamic/registry.py:91-196), with their dims
    ("gqa_paged_decode", dict(num_qo_heads=32, num_kv_heads=8, head_dim=128, page_size=1)),
    ("gqa_paged_decode", dict(num_qo_heads=32, num_kv_heads=4, head_dim=128, page_size=1)),
    ("gqa_paged_decode", dict(num_qo_heads=32, num_kv_heads=8, head_dim=128, page_size=64)),
    ("gqa_paged_prefill_causal", dict(num_qo_heads=32, num_kv_heads=8, head_dim=128)),
    ("gqa_paged_prefill_causal", dict(num_qo_heads=32, num_kv_heads=4, head_dim=128)),
    ("gqa_ragged_prefill_causal", dict(num_qo_heads=32, num_kv_heads=8, head_dim=128)),
    ("gqa_ragged_prefill_causal", dict(num_qo_heads=32, num_kv_heads=4, head_dim=128)),
    ("mla_paged_decode", dict(num_qo_heads=16, head_dim_ckv=512, head_dim_kpe=64)),
    ("mla_paged_prefill_causal", dict(num_qo_heads=16, head_dim_ckv=512, head_dim_kpe=64)),
]


@pytest.mark.parametrize("op,dims", SHIPPED, ids=[f"{o}-{'-'.join(str(v) for v in d.values())}" for o, d in SHIPPED])
def test_every_shipped_paged_operator_at_its_own_dims(op, dims):
    """Each operator the reference ships, with the head counts and page size it ships them with: compiled, validated
    over workloads, and called on fresh inputs against the reference's torch semantics."""
    import cleave_b200 as cleave
    from cleave_b200.pipeline.dynamic import OPERATORS, make_inputs, reference

    family = OPERATORS[op][0]
    prefill = "prefill" in family
    wl = ([("a", ([90, 0, 260], [300, 40, 260])), ("b", ([1, 129], [700, 129]))] if prefill
          else [("a", [700, 1, 129, 64]), ("b", [5, 0, 2100])])
    k = cleave.compile(op, dtype="bfloat16", workloads=wl, **dims)
    assert k.report.n_workloads == 2 and k.report.best() is not None
    lens = ([150, 0, 64], [410, 12, 64]) if prefill else [333, 0, 65, 1500]
    args = make_inputs(family, dims, lens, "bfloat16", seed=11)
    want_out, want_lse = reference(family, args)
    out, lse = k(*args)
    torch.testing.assert_close(out.float(), want_out.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(lse, want_lse, rtol=1e-2, atol=1e-2)


def test_check_code_in_a_spawned_worker(tmp_path):
    """The default check function is picklable and runs in a spawned worker with its own CUDA context,
    reading the parent-built reference file (reference: python/cleave/runtime/workers.py:104-122)."""
    from cleave_b200.codegen import make_spec
    from cleave_b200.runtime.evaluate import run_candidates
    from cleave_b200.runtime.validate import BenchOptions, publish_reference

    specs = [make_spec("matmul", "float16", {"M": 64, "N": 128, "K": 512}, split=s) for s in (1, 4)]
    res = run_candidates(specs, reference_fn=lambda d: publish_reference(d, specs[0])[0], pool="spawn",
                         max_parallel=1, timeout_s=240, benchmark=BenchOptions(2, 10))
    assert [r.status for r in res] == ["ok", "ok"], [str(r.error) for r in res]
    assert all(r.latency_ms and r.latency_ms > 0 for r in res)


def test_two_stage_split_k_chain_and_fused_kernel_agree(tmp_path, monkeypatch):
    """Reference: tests/pipeline_api/test_e2e.py:58-81 - a split-K variant whose partial and combine plans are
    built and timed separately runs as ONE Kernel of two chained stages, its latency the sum of its members',
    and equals x.float() @ w.float(). Here that form is scheduled beside the fused split kernel on request."""
    import cleave_b200 as cleave
    import cleave_b200.lang as cl

    monkeypatch.setenv("CLEAVE_CACHE_ROOT", str(tmp_path / "cache"))

    @cleave.jit
    def matmul(x: cl.Tensor["M", "K"], w: cl.Tensor["K", "N"]):
        return x @ w

    k = cleave.compile(matmul, shapes=dict(M=128, N=128, K=4096), dtype=cl.f16, split=cl.Split("K", (4, 8)),
                       eval=_fast(), two_stage=True)
    rep = k.report
    assert {"solo", "split-k=4", "split-k=8", "split-k=4/two-stage", "split-k=8/two-stage"} == set(rep.variants())
    assert not rep.failures, rep.summary()
    pair = rep.best("split-k=4/two-stage")
    assert [s.role for s in pair.stages] == ["partial", "combine"] and pair.unrunnable is None
    members = rep.variants()["split-k=4/two-stage"].members
    assert pair.latency_us == pytest.approx(sum(m.latency_us for m in members))
    x = torch.randn(128, 4096, device="cuda").half()
    w = (torch.randn(4096, 128, device="cuda") / 64).half()
    want = x.float() @ w.float()
    torch.testing.assert_close(pair(x, w).float(), want, rtol=2e-2, atol=5e-2)
    torch.testing.assert_close(rep.best("split-k=4")(x, w).float(), want, rtol=2e-2, atol=5e-2)
    loaded = cleave.load(pair.save(tmp_path / "pair"))
    assert [s.role for s in loaded.stages] == ["partial", "combine"] and torch.equal(loaded(x, w), pair(x, w))
    assert (tmp_path / "pair" / "kernel_0_partial.py").exists() and (tmp_path / "pair" / "kernel_1_combine.py").exists()


def test_two_stage_split_kv_decode_attention():
    """The split-KV partial + combine pair of decode attention (reference kernels:
    tests/graph/handwritten/expected_kernels/gqa_split_partial.py + mha_split_combine.py) against the unsplit
    fp32 reference, and the partial stage alone against the per-split sums it is defined to emit."""
    import cleave_b200 as cleave
    import cleave_b200.lang as cl
    from cleave_b200.runtime import reference as R

    @cleave.jit
    def att(q: cl.Tensor["HQ", "SQ", "D"], k: cl.Tensor["HKV", "SKV", "D"], v: cl.Tensor["HKV", "SKV", "D"]):
        n = q.shape[-1] ** 0.5
        return cl.softmax((q @ k.mT) / n, dim=-1, shift=-50 / n) @ v

    kern = cleave.compile(att, shapes=dict(HQ=32, HKV=8, SQ=1, SKV=4096, D=128), dtype=cl.f16, split=cl.Split("SKV", (4, 8)),
                          eval=_fast(), two_stage=True, cache_kernels=False)
    rep = kern.report
    assert not rep.failures, rep.summary()
    assert {"solo", "split-k=4/two-stage", "split-k=8/two-stage"} <= set(rep.variants())
    g = torch.Generator(device="cuda").manual_seed(3)
    q = torch.randn(32, 1, 128, device="cuda", generator=g).half()
    k = torch.randn(8, 4096, 128, device="cuda", generator=g).half()
    v = torch.randn(8, 4096, 128, device="cuda", generator=g).half()
    want = R.attention(q, k, v, 128 ** -0.5)
    for variant in ("solo", "split-k=8/two-stage"):
        torch.testing.assert_close(rep.best(variant)(q, k, v).float(), want.float(), rtol=2e-2, atol=2e-2)


def test_real_reference_split_plans_run_as_two_stages():
    """The partial and combine plans the reference's scheduler really emits (recorded in tests/golden/plans.json)
    go through the code generator one by one, as the reference's build does (python/cleave/pipeline/build.py:165),
    and the two kernels chained give the operator's result: split-K matmul, split-KV GQA decode."""
    import plans as plan_fixtures
    from cleave_b200.codegen import B200CodeGen
    from cleave_b200.runtime.compile import _compile, _load_main_kernel_from_code
    from cleave_b200.runtime.reference import order_inputs_for_kernel

    data = plan_fixtures.load()
    gen = B200CodeGen()

    def bind(plan):
        spec = _load_main_kernel_from_code(gen.gen(plan))
        return spec, _compile(spec, list(range(-len(spec.outputs), 0)))

    g = torch.Generator(device="cuda").manual_seed(5)
    # ---- configuration 1, split-K 8
    c = data["cfg1_matmul"]
    partial = next(p for p in c["plans"] if p.role == "partial" and p.split_factor == 8)
    combine = next(p for p in c["plans"] if p.role == "combine" and p.split_factor == 8)
    (ps, pk), (cs, ck) = bind(partial), bind(combine)
    x = torch.randn(128, 4096, device="cuda", generator=g).half()
    w = (torch.randn(4096, 128, device="cuda", generator=g) / 64).half()
    roles = dict(zip(ps.input_roles(), [p.name for p in ps.inputs]))
    parts = pk(*order_inputs_for_kernel({roles["x"]: x, roles["w"]: w}, pk))
    assert tuple(parts.shape) == (8, 128, 128)
    torch.testing.assert_close(parts.float(), torch.stack([x[:, i * 512:(i + 1) * 512].float() @ w[i * 512:(i + 1) * 512].float()
                                                           for i in range(8)]), rtol=2e-2, atol=2e-2)
    y = ck(parts)
    torch.testing.assert_close(y.float(), x.float() @ w.float(), rtol=2e-2, atol=5e-2)
    # ---- configuration 3, split-KV 8 (both output orders the search emits)
    c = data["cfg3_gqa_decode"]
    q = torch.randn(256, 1, 128, device="cuda", generator=g).half()
    k = torch.randn(64, 8192, 128, device="cuda", generator=g).half()
    v = torch.randn(64, 8192, 128, device="cuda", generator=g).half()
    from cleave_b200.runtime import reference as R

    want = R.attention(q, k, v, 128 ** -0.5).float()
    combine = next(p for p in c["plans"] if p.role == "combine" and p.split_factor == 8)
    cs, ck = bind(combine)
    seen = set()
    for partial in (p for p in c["plans"] if p.role == "partial" and p.split_factor == 8):
        ps, pk = bind(partial)
        order = tuple(tuple(o.dims) for o in ps.outputs)
        if order in seen:
            continue
        seen.add(order)
        roles = dict(zip(ps.input_roles(), [p.name for p in ps.inputs]))
        outs = pk(*order_inputs_for_kernel({roles["q"]: q, roles["k"]: k, roles["v"]: v}, pk))
        by_size = sorted(outs, key=lambda t: -t.numel())          # weighted values, then weight sums
        feed = [None, None]
        feed[cs.attrs["num"]], feed[cs.attrs["den"]] = by_size[0], by_size[1]
        shaped = [t.reshape([int(d) for d in p.dims]) for t, p in zip(feed, cs.inputs)]
        out = ck(*shaped)
        torch.testing.assert_close(out.float().reshape(256, 1, 128), want, rtol=2e-2, atol=2e-2)
    assert len(seen) >= 1
