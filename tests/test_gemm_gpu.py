"""GPU parity of the tcgen05 GEMM family (through the C ABI) against the reference's golden
vectors, the oracle, and size-independent properties."""

import numpy as np
import pytest
import torch

import cases
from _util import assert_close, dev, host
from oracle import cleave_oracle as orc

pytestmark = pytest.mark.gpu

GOLDEN = cases.load_golden()


def _ops():
    from cleave_b200 import ops

    return ops


def _check_ws():
    ops = _ops()
    ops.check_workspace(ops.workspace("gemm", 0, "cuda"))


def _run(family, inp, opt, split_k=0, max_ctas=0):
    ops, dt = _ops(), opt["dtype"]
    x, w0 = dev(inp["x"], dt), dev(inp["w0"], dt)
    if family == "matmul":
        y = ops.matmul(x, w0, split_k=split_k, max_ctas=max_ctas)
    elif family == "rmsnorm_matmul":
        g = dev(inp["gamma"], dt) if "gamma" in inp else None
        y = ops.rmsnorm_matmul(x, w0, eps=opt["eps"], gamma=g, split_k=split_k, max_ctas=max_ctas)
    else:
        y = ops.swiglu(x, w0, dev(inp["w1"], dt), split_k=split_k, max_ctas=max_ctas)
    _check_ws()
    return host(y)


GEMM_CASES = [n for n, c in cases.CASES.items() if c[0] in ("matmul", "rmsnorm_matmul", "swiglu")]


@pytest.mark.parametrize("split_k", [0, 1, 4, 8])
@pytest.mark.parametrize("name", GEMM_CASES)
def test_gemm_family_matches_reference_golden(name, split_k):
    family, inp, opt = cases.build(name)
    assert_close(_run(family, inp, opt, split_k), GOLDEN[name][0])


@pytest.mark.parametrize("m,n,k", [(128, 128, 4096), (64, 1024, 4096), (1, 64, 64), (300, 520, 1000), (129, 136, 72)])
@pytest.mark.parametrize("split_k", [0, 1, 3, 4, 16])
@pytest.mark.parametrize("dt", ["f16", "bf16"])
def test_matmul_vs_oracle(m, n, k, split_k, dt):
    inp = cases.gemm_inputs(m + n + k, m, n, k, dt)
    got = _run("matmul", inp, {"dtype": dt}, split_k)
    assert_close(got, orc.matmul(inp["x"], inp["w0"], dt))


@pytest.mark.parametrize("m,n,k", [(64, 1280, 4096), (200, 264, 520)])
@pytest.mark.parametrize("split_k", [0, 1, 3, 8])
@pytest.mark.parametrize("gamma", [False, True])
def test_rmsnorm_matmul_vs_oracle(m, n, k, split_k, gamma):
    inp = cases.gemm_inputs(7, m, n, k, "f16", gamma=gamma)
    got = _run("rmsnorm_matmul", inp, {"dtype": "f16", "eps": 1e-6}, split_k)
    assert_close(got, orc.rmsnorm_matmul(inp["x"], inp["w0"], 1e-6, inp.get("gamma"), "f16"))


@pytest.mark.parametrize("m,n,k", [(256, 512, 1024), (70, 200, 328)])
@pytest.mark.parametrize("split_k", [0, 1, 4, 5])
def test_swiglu_vs_oracle(m, n, k, split_k):
    inp = cases.gemm_inputs(8, m, n, k, "bf16", n_w=2)
    got = _run("swiglu", inp, {"dtype": "bf16"}, split_k)
    assert_close(got, orc.swiglu(inp["x"], inp["w0"], inp["w1"], "bf16"))


@pytest.mark.parametrize("family,m,n,k,dt", [
    ("matmul", 3000, 3336, 200, "f16"),    # ragged in M, N and K; a K shorter than the stage ring
    ("matmul", 2048, 4864, 1032, "bf16"),  # 17 K blocks: the stage ring wraps inside a tile
    ("swiglu", 2100, 2504, 136, "bf16"),
    ("swiglu", 1024, 4736, 520, "f16"),
    ("rmsnorm_matmul", 2048, 4864, 1032, "f16"),
    ("rmsnorm_gamma", 3000, 3336, 200, "bf16"),
    ("rmsnorm_gamma", 1024, 9728, 712, "f16"),
    # few 256 x 256 tiles and a long K: the K dimension is split over the pairs of one cluster
    ("matmul", 512, 4096, 4096, "f16"),
    ("matmul", 256, 4096, 4096, "bf16"),
    ("matmul", 300, 3336, 2056, "f16"),
    ("swiglu", 512, 2048, 4096, "bf16"),
    ("rmsnorm_gamma", 512, 4096, 2048, "f16"),
    ("rmsnorm_matmul", 257, 4096, 4096, "bf16"),
])
def test_large_gemms_on_cta_pairs(family, m, n, k, dt):
    """Shapes with at least one 256 x 256 tile per CTA pair take the cta_group::2 kernel."""
    gamma = family == "rmsnorm_gamma"
    fam = "rmsnorm_matmul" if gamma else family
    inp = cases.gemm_inputs(m + k, m, n, k, dt, n_w=2 if family == "swiglu" else 1, gamma=gamma)
    opt = {"dtype": dt, "eps": 1e-6}
    got = _run(fam, inp, opt)
    if family == "swiglu":
        want = orc.swiglu(inp["x"], inp["w0"], inp["w1"], dt)
    elif fam == "rmsnorm_matmul":
        want = orc.rmsnorm_matmul(inp["x"], inp["w0"], 1e-6, inp.get("gamma"), dt)
    else:
        want = orc.matmul(inp["x"], inp["w0"], dt)
    assert_close(got, want)
    assert np.array_equal(got, _run(fam, inp, opt))


def test_scratch_behind_the_counters_never_lands_in_another_shape_s_counters():
    """A launch that parks scratch behind the arrival counters (the RMSNorm pre-pass of the pair kernel)
    followed, on the same workspace, by a split launch of another shape with more tiles than the first:
    its counters must still read zero."""
    g = cases.gemm_inputs(21, 1024, 9728, 712, "f16", gamma=True)
    _run("rmsnorm_matmul", g, {"dtype": "f16", "eps": 1e-6})
    inp = cases.gemm_inputs(22, 2048, 2048, 256, "f16")
    got = _run("matmul", inp, {"dtype": "f16"}, split_k=4, max_ctas=5)
    assert_close(got, orc.matmul(inp["x"], inp["w0"], "f16"))


def test_automatic_plans_for_the_benchmark_shapes():
    """What the planner's cost model picks when the caller leaves the split to it: one cluster of 16 for
    the 128 x 128 x 4096 matmul, clusters of 3 for the 64 x 11008 x 4096 RMSNorm GEMM, whole tiles for a
    large square; an explicit factor is honoured."""
    import ctypes as C

    from cleave_b200 import _lib

    def split(m, n, k, op=0, split_k=0):
        a = _lib.GemmArgs()
        a.m, a.n, a.k, a.op, a.dtype, a.split_k = m, n, k, op, 0, split_k
        return _lib.lib().cb200_gemm_effective_split(C.byref(a))

    assert split(128, 128, 4096) == 16
    assert split(64, 11008, 4096, op=1) == 3
    assert split(8192, 8192, 4096) == 1
    assert split(128, 128, 4096, split_k=4) == 4


def test_sm100_policy_scores_and_ranks_gemm_candidates():
    """The sm_100 counterpart of the reference's tile policy (python/cleave/schedule/policy/default.py:1015-1110):
    the plan the kernels would run for a candidate and the cost model's estimate for it, and candidates ranked
    by that estimate - a split of 16 beats no split on the 128 x 128 x 4096 product, whole CTA-pair tiles win
    on a large square."""
    from cleave_b200.arch import TCPolicyB200
    from cleave_b200.codegen import make_spec

    pol = TCPolicyB200()
    small = pol.plan("matmul", {"M": 128, "N": 128, "K": 4096})
    assert small["kind"] == "cluster split-K" and small["split"] == 16 and small["grid"] == 16 and small["estimate_us"] > 0
    cfg2 = pol.plan("rmsnorm_matmul", {"M": 64, "N": 11008, "K": 4096})
    assert (cfg2["kind"], cfg2["split"], cfg2["tile"], cfg2["grid"]) == ("cluster split-K", 3, (128, 256), 129)
    big = pol.plan("matmul", {"M": 8192, "N": 8192, "K": 4096})
    assert big["kind"] == "CTA pairs" and big["tile"] == (256, 256)
    dims = {"M": 128, "N": 128, "K": 4096}
    specs = [make_spec("matmul", "float16", dims, split=s) for s in (1, 4, 16)]
    ranked = pol.rank(specs)
    assert [s.split for _, s in ranked][0] == 16 and ranked[0][0] <= ranked[-1][0]


def test_split_k_partials_sum_like_the_unsplit_product():
    """Reference: tests/pipeline_api/test_e2e.py:58-81 (the split-K chain equals x.float() @ w.float());
    here every split factor and every grid size must agree with the unsplit launch to fp32 round-off."""
    inp = cases.gemm_inputs(3, 128, 128, 4096, "f16")
    base = _run("matmul", inp, {"dtype": "f16"}, 1)
    for split_k, max_ctas in [(4, 0), (8, 0), (16, 0), (16, 3), (64, 0)]:
        got = _run("matmul", inp, {"dtype": "f16"}, split_k, max_ctas)
        np.testing.assert_allclose(got, base, rtol=2e-3, atol=2e-3)


def test_repeat_launches_are_bit_identical():
    inp = cases.gemm_inputs(4, 64, 1024, 2048, "f16", gamma=True)
    a = _run("rmsnorm_matmul", inp, {"dtype": "f16", "eps": 1e-6}, 8)
    b = _run("rmsnorm_matmul", inp, {"dtype": "f16", "eps": 1e-6}, 8)
    assert np.array_equal(a, b)


def test_linearity_at_full_rmsnorm_config():
    """Benchmark configuration 2 at full size (M 64, K 4096, N 11008, fp16): compared with the oracle, and
    scaling X by 2 leaves RMSNorm(X) @ W unchanged (the norm is scale-invariant when eps is tiny)."""
    g = torch.Generator(device="cpu").manual_seed(0)
    x = torch.randn(64, 4096, generator=g).half()
    gamma = (1 + 0.1 * torch.randn(4096, generator=g)).half()
    w = (torch.randn(4096, 11008, generator=g) / 64).half()
    ops = _ops()
    y = ops.rmsnorm_matmul(x.cuda(), w.cuda(), eps=1e-6, gamma=gamma.cuda())
    y2 = ops.rmsnorm_matmul((2 * x).cuda(), w.cuda(), eps=1e-6, gamma=gamma.cuda())
    _check_ws()
    assert_close(host(y), host(y2), rtol=4e-3, atol=4e-3)
    want = orc.rmsnorm_matmul(x.float().numpy(), w.float().numpy(), 1e-6, gamma.float().numpy(), "f16")
    assert_close(host(y), want)


def test_gemm_bad_arguments():
    from cleave_b200 import Cb200Error

    ops = _ops()
    x = torch.zeros(8, 60, dtype=torch.float16, device="cuda")
    w = torch.zeros(60, 64, dtype=torch.float16, device="cuda")
    with pytest.raises(Cb200Error):
        ops.matmul(x, w)  # K not a multiple of 8
