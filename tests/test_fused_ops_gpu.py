"""GPU parity, through the C ABI, of the remaining fused operators of the reference's demo set:
exact-softmax attention (demo/mha_decode_exact.py), (Q K^T) V (demo/matmul_matmul.py), QK-norm attention
(demo/qknorm.py), rowsum(X @ W) (demo/matmul_rowsum.py) and LoRA (demo/lora.py) - against golden outputs of
the reference's own torch path, against the oracle over shape sweeps, and at the demos' full sizes."""

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


def _check(kind):
    ops = _ops()
    ops.check_workspace(ops.workspace(kind, 0, "cuda"))


def _run(name):
    family, inp, opt = cases.build(name)
    dt, ops = opt["dtype"], _ops()
    d = lambda k: dev(inp[k], dt)  # noqa: E731
    if family == "attention_exact":
        out = ops.attention_prefill(d("q"), d("k"), d("v"))
        _check("attn_prefill")
    elif family == "matmul_matmul":
        out = ops.matmul_matmul(d("q"), d("k"), d("v"))
        _check("attn_prefill")
    elif family == "qknorm":
        out = ops.qknorm_attention(d("q"), d("k"), d("v"), eps=opt["eps"])
        _check("attn_prefill")
    elif family == "matmul_rowsum":
        out = ops.matmul_rowsum(d("x"), d("w0"))
    else:
        out = ops.lora(d("x"), d("w"), d("a"), d("b"))
        _check("lora")
    return host(out)


NEW = ("attention_exact", "matmul_matmul", "qknorm", "matmul_rowsum", "lora")


@pytest.mark.parametrize("name", [n for n, c in cases.CASES.items() if c[0] in NEW])
def test_matches_reference_golden(name):
    """Golden outputs of the reference's own torch path (cleave.trace(...).reference / Program.reference)."""
    assert_close(_run(name), GOLDEN[name][0])


@pytest.mark.parametrize("dt", ["f16", "bf16"])
@pytest.mark.parametrize("hq,hkv,sq,skv,d", [(4, 4, 256, 256, 64), (8, 2, 300, 517, 128), (4, 1, 130, 1000, 64),
                                             (3, 3, 1, 77, 64), (2, 1, 640, 640, 128), (160, 32, 129, 260, 64)])
@pytest.mark.parametrize("impl", ["scores_first", "chain"])
def test_matmul_matmul_vs_oracle(hq, hkv, sq, skv, d, dt, impl):
    """Reference: demo/matmul_matmul.py:11-13, in both evaluation orders. Key counts that are not multiples
    of the tile sizes check that rows past the end contribute nothing (they are zero rows of K and V)."""
    inp = cases.matmul_matmul_inputs(hq * 1000 + sq, hq, hkv, sq, skv, d, dt)
    got = _ops().matmul_matmul(dev(inp["q"], dt), dev(inp["k"], dt), dev(inp["v"], dt), impl=impl)
    _check("attn_prefill")
    assert_close(host(got), orc.matmul_matmul(inp["q"], inp["k"], inp["v"], dt))


def test_matmul_matmul_chain_is_bit_stable_and_picked_for_long_sequences():
    """The token chunks of K^T V are summed in a fixed order by the last CTA to arrive: repeat launches give
    the same bits. The automatic choice takes the chain at the demo shape and keeps (Q K^T) V where the
    chain saves little (demo/matmul_matmul.py's split preset, S_Q = 64)."""
    import ctypes as C

    from cleave_b200 import _lib

    inp = cases.matmul_matmul_inputs(3, 8, 4, 1000, 3000, 64, "f16")
    q, k, v = dev(inp["q"], "f16"), dev(inp["k"], "f16"), dev(inp["v"], "f16")
    first = _ops().matmul_matmul(q, k, v, impl="chain")
    for _ in range(3):
        assert torch.equal(_ops().matmul_matmul(q, k, v, impl="chain"), first)
    a = _lib.MatmulMatmulArgs()
    a.num_qo_heads, a.num_kv_heads, a.q_len, a.kv_len, a.head_dim, a.dtype = 32, 32, 4096, 4096, 64, _lib.F16
    assert _lib.lib().cb200_matmul_matmul_uses_chain(C.byref(a)) == 1
    a.q_len = 64
    assert _lib.lib().cb200_matmul_matmul_uses_chain(C.byref(a)) == 0


@pytest.mark.parametrize("dt", ["f16", "bf16"])
@pytest.mark.parametrize("hq,hkv,sq,skv,d", [(4, 4, 256, 256, 64), (8, 2, 300, 517, 128), (4, 1, 130, 1000, 64),
                                             (2, 2, 1, 77, 128), (160, 32, 129, 260, 64)])
@pytest.mark.parametrize("eps", [1e-6, 0.5])
def test_qknorm_attention_vs_oracle(hq, hkv, sq, skv, d, dt, eps):
    """Reference: demo/qknorm.py:17-24. eps = 0.5 makes the epsilon visible next to mean(x^2) ~ 1."""
    inp = cases.attention_inputs(hq * 1000 + skv, hq, hkv, sq, skv, d, dt)
    got = _ops().qknorm_attention(dev(inp["q"], dt), dev(inp["k"], dt), dev(inp["v"], dt), eps=eps)
    _check("attn_prefill")
    assert_close(host(got), orc.qknorm_attention(inp["q"], inp["k"], inp["v"], eps, dt))


def test_qknorm_is_invariant_under_row_scaling():
    """RMS normalisation removes a per-row factor: scaling every q row and k row by its own power of two
    (exact in 16 bits) must not change the result beyond eps effects (eps = 0 here)."""
    inp = cases.attention_inputs(7, 8, 2, 200, 300, 128, "f16")
    ops = _ops()
    q, k, v = dev(inp["q"], "f16"), dev(inp["k"], "f16"), dev(inp["v"], "f16")
    base = ops.qknorm_attention(q, k, v, eps=0.0)
    g = torch.Generator(device="cpu").manual_seed(0)
    fq = (2.0 ** torch.randint(-2, 3, (8, 200, 1), generator=g)).half().cuda()
    fk = (2.0 ** torch.randint(-2, 3, (2, 300, 1), generator=g)).half().cuda()
    scaled = ops.qknorm_attention(q * fq, k * fk, v, eps=0.0)
    _check("attn_prefill")
    assert_close(host(scaled), host(base), rtol=2e-3, atol=2e-3)


def test_exact_softmax_shapes_route_to_the_same_kernel_as_shifted():
    """demo/mha_decode_exact.py (H 32, S_Q 64, S_KV 256, D 64): the exact row maximum and the demos' fixed
    shift are the same function; one kernel serves both and matches both oracles."""
    inp = cases.attention_inputs(99, 32, 32, 64, 256, 64, "f16")
    got = host(_ops().attention_prefill(dev(inp["q"], "f16"), dev(inp["k"], "f16"), dev(inp["v"], "f16")))
    _check("attn_prefill")
    assert_close(got, orc.attention_exact(inp["q"], inp["k"], inp["v"], "f16"))
    assert_close(got, orc.attention(inp["q"], inp["k"], inp["v"], "f16"))


@pytest.mark.parametrize("dt", ["f16", "bf16"])
@pytest.mark.parametrize("m,n,k", [(4096, 4096, 64), (1, 8, 8), (33, 72, 320), (1000, 1032, 4096), (7, 16384, 264)])
def test_matmul_rowsum_vs_oracle(m, n, k, dt):
    """Reference: demo/matmul_rowsum.py:6-8 (first shape: the demo's own)."""
    inp = cases.gemm_inputs(m + n, m, n, k, dt)
    got = _ops().matmul_rowsum(dev(inp["x"], dt), dev(inp["w0"], dt))
    assert got.shape == (m, 1)
    assert_close(host(got), orc.matmul_rowsum(inp["x"], inp["w0"], dt))


@pytest.mark.parametrize("dt", ["f16", "bf16"])
@pytest.mark.parametrize("m,n,k,r", [(16, 4096, 4096, 16), (1, 8, 64, 8), (200, 264, 320, 8), (128, 1024, 512, 64),
                                     (600, 2048, 1024, 16), (16, 11008, 4096, 32)])
def test_lora_vs_oracle(m, n, k, r, dt):
    """Reference: demo/lora.py:11-18 (first shape: the demo's own, Mirage's demo_lora dims)."""
    inp = cases.lora_inputs(m + n + r, m, n, k, r, dt)
    got = _ops().lora(*(dev(inp[x], dt) for x in ("x", "w", "a", "b")))
    _check("lora")
    assert_close(host(got), orc.lora(inp["x"], inp["w"], inp["a"], inp["b"], dt))


def test_lora_with_zero_adapter_equals_matmul():
    """B = 0 makes the low-rank K block contribute exact zeros to the accumulator: the result is the plain
    product up to the order of the fp32 sum (the K split of a product with one more K block may differ)."""
    inp = cases.lora_inputs(5, 48, 520, 1024, 16, "f16")
    ops = _ops()
    x, w, a = dev(inp["x"], "f16"), dev(inp["w"], "f16"), dev(inp["a"], "f16")
    got = ops.lora(x, w, a, torch.zeros(16, 520, dtype=torch.float16, device="cuda"))
    assert_close(host(got), host(ops.matmul(x, w)), rtol=2.0 ** -9, atol=2.0 ** -9)


@pytest.mark.parametrize("dt", ["f16", "bf16"])
@pytest.mark.parametrize("m,n,k,k2,split_k", [(16, 4096, 4096, 16, 0), (128, 256, 512, 64, 0), (200, 264, 320, 8, 0),
                                              (64, 512, 1024, 72, 4), (600, 2048, 1024, 136, 0), (1024, 2048, 1024, 16, 0),
                                              (40, 72, 64, 200, 2)])
def test_matmul_with_a_second_operand_pair_and_an_addend(m, n, k, k2, split_k, dt):
    """``Y = X @ W + X2 @ W2 + C`` in one launch: the K blocks of the second pair follow those of the first
    in the same accumulator, C is added in the epilogue. Cluster plans, the stream-K walk (explicit split)
    and sizes the CTA-pair kernel would otherwise take."""
    rng = np.random.default_rng(m + n + k2)
    r = lambda shape, sc: orc.round_to(rng.standard_normal(shape, dtype=np.float32) * np.float32(sc), dt)  # noqa: E731
    x, w = r((m, k), 1.0), r((k, n), k ** -0.5)
    x2, w2, c = r((m, k2), 1.0), r((k2, n), k2 ** -0.5), r((m, n), 1.0)
    got = _ops().matmul(dev(x, dt), dev(w, dt), split_k=split_k, addend=dev(c, dt), x2=dev(x2, dt), w2=dev(w2, dt))
    _check("gemm")
    assert_close(host(got), orc.round_to(x @ w + x2 @ w2 + c, dt))
    only_pair = _ops().matmul(dev(x, dt), dev(w, dt), split_k=split_k, x2=dev(x2, dt), w2=dev(w2, dt))
    assert_close(host(only_pair), orc.round_to(x @ w + x2 @ w2, dt))


def test_gemm_addend_rejected_outside_plain_matmul():
    import ctypes as C

    from cleave_b200 import _lib

    a = _lib.GemmArgs()
    a.m, a.n, a.k, a.op, a.dtype, a.addend = 64, 64, 64, _lib.GEMM_SWIGLU, _lib.F16, 16
    assert _lib.lib().cb200_gemm_workspace_bytes(C.byref(a)) == 0
    b = _lib.GemmArgs()
    b.m, b.n, b.k, b.op, b.dtype, b.k2 = 64, 64, 64, _lib.GEMM_RMSNORM, _lib.F16, 16
    assert _lib.lib().cb200_gemm_workspace_bytes(C.byref(b)) == 0  # the second operand pair is plain-matmul only
    b.op, b.k2, b.dependent_launch = _lib.GEMM_MATMUL, 0, 3
    assert _lib.lib().cb200_gemm_workspace_bytes(C.byref(b)) == 0  # mode 3 waits on a second pair that is not there


def test_demo_sizes_against_oracle_slices():
    """The demos' full sizes: (Q K^T) V at B*H 32, S 4096, D 64 and QK-norm attention at 64 / 8 heads,
    S 4096, D 128. Heads are independent, so the first and last query heads are compared with the oracle
    run on their slices (the whole problem is minutes of CPU work)."""
    ops = _ops()
    inp = cases.matmul_matmul_inputs(1, 32, 32, 4096, 4096, 64, "f16")
    for impl in ("chain", "scores_first"):
        got = host(ops.matmul_matmul(dev(inp["q"], "f16"), dev(inp["k"], "f16"), dev(inp["v"], "f16"), impl=impl))
        for h in (0, 31):
            assert_close(got[h:h + 1], orc.matmul_matmul(inp["q"][h:h + 1], inp["k"][h:h + 1], inp["v"][h:h + 1], "f16"))
    inp = cases.attention_inputs(2, 64, 8, 4096, 4096, 128, "f16")
    got = host(ops.qknorm_attention(dev(inp["q"], "f16"), dev(inp["k"], "f16"), dev(inp["v"], "f16"), eps=1e-6))
    _check("attn_prefill")
    for h in (0, 63):
        kv = h // 8
        assert_close(got[h:h + 1], orc.qknorm_attention(inp["q"][h:h + 1], inp["k"][kv:kv + 1], inp["v"][kv:kv + 1],
                                                        1e-6, "f16"))


def test_compile_the_remaining_demo_operators(tmp_path):
    """``compile`` on the demo programs, written as the reference's demos write them (jit functions for four,
    the imperative Program builder for LoRA): validated against the torch reference inside the pipeline,
    then called, saved and loaded."""
    import cleave_b200 as cleave
    import cleave_b200.lang as cl
    from cleave_b200.pipeline import EvalConfig
    from cleave_b200.runtime import reference as R

    fast = EvalConfig(warmup=2, iters=20)

    def attention(q, k, v):
        n = q.shape[-1] ** 0.5
        return cl.softmax((q @ k.mT) / n, dim=-1, shift=-50 / n) @ v

    @cleave.jit
    def matmul_matmul(q: cl.Tensor["BH", "SQ", "D"], k: cl.Tensor["BH", "SKV", "D"], v: cl.Tensor["BH", "SKV", "D"]):
        return (q @ k.mT) @ v

    @cleave.jit
    def matmul_rowsum(x: cl.Tensor["M", "K"], w: cl.Tensor["K", "N"]):
        return (x @ w).sum(-1, keepdim=True)

    @cleave.jit
    def qknorm(q: cl.Tensor["HQ", "SQ", "D"], k: cl.Tensor["HKV", "SKV", "D"], v: cl.Tensor["HKV", "SKV", "D"]):
        q_sq, k_sq = q * q, k * k
        q_ms, k_ms = q_sq.mean(-1, keepdim=True), k_sq.mean(-1, keepdim=True)
        qn = q * cl.rsqrt(q_ms + 1e-6)
        kn = k * cl.rsqrt(k_ms + 1e-6)
        return attention(qn, kn, v)

    @cleave.jit
    def mha_decode_exact(q: cl.Tensor["H", "SQ", "D"], k: cl.Tensor["H", "SKV", "D"], v: cl.Tensor["H", "SKV", "D"]):
        return cl.softmax((q @ k.mT) / q.shape[-1] ** 0.5, dim=-1) @ v

    def lora(M=16, N=4096, K=4096, R=16):
        p = cleave.Program("lora", dtype=cl.f16)
        M, K, N, R = p.dims(M=M, K=K, N=N, R=R)
        x, w = p.input("x", (M, K)), p.input("w", (K, N))
        a, b = p.input("a", (K, R)), p.input("b", (R, N))
        p.output(x @ w + (x @ a) @ b, name="y")
        return p

    g = torch.Generator(device="cuda").manual_seed(3)
    rnd = lambda *s: torch.randn(*s, device="cuda", generator=g).half()  # noqa: E731
    k1 = cleave.compile(matmul_matmul, shapes=dict(BH=4, SQ=300, SKV=300, D=64), dtype=cl.f16, eval=fast,
                        cache_kernels=False)
    q, k, v = rnd(4, 300, 64), rnd(4, 300, 64), rnd(4, 300, 64) / 140
    torch.testing.assert_close(k1(q, k, v).float(), R.matmul_matmul(q, k, v), rtol=2e-2, atol=2e-2)
    k2 = cleave.compile(matmul_rowsum, shapes=dict(M=4096, N=4096, K=64), dtype=cl.f16, eval=fast, cache_kernels=False)
    x, w = rnd(4096, 64), rnd(64, 4096) / 8
    y = k2(x, w)
    assert y.shape == (4096, 1)
    torch.testing.assert_close(y.float(), R.matmul_rowsum(x, w), rtol=2e-2, atol=2e-2)
    k3 = cleave.compile(qknorm, shapes=dict(HQ=8, HKV=2, SQ=300, SKV=300, D=128), dtype=cl.f16, eval=fast,
                        cache_kernels=False)
    q, k, v = rnd(8, 300, 128), rnd(2, 300, 128), rnd(2, 300, 128)
    torch.testing.assert_close(k3(q, k, v).float(), R.qknorm_attention(q, k, v, 1e-6), rtol=2e-2, atol=2e-2)
    k4 = cleave.compile(mha_decode_exact, shapes=dict(H=32, SQ=64, SKV=256, D=64), dtype=cl.f16, eval=fast, split=False,
                        cache_kernels=False)
    q, k, v = rnd(32, 64, 64), rnd(32, 256, 64), rnd(32, 256, 64)
    torch.testing.assert_close(k4(q, k, v).float(), R.attention(q, k, v), rtol=2e-2, atol=2e-2)
    k5 = cleave.compile(lora(), eval=fast, cache_kernels=False)
    x, w, a, b = rnd(16, 4096), rnd(4096, 4096) / 64, rnd(4096, 16) / 64, rnd(16, 4096) / 4
    y = k5(x, w, a, b)
    torch.testing.assert_close(y.float(), R.lora(x, w, a, b), rtol=2e-2, atol=2e-2)
    assert torch.equal(k5(x=x, w=w, a=a, b=b), y)
    loaded = cleave.load(k5.save(tmp_path / "lora"))
    assert torch.equal(loaded(x, w, a, b), y)
