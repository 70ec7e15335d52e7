"""GPU parity of the MLA decode kernels (through the C ABI) against the reference's golden
vectors, the oracle, and size-independent properties."""

import numpy as np
import pytest
import torch

import cases
from _util import assert_close, assert_lse_close, dev, host
from oracle import cleave_oracle as orc

pytestmark = pytest.mark.gpu

GOLDEN = cases.load_golden()


def _ops():
    from cleave_b200 import ops

    return ops


def _check_ws():
    ops = _ops()
    ops.check_workspace(ops.workspace("mla_decode", 0, "cuda"))


def _run_static(inp, dt, scale, **kw):
    out = _ops().mla_decode(dev(inp["q"], dt), dev(inp["kv"], dt), dev(inp["q_pe"], dt), dev(inp["k_pe"], dt),
                            scale, **kw)
    _check_ws()
    return host(out)


def _run_paged(inp, dt, **kw):
    out, lse = _ops().mla_paged_decode(dev(inp["q_nope"], dt), dev(inp["q_pe"], dt), dev(inp["ckv_cache"], dt),
                                       dev(inp["kpe_cache"], dt), dev(inp["kv_indptr"]), dev(inp["kv_indices"]),
                                       inp["sm_scale"], **kw)
    _check_ws()
    return host(out), host(lse)


@pytest.mark.parametrize("name", [n for n, c in cases.CASES.items() if c[0] == "mla"])
def test_static_mla_matches_reference_golden(name):
    _, inp, opt = cases.build(name)
    assert_close(_run_static(inp, opt["dtype"], opt["scale"]), GOLDEN[name][0])


@pytest.mark.parametrize("name", [n for n, c in cases.CASES.items() if c[0] == "mla_paged"])
def test_paged_mla_matches_reference_golden(name):
    _, inp, opt = cases.build(name)
    out, lse = _run_paged(inp, opt["dtype"])
    assert_close(out, GOLDEN[name][0])
    assert_lse_close(lse, GOLDEN[name][1])


@pytest.mark.parametrize("impl", ["tcgen05", "mma_sync"])
@pytest.mark.parametrize("b,h,skv", [(1, 16, 64), (2, 128, 1000), (3, 32, 65), (1, 48, 4097), (1, 200, 33), (5, 128, 700), (9, 72, 600)])
@pytest.mark.parametrize("dt", ["bf16", "f16"])
@pytest.mark.parametrize("max_ctas", [0, 1, 5])
def test_static_mla_vs_oracle(b, h, skv, dt, max_ctas, impl):
    inp = cases.mla_inputs(b + h + skv, b, h, skv, 512, 64, dt)
    scale = 192 ** -0.5
    got = _run_static(inp, dt, scale, max_ctas=max_ctas, impl=impl)
    assert_close(got, orc.mla_decode(inp["q"], inp["kv"], inp["q_pe"], inp["k_pe"], scale, dt))


@pytest.mark.parametrize("h,impl", [(16, "tcgen05"), (16, "mma_sync"), (8, "auto"), (128, "auto")])
@pytest.mark.parametrize("max_ctas", [0, 2])
def test_paged_mla_vs_oracle(h, impl, max_ctas):
    lens = [0, 1, 63, 64, 65, 127, 128, 129, 700, 3001, 17]
    inp = cases.mla_paged_inputs(77, lens, h, 512, 64, "bf16", cases.MLA_SM_SCALE)
    out, lse = _run_paged(inp, "bf16", max_ctas=max_ctas, impl=impl)
    want_out, want_lse = orc.mla_paged_decode(inp["q_nope"], inp["q_pe"], inp["ckv_cache"], inp["kpe_cache"],
                                              inp["kv_indptr"], inp["kv_indices"], inp["sm_scale"])
    assert_close(out, want_out)
    assert_lse_close(lse, want_lse)


def test_paged_mla_ranges_beyond_the_page_table_are_clipped():
    """kv_indptr is caller data: ranges that run past the ``num_kv_indices`` entries of kv_indices are read as
    shorter requests (the entries that exist), never as memory behind the table."""
    lens = [300, 65, 2000, 900]
    inp = cases.mla_paged_inputs(78, lens, 16, 512, 64, "bf16", cases.MLA_SM_SCALE)
    keep = int(inp["kv_indptr"][2]) + 130   # request 2 keeps 130 of its tokens, request 3 none
    inp["kv_indices"] = np.ascontiguousarray(inp["kv_indices"][:keep])
    out, lse = _run_paged(inp, "bf16")
    clipped = np.minimum(inp["kv_indptr"], keep).astype(np.int32)
    want_out, want_lse = orc.mla_paged_decode(inp["q_nope"], inp["q_pe"], inp["ckv_cache"], inp["kpe_cache"],
                                              clipped, inp["kv_indices"], inp["sm_scale"])
    assert_close(out, want_out)
    assert_lse_close(lse, want_lse)
    assert (out[3] == 0).all() and np.isneginf(lse[3]).all()


def test_static_mla_large_logits_rescale_path():
    """Logits that jump half-way along the sequence force the tensor-memory kernel through its
    rescale of the accumulator (the running maximum grows by far more than 2^8 between two tiles)."""
    inp = cases.mla_inputs(99, 1, 128, 512, 512, 64, "bf16")
    step = np.where(np.arange(512) < 256, 0.2, 3.0).astype(np.float32)[None, :, None]
    inp["kv"] = orc.round_to(inp["kv"] * step, "bf16")
    scale = 0.1
    want = orc.mla_decode(inp["q"], inp["kv"], inp["q_pe"], inp["k_pe"], scale, "bf16")
    assert np.isfinite(want).all()
    for impl in ("tcgen05", "mma_sync"):
        assert_close(_run_static(inp, "bf16", scale, impl=impl), want, rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("dt", ["bf16", "f16"])
def test_paged_mla_tcgen05_large_logits_rescale_and_repeat(dt):
    """Paged form on the tcgen05 kernel: the tokens late in every request have cache rows fifteen times larger,
    so the running maxima grow by far more than 2^8 between two tiles and the accumulator in tensor memory is
    rescaled; a single CTA walks all requests (several pieces per CTA), and two launches are bit-identical."""
    lens = [1000, 260, 515]
    inp = cases.mla_paged_inputs(101, lens, 16, 512, 64, dt, 0.1)
    for b in range(len(lens)):
        lo, hi = int(inp["kv_indptr"][b]), int(inp["kv_indptr"][b + 1])
        late = inp["kv_indices"][lo + (hi - lo) // 2:hi]
        inp["ckv_cache"][late] = orc.round_to(inp["ckv_cache"][late] * 3.0, dt)
        early = inp["kv_indices"][lo:lo + (hi - lo) // 2]
        inp["ckv_cache"][early] = orc.round_to(inp["ckv_cache"][early] * 0.2, dt)
    want_out, want_lse = orc.mla_paged_decode(inp["q_nope"], inp["q_pe"], inp["ckv_cache"], inp["kpe_cache"],
                                              inp["kv_indptr"], inp["kv_indices"], inp["sm_scale"], dt)
    assert np.isfinite(want_out).all()
    for max_ctas in (1, 0):
        out, lse = _run_paged(inp, dt, max_ctas=max_ctas, impl="tcgen05")
        out2, lse2 = _run_paged(inp, dt, max_ctas=max_ctas, impl="tcgen05")
        assert np.array_equal(out, out2) and np.array_equal(lse, lse2)
        assert_close(out, want_out, rtol=3e-2, atol=3e-2)
        assert_lse_close(lse, want_lse)


def test_paged_mla_tcgen05_large_batch():
    """700 short requests, some of them empty: every CTA walks many pieces, and most requests are whole inside
    one CTA."""
    rng = np.random.default_rng(5)
    lens = [int(x) for x in rng.integers(0, 200, size=700)]
    inp = cases.mla_paged_inputs(102, lens, 16, 512, 64, "bf16", cases.MLA_SM_SCALE)
    out, lse = _run_paged(inp, "bf16", impl="tcgen05")
    want_out, want_lse = orc.mla_paged_decode(inp["q_nope"], inp["q_pe"], inp["ckv_cache"], inp["kpe_cache"],
                                              inp["kv_indptr"], inp["kv_indices"], inp["sm_scale"])
    assert_close(out, want_out)
    assert_lse_close(lse, want_lse)


def test_mla_full_config_properties():
    """Benchmark configuration 4 at full size (batch 16, 128 heads, 512 + 64, KV 4096, bf16): compared with
    the oracle on one request, invariant under a permutation of the KV positions, and repeat
    launches are bit-identical."""
    g = torch.Generator(device="cpu").manual_seed(0)
    q = torch.randn(16, 128, 512, generator=g).bfloat16()
    qp = torch.randn(16, 128, 64, generator=g).bfloat16()
    kv = torch.randn(16, 4096, 512, generator=g).bfloat16()
    kp = torch.randn(16, 4096, 64, generator=g).bfloat16()
    scale = 192 ** -0.5
    ops = _ops()
    out = ops.mla_decode(q.cuda(), kv.cuda(), qp.cuda(), kp.cuda(), scale)
    out2 = ops.mla_decode(q.cuda(), kv.cuda(), qp.cuda(), kp.cuda(), scale)
    assert torch.equal(out, out2)
    perm = torch.randperm(4096, generator=g)
    out_p = ops.mla_decode(q.cuda(), kv[:, perm].contiguous().cuda(), qp.cuda(), kp[:, perm].contiguous().cuda(), scale)
    _check_ws()
    assert_close(host(out), host(out_p), rtol=1e-2, atol=1e-2)
    want = orc.mla_decode(q[3:4].float().numpy(), kv[3:4].float().numpy(), qp[3:4].float().numpy(),
                          kp[3:4].float().numpy(), scale, "bf16")
    assert_close(host(out[3:4]), want)


@pytest.mark.parametrize("impl", ["tcgen05", "mma_sync"])
def test_static_mla_after_a_kernel_that_appends_to_the_caches(impl):
    """A decode loop appends the step's rows to the caches right before it calls the operator, on the same
    stream. The operator's launches may be scheduled while that kernel still runs (dependent launches) and
    must not read the caches before it has finished: the result has to see the appended rows."""
    b, h, skv = 4, 128, 2048
    inp = cases.mla_inputs(123, b, h, skv, 512, 64, "bf16")
    new = cases.mla_inputs(124, b, h, skv, 512, 64, "bf16")
    scale = 192 ** -0.5
    q, qp = dev(inp["q"], "bf16"), dev(inp["q_pe"], "bf16")
    kv, kp = dev(inp["kv"], "bf16"), dev(inp["k_pe"], "bf16")
    kv_new, kp_new = dev(new["kv"], "bf16"), dev(new["k_pe"], "bf16")
    ops = _ops()
    ops.mla_decode(q, kv, qp, kp, scale, impl=impl)           # warm: modules loaded, workspace allocated
    torch.cuda.synchronize()
    for _ in range(3):
        kv.copy_(kv_new)                                      # the "append": rewrites every row of both caches
        kp.copy_(kp_new)
        out = ops.mla_decode(q, kv, qp, kp, scale, impl=impl)
        _check_ws()
        assert_close(host(out), orc.mla_decode(inp["q"], new["kv"], inp["q_pe"], new["k_pe"], scale, "bf16"))
        kv.copy_(dev(inp["kv"], "bf16"))
        kp.copy_(dev(inp["k_pe"], "bf16"))
        torch.cuda.synchronize()


def test_paged_mla_tcgen05_after_a_kernel_that_rewrites_its_inputs():
    """The paged tcgen05 kernel is a dependent launch too: it may be scheduled while the kernel before it on the
    stream still runs and must not read the caches, Q or the page table before that kernel has finished."""
    lens = [700, 64, 1300, 90]
    a = cases.mla_paged_inputs(201, lens, 16, 512, 64, "bf16", cases.MLA_SM_SCALE)
    b = cases.mla_paged_inputs(202, lens, 16, 512, 64, "bf16", cases.MLA_SM_SCALE)   # same shapes, other data and pages
    ops = _ops()
    dev_a = {k: dev(v, "bf16") if v.dtype != np.int32 else dev(v) for k, v in a.items() if isinstance(v, np.ndarray)}
    dev_b = {k: dev(v, "bf16") if v.dtype != np.int32 else dev(v) for k, v in b.items() if isinstance(v, np.ndarray)}
    names = ("q_nope", "q_pe", "ckv_cache", "kpe_cache", "kv_indptr", "kv_indices")
    live = {k: dev_a[k].clone() for k in names}
    run = lambda: ops.mla_paged_decode(live["q_nope"], live["q_pe"], live["ckv_cache"], live["kpe_cache"],   # noqa: E731
                                       live["kv_indptr"], live["kv_indices"], a["sm_scale"], impl="tcgen05")
    run()
    torch.cuda.synchronize()
    want = {}
    for tag, src in (("a", a), ("b", b)):
        want[tag] = orc.mla_paged_decode(src["q_nope"], src["q_pe"], src["ckv_cache"], src["kpe_cache"],
                                         src["kv_indptr"], src["kv_indices"], src["sm_scale"])
    for tag, src in (("b", dev_b), ("a", dev_a), ("b", dev_b)):
        for k in names:
            live[k].copy_(src[k])          # rewrites every input right before the launch, on the same stream
        out, lse = run()
        _check_ws()
        assert_close(host(out), want[tag][0])
        assert_lse_close(host(lse), want[tag][1])


@pytest.mark.parametrize("impl", ["tile", "per_token"])
def test_paged_causal_mla_prefill_matches_reference_golden_and_oracle(impl):
    """Reference: python/cleave/dynamic/reference.py:324-365 (mla_paged_prefill_causal_h16_ckv512_kpe64_ps1):
    the golden case from the reference's own definition, and a second seeded case against the oracle with
    requests without queries, without keys, and with more queries than keys. Both implementations: the
    tcgen05 query-tile kernel and the per-token form on the paged decode kernel."""
    ops = _ops()
    _, inp, opt = cases.build("mla_paged_prefill_bf16")
    i32 = lambda a: torch.from_numpy(a).cuda()  # noqa: E731
    out, lse = ops.mla_paged_prefill(dev(inp["q_nope"], "bf16"), dev(inp["q_pe"], "bf16"), dev(inp["ckv_cache"], "bf16"),
                                     dev(inp["kpe_cache"], "bf16"), i32(inp["qo_indptr"]), i32(inp["kv_indptr"]),
                                     i32(inp["kv_indices"]), inp["sm_scale"], impl=impl)
    _check_ws()
    ops.check_workspace(ops.workspace("mla_prefill", 0, "cuda"))
    assert_close(host(out), GOLDEN["mla_paged_prefill_bf16"][0])
    assert_lse_close(host(lse), GOLDEN["mla_paged_prefill_bf16"][1])
    inp = cases.mla_prefill_inputs(9, [33, 200, 0, 7, 20], [64, 260, 5, 0, 12], 16, 512, 64, "bf16", cases.MLA_SM_SCALE)
    out, lse = ops.mla_paged_prefill(dev(inp["q_nope"], "bf16"), dev(inp["q_pe"], "bf16"), dev(inp["ckv_cache"], "bf16"),
                                     dev(inp["kpe_cache"], "bf16"), i32(inp["qo_indptr"]), i32(inp["kv_indptr"]),
                                     i32(inp["kv_indices"]), inp["sm_scale"], impl=impl)
    _check_ws()
    ops.check_workspace(ops.workspace("mla_prefill", 0, "cuda"))
    want, want_lse = orc.mla_paged_prefill(inp["q_nope"], inp["q_pe"], inp["ckv_cache"], inp["kpe_cache"], inp["qo_indptr"],
                                           inp["kv_indptr"], inp["kv_indices"], inp["sm_scale"])
    assert_close(host(out), want)
    assert_lse_close(host(lse), want_lse)


def test_mla_prefill_many_short_prompts():
    """Ninety prompts of 0...120 tokens with up to 200 cached tokens in front: more than a thousand (block, column half)
    items of one or two KV tiles, which the host hands to the persistent form of the kernel (items dealt by a counter
    in the workspace header, barrier phases running on across items). Against the oracle, twice on one workspace."""
    ops = _ops()
    rng = np.random.default_rng(90)
    q_lens = [int(x) for x in rng.integers(0, 121, 90)]
    kv_lens = [int(q + c) for q, c in zip(q_lens, rng.integers(0, 201, 90))]
    kv_lens[5] = 0
    q_lens[11], kv_lens[11] = 100, 30   # leading blocks blind
    inp = cases.mla_prefill_inputs(91, q_lens, kv_lens, 16, 512, 64, "bf16", cases.MLA_SM_SCALE)
    i32 = lambda a: torch.from_numpy(a).cuda()  # noqa: E731
    args = (dev(inp["q_nope"], "bf16"), dev(inp["q_pe"], "bf16"), dev(inp["ckv_cache"], "bf16"), dev(inp["kpe_cache"], "bf16"),
            i32(inp["qo_indptr"]), i32(inp["kv_indptr"]), i32(inp["kv_indices"]), inp["sm_scale"])
    assert 2 * (sum(-(-q // 8) for q in q_lens) + 90) >= 3 * 148 and sum(kv_lens) <= 320 * 90  # the host's rule
    want, want_lse = orc.mla_paged_prefill(inp["q_nope"], inp["q_pe"], inp["ckv_cache"], inp["kpe_cache"], inp["qo_indptr"],
                                           inp["kv_indptr"], inp["kv_indices"], inp["sm_scale"], dtype="bf16")
    first = None
    for _ in range(2):
        out, lse = ops.mla_paged_prefill(*args, impl="tile")
        ops.check_workspace(ops.workspace("mla_prefill", 0, "cuda"))
        assert_close(host(out), want)
        assert_lse_close(host(lse), want_lse)
        if first is None:
            first = out.clone()
    assert torch.equal(first, out)


@pytest.mark.parametrize("heads", [16, 64])
def test_mla_prefill_short_and_ragged_key_windows(heads):
    """Key counts on both sides of every boundary the kernel treats specially: the 16-row rounds of the gather (rows
    past a request's last key are zero-filled in shared memory, not fetched), the 32- and 64-score groups the softmax
    skips when no row of a warp sees them, and the 128-token tile. The shared memory a launch finds may hold anything:
    a launch over NaN caches runs first."""
    ops = _ops()
    q_lens = [1, 3, 8, 1, 2, 9, 1, 20, 5, 1, 40]
    kv_lens = [1, 15, 16, 17, 31, 32, 33, 63, 64, 65, 129 + 47]
    inp = cases.mla_prefill_inputs(77 + heads, q_lens, kv_lens, heads, 512, 64, "bf16", cases.MLA_SM_SCALE)
    i32 = lambda a: torch.from_numpy(a).cuda()  # noqa: E731
    args = [dev(inp["q_nope"], "bf16"), dev(inp["q_pe"], "bf16"), dev(inp["ckv_cache"], "bf16"), dev(inp["kpe_cache"], "bf16"),
            i32(inp["qo_indptr"]), i32(inp["kv_indptr"]), i32(inp["kv_indices"]), inp["sm_scale"]]
    poisoned = list(args)
    poisoned[2] = torch.full_like(args[2], float("nan"))
    poisoned[3] = torch.full_like(args[3], float("nan"))
    ops.mla_paged_prefill(*poisoned, impl="tile")  # leaves NaN rows behind in shared memory
    out, lse = ops.mla_paged_prefill(*args, impl="tile")
    ops.check_workspace(ops.workspace("mla_prefill", 0, "cuda"))
    want, want_lse = orc.mla_paged_prefill(inp["q_nope"], inp["q_pe"], inp["ckv_cache"], inp["kpe_cache"], inp["qo_indptr"],
                                           inp["kv_indptr"], inp["kv_indices"], inp["sm_scale"], dtype="bf16")
    assert_close(host(out), want)
    assert_lse_close(host(lse), want_lse)


@pytest.mark.parametrize("heads,dt", [(16, "f16"), (32, "bf16"), (128, "bf16"), (8, "bf16")])
def test_mla_prefill_tile_kernel_vs_oracle(heads, dt):
    """The query-tile kernel over head counts that pack 8, 4, 1 and 16 query tokens into the 128 MMA rows, with
    query lengths that are not multiples of the block, prefixes longer than a KV tile, chunked prefill
    (fewer queries than keys) and the two implementations agreeing with each other."""
    ops = _ops()
    q_lens, kv_lens = [130, 1, 257, 40, 0], [130, 300, 257, 1000, 9]
    inp = cases.mla_prefill_inputs(40 + heads, q_lens, kv_lens, heads, 512, 64, dt, cases.MLA_SM_SCALE)
    i32 = lambda a: torch.from_numpy(a).cuda()  # noqa: E731
    args = (dev(inp["q_nope"], dt), dev(inp["q_pe"], dt), dev(inp["ckv_cache"], dt), dev(inp["kpe_cache"], dt),
            i32(inp["qo_indptr"]), i32(inp["kv_indptr"]), i32(inp["kv_indices"]), inp["sm_scale"])
    out, lse = ops.mla_paged_prefill(*args, impl="tile")
    ops.check_workspace(ops.workspace("mla_prefill", 0, "cuda"))
    want, want_lse = orc.mla_paged_prefill(inp["q_nope"], inp["q_pe"], inp["ckv_cache"], inp["kpe_cache"], inp["qo_indptr"],
                                           inp["kv_indptr"], inp["kv_indices"], inp["sm_scale"], dtype=dt)
    assert_close(host(out), want)
    assert_lse_close(host(lse), want_lse)
    out2, lse2 = ops.mla_paged_prefill(*args, impl="per_token")
    _check_ws()
    assert_close(host(out), host(out2))
    out3, _ = ops.mla_paged_prefill(*args, impl="tile")
    assert torch.equal(out, out3)   # repeat launches are bit-identical
