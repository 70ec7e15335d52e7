"""GPU parity of the decode-attention kernels (through the C ABI) against the oracle, the
reference's golden vectors and size-independent properties."""

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


def _run_paged(inp, dt, page_size, **kw):
    ops = _ops()
    last = dev(inp["kv_last_page_len"]) if page_size != 1 else None
    out, lse = ops.gqa_paged_decode(dev(inp["q"], dt), dev(inp["k_cache"], dt), dev(inp["v_cache"], dt),
                                    dev(inp["kv_indptr"]), dev(inp["kv_indices"]), last, inp["sm_scale"], **kw)
    ops.check_workspace(ops.workspace("attn_decode", 0, "cuda"))
    return host(out), host(lse)


@pytest.mark.parametrize("name", [n for n, c in cases.CASES.items() if c[0] == "gqa_paged"])
def test_paged_decode_matches_reference_golden(name):
    _, inp, opt = cases.build(name)
    out, lse = _run_paged(inp, opt["dtype"], opt["page_size"])
    want_out, want_lse = GOLDEN[name]
    assert_close(out, want_out)
    assert_lse_close(lse, want_lse)


@pytest.mark.parametrize("name", [n for n, c in cases.CASES.items() if c[0] == "attention" and c[1]["sq"] == 1])
def test_static_decode_matches_reference_golden(name):
    _, inp, opt = cases.build(name)
    dt = opt["dtype"]
    out = _ops().attention_decode(dev(inp["q"], dt), dev(inp["k"], dt), dev(inp["v"], dt))
    assert_close(host(out), GOLDEN[name][0])


@pytest.mark.parametrize("dt", ["f16", "bf16"])
@pytest.mark.parametrize("page_size", [1, 8, 16, 64, 128, 5])
@pytest.mark.parametrize("hq,hkv", [(32, 8), (8, 8), (32, 1), (16, 4)])
def test_paged_decode_vs_oracle(dt, page_size, hq, hkv):
    lens = [0, 1, 63, 64, 65, 700, 2049, 17]
    inp = cases.gqa_paged_inputs(100 + page_size, lens, hq, hkv, 128, page_size, dt)
    out, lse = _run_paged(inp, dt, page_size)
    last = inp["kv_last_page_len"] if page_size != 1 else None
    want_out, want_lse = orc.gqa_paged_decode(inp["q"], inp["k_cache"], inp["v_cache"], inp["kv_indptr"],
                                              inp["kv_indices"], last, inp["sm_scale"], out_dtype=dt)
    assert_close(out, want_out)
    assert_lse_close(lse, want_lse)


@pytest.mark.parametrize("max_ctas", [1, 3, 148])
def test_split_kv_combine_is_grid_invariant(max_ctas):
    """Cutting the tile stream over 1, 3 or all CTAs changes only the summation order."""
    lens = [5000, 1, 300, 4097, 129]
    inp = cases.gqa_paged_inputs(7, lens, 32, 8, 128, 64, "bf16")
    out, lse = _run_paged(inp, "bf16", 64, max_ctas=max_ctas)
    want_out, want_lse = orc.gqa_paged_decode(inp["q"], inp["k_cache"], inp["v_cache"], inp["kv_indptr"],
                                              inp["kv_indices"], inp["kv_last_page_len"], inp["sm_scale"])
    assert_close(out, want_out)
    assert_lse_close(lse, want_lse)


def test_paged_decode_d64():
    inp = cases.gqa_paged_inputs(9, [100, 0, 257], 16, 4, 64, 16, "f16")
    out, lse = _run_paged(inp, "f16", 16)
    want_out, want_lse = orc.gqa_paged_decode(inp["q"], inp["k_cache"], inp["v_cache"], inp["kv_indptr"],
                                              inp["kv_indices"], inp["kv_last_page_len"], inp["sm_scale"], "f16")
    assert_close(out, want_out)
    assert_lse_close(lse, want_lse)


def test_valid_len_clamp_on_device():
    """A last-page length larger than the page, or negative, is clamped exactly as the
    reference's access layer clamps it (python/cleave/dynamic/paging/builders/slab.py:132-142)."""
    inp = cases.gqa_paged_inputs(11, [128, 70, 64], 32, 8, 128, 64, "bf16")
    inp["kv_last_page_len"] = np.array([999, -4, 64], dtype=np.int32)
    out, lse = _run_paged(inp, "bf16", 64)
    want_out, want_lse = orc.gqa_paged_decode(inp["q"], inp["k_cache"], inp["v_cache"], inp["kv_indptr"],
                                              inp["kv_indices"], inp["kv_last_page_len"], inp["sm_scale"])
    assert_close(out, want_out)
    assert_lse_close(lse, want_lse)


def test_named_and_repeat_calls_are_bit_identical():
    """Reference: tests/frontend_dynamic/test_paged_pipeline.py:63-92 (a second call reproduces
    the same bits; the workspace is left clean by every launch)."""
    inp = cases.gqa_paged_inputs(12, [700, 1, 129, 64, 9000], 32, 8, 128, 64, "bf16")
    a = _run_paged(inp, "bf16", 64)
    b = _run_paged(inp, "bf16", 64)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])


@pytest.mark.parametrize("hq,hkv,sq", [(32, 8, 1), (8, 8, 1), (32, 1, 1), (8, 2, 3), (64, 8, 1)])
def test_static_decode_vs_oracle(hq, hkv, sq):
    inp = cases.attention_inputs(5, hq, hkv, sq, 1500, 128, "f16")
    out = _ops().attention_decode(dev(inp["q"], "f16"), dev(inp["k"], "f16"), dev(inp["v"], "f16"))
    assert_close(host(out), orc.attention(inp["q"], inp["k"], inp["v"], "f16"))


def test_static_gqa_decode_full_config_properties():
    """Benchmark configuration 3 at full size (batch 8, 32/8 heads, d 128, KV 8192, fp16): compared with
    the oracle on a sample of kv heads, and invariant under a permutation of the KV positions."""
    g = torch.Generator(device="cpu").manual_seed(0)
    q = torch.randn(8 * 32, 1, 128, generator=g).half()
    k = torch.randn(8 * 8, 8192, 128, generator=g).half()
    v = torch.randn(8 * 8, 8192, 128, generator=g).half()
    ops = _ops()
    out = ops.attention_decode(q.cuda(), k.cuda(), v.cuda())
    perm = torch.randperm(8192, generator=g)
    out_p = ops.attention_decode(q.cuda(), k[:, perm].contiguous().cuda(), v[:, perm].contiguous().cuda())
    assert_close(host(out), host(out_p), rtol=5e-3, atol=5e-3)
    for h in (0, 17, 63):
        want = orc.attention(q[h * 4:(h + 1) * 4].float().numpy(), k[h:h + 1].float().numpy(),
                             v[h:h + 1].float().numpy(), "f16")
        assert_close(host(out[h * 4:(h + 1) * 4]), want)


def test_unsupported_and_bad_arguments_raise():
    from cleave_b200 import Cb200Error

    ops = _ops()
    q = torch.zeros(2, 8, 96, dtype=torch.float16, device="cuda")
    kc = torch.zeros(4, 16, 2, 96, dtype=torch.float16, device="cuda")
    ptr = torch.tensor([0, 1, 2], dtype=torch.int32, device="cuda")
    idx = torch.tensor([0, 1], dtype=torch.int32, device="cuda")
    last = torch.tensor([3, 3], dtype=torch.int32, device="cuda")
    with pytest.raises(Cb200Error):
        ops.gqa_paged_decode(q, kc, kc, ptr, idx, last, 0.1)  # head_dim 96
    with pytest.raises(ValueError):
        ops.gqa_paged_decode(q.cpu(), kc, kc, ptr, idx, last, 0.1)


def test_workspace_shared_by_launches_of_different_shapes():
    """One workspace serves launches of different batch and head counts back to back: the
    arrival counters live at a shape-independent offset, so partials left by a small problem are
    never read as counters by a larger one."""
    small = cases.gqa_paged_inputs(21, [5000, 3000], 8, 2, 128, 64, "bf16")
    large = cases.gqa_paged_inputs(22, [300] * 40 + [9000] * 8, 32, 8, 128, 64, "bf16")
    for inp in (small, large, small, large):
        out, lse = _run_paged(inp, "bf16", 64)
        want_out, want_lse = orc.gqa_paged_decode(inp["q"], inp["k_cache"], inp["v_cache"], inp["kv_indptr"],
                                                  inp["kv_indices"], inp["kv_last_page_len"], inp["sm_scale"])
        assert_close(out, want_out)
        assert_lse_close(lse, want_lse)


@pytest.mark.parametrize("seed,dtype", [(0, torch.float16), (7, torch.float16), (7, torch.bfloat16)])
def test_paged_decode_full_benchmark_config(seed, dtype):
    """Benchmark configuration 5 at full size (batch 128, 32/8 heads, d 128, page 64, lengths uniform in
    [512, 32768]; the seed-0 draw is the one bench.py times, the seed-7 draw holds 2.33 M tokens: a page pool of
    more than 2^31 elements). A request spans up to 512 tiles and every CTA of the grid, and the combine
    merges up to 148 partials. Six requests, the longest and the shortest among them, are compared with the
    oracle over a private pool holding only their pages
    (operator semantics: python/cleave/dynamic/reference.py:180-200)."""
    from cleave_b200.workloads import paged_decode_workload, sub_workload

    ops = _ops()
    w = paged_decode_workload(seed=seed, dtype=dtype)
    out, lse = ops.gqa_paged_decode(*w.args())
    ops.check_workspace(ops.workspace("attn_decode", 0, "cuda"))
    lens = w.kv_lens.tolist()
    picks = sorted({lens.index(max(lens)), lens.index(min(lens)), 0, 41, 86, 127})
    s = sub_workload(w, picks)
    dt = "f16" if dtype == torch.float16 else "bf16"
    want_out, want_lse = orc.gqa_paged_decode(s.q.float().numpy(), s.k_cache.float().numpy(), s.v_cache.float().numpy(),
                                              s.kv_indptr.numpy(), s.kv_indices.numpy(), s.kv_last_page_len.numpy(),
                                              s.sm_scale, out_dtype=dt)
    sel = torch.tensor(picks, device="cuda")
    assert_close(host(out[sel]), want_out)
    assert_lse_close(host(lse[sel]), want_lse)
    del w, out, lse
    torch.cuda.empty_cache()


def test_kv_indptr_beyond_the_page_table_is_clipped():
    """A kv_indptr whose ranges run past the end of kv_indices (caller error, or tables of the wrong width)
    must not make the kernel read outside the table: the range of every request is clipped to the
    ``num_kv_indices`` entries that exist. Requests that lie inside the table are unaffected; the clipped
    one attends over the pages that are really there."""
    lens = [700, 129, 5000, 3000]
    inp = cases.gqa_paged_inputs(31, lens, 32, 8, 128, 64, "bf16")
    full_idx = inp["kv_indices"]
    keep = int(inp["kv_indptr"][3]) + 10           # the last request keeps 10 of its 47 pages
    inp["kv_indices"] = np.ascontiguousarray(full_idx[:keep])
    out, lse = _run_paged(inp, "bf16", 64)
    assert np.isfinite(out).all()
    clipped = dict(inp)
    clipped["kv_indptr"] = np.minimum(inp["kv_indptr"], keep).astype(np.int32)
    want_out, want_lse = orc.gqa_paged_decode(clipped["q"], clipped["k_cache"], clipped["v_cache"], clipped["kv_indptr"],
                                              clipped["kv_indices"], clipped["kv_last_page_len"], clipped["sm_scale"])
    assert_close(out, want_out)
    assert_lse_close(lse, want_lse)
    # a table that claims pages although none exist: every request is empty
    inp["kv_indices"] = np.zeros(0, dtype=np.int32)
    ops = _ops()
    o, l = ops.gqa_paged_decode(dev(inp["q"], "bf16"), dev(inp["k_cache"], "bf16"), dev(inp["v_cache"], "bf16"),
                                dev(inp["kv_indptr"]), torch.zeros(0, dtype=torch.int32, device="cuda"),
                                dev(inp["kv_last_page_len"]), inp["sm_scale"])
    ops.check_workspace(ops.workspace("attn_decode", 0, "cuda"))
    assert (host(o) == 0).all() and np.isneginf(host(l)).all()


def test_wrong_output_buffers_are_refused():
    ops = _ops()
    inp = cases.gqa_paged_inputs(32, [100, 64], 32, 8, 128, 64, "f16")
    args = (dev(inp["q"], "f16"), dev(inp["k_cache"], "f16"), dev(inp["v_cache"], "f16"), dev(inp["kv_indptr"]),
            dev(inp["kv_indices"]), dev(inp["kv_last_page_len"]), inp["sm_scale"])
    good_out = torch.empty_like(args[0])
    good_lse = torch.empty(2, 32, dtype=torch.float32, device="cuda")
    for fn in (ops.gqa_paged_decode, ops.gqa_paged_decode_static_scratch):
        with pytest.raises(ValueError):
            fn(*args, out=torch.empty(2, 32, 64, dtype=torch.float16, device="cuda"), lse=good_lse)
        with pytest.raises(ValueError):
            fn(*args, out=good_out.bfloat16(), lse=good_lse)
        with pytest.raises(ValueError):
            fn(*args, out=good_out, lse=torch.empty(2, 32, dtype=torch.float16, device="cuda"))
        with pytest.raises(TypeError):
            fn(args[0], args[1], args[2], args[3].long(), args[4], args[5], args[6], out=good_out, lse=good_lse)


def test_fault_code_in_a_workspace_reaches_the_host_once():
    """A kernel whose bounded wait gives up writes a fault code into the first word of its workspace. No
    wait is made to run out here: the code is written from the host, which is all the host path can see.
    The check raises status 6, leaves the workspace zero-filled, and the next launch on it is clean."""
    from cleave_b200 import Cb200Error

    ops = _ops()
    inp = cases.gqa_paged_inputs(33, [5000, 300], 32, 8, 128, 64, "bf16")
    _run_paged(inp, "bf16", 64)
    ws = ops.workspace("attn_decode", 0, "cuda")
    ws[:4] = torch.tensor([2, 0, 0, 0], dtype=torch.uint8, device="cuda")   # kFaultEmptyBarrier
    ws[-8:] = 7                                                             # and a dirty arrival counter
    with pytest.raises(Cb200Error) as e:
        ops.check_workspace(ws)
    assert e.value.status == 6
    torch.cuda.synchronize()
    assert int(ws.count_nonzero()) == 0
    ops.check_workspace(ws)
    out, lse = _run_paged(inp, "bf16", 64)
    want_out, want_lse = orc.gqa_paged_decode(inp["q"], inp["k_cache"], inp["v_cache"], inp["kv_indptr"],
                                              inp["kv_indices"], inp["kv_last_page_len"], inp["sm_scale"])
    assert_close(out, want_out)
    assert_lse_close(lse, want_lse)
