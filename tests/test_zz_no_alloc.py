"""The decode entry point that brings its own scratch, for hosts that cannot allocate.

Some callers of this library are not free to call cudaMalloc: a serving process that carved
all device memory into its own arena at start-up and hands out only slices of it, a plugin
host that forbids allocation once it is running, a GPU whose memory is already committed to
the KV cache. For them ``cb200_attn_decode_static_scratch`` keeps the split-KV workspace in a
fixed array inside the library. This file checks, through the C ABI, that it gives the same
answer as the entry point with a caller-owned workspace and as the CPU oracle, twice in a row (the array keeps the
previous call's contents), and that it refuses a problem that does not fit.

The file name sorts last on purpose: a run that stops at the first failure has then already
run every other test.
"""

import ctypes as C

import numpy as np
import pytest
import torch

import cases
from _util import ATOL, RTOL, dev, host
from oracle import cleave_oracle as orc

pytestmark = pytest.mark.gpu


def _both(inp, dt, page_size):
    from cleave_b200 import ops

    last = dev(inp["kv_last_page_len"]) if page_size != 1 else None
    args = (dev(inp["q"], dt), dev(inp["k_cache"], dt), dev(inp["v_cache"], dt), dev(inp["kv_indptr"]),
            dev(inp["kv_indices"]), last, inp["sm_scale"])
    want_out, want_lse = ops.gqa_paged_decode(*args)
    got_out = torch.full_like(want_out, float("nan"))
    got_lse = torch.full_like(want_lse, float("nan"))
    before = torch.cuda.memory_allocated()
    ops.gqa_paged_decode_static_scratch(*args, out=got_out, lse=got_lse)
    ops.check_static_scratch()  # synchronises; raises if a bounded wait of that launch gave up
    assert torch.cuda.memory_allocated() == before  # the call itself allocated nothing through torch
    # and against the CPU oracle, not only against the sibling entry point
    last_np = inp["kv_last_page_len"] if page_size != 1 else None
    orc_out, orc_lse = orc.gqa_paged_decode(inp["q"], inp["k_cache"], inp["v_cache"], inp["kv_indptr"],
                                            inp["kv_indices"], last_np, inp["sm_scale"], out_dtype=dt)
    _check(host(got_out), host(got_lse), orc_out, orc_lse)
    return host(got_out), host(got_lse), host(want_out), host(want_lse)


def _check(got_out, got_lse, want_out, want_lse):
    np.testing.assert_allclose(got_out, want_out, rtol=RTOL, atol=ATOL)
    assert np.array_equal(np.isneginf(got_lse), np.isneginf(want_lse))
    live = ~np.isneginf(want_lse)
    np.testing.assert_allclose(got_lse[live], want_lse[live], rtol=1e-3, atol=2e-3)


def test_static_scratch_matches_workspace_entry_point_twice_in_a_row():
    # long requests are cut across CTAs, so the scratch (partials + arrival counters) is in use
    first = cases.gqa_paged_inputs(51, [9000, 0, 129, 64, 5000, 1], 32, 8, 128, 64, "bf16")
    _check(*_both(first, "bf16", 64))
    # a second call with another shape reuses the array with the first call's leftovers in it
    second = cases.gqa_paged_inputs(52, [300] * 20 + [7000] * 6, 32, 4, 128, 16, "f16")
    _check(*_both(second, "f16", 16))
    _check(*_both(first, "bf16", 64))


def test_static_scratch_refuses_a_problem_that_does_not_fit():
    from cleave_b200 import _lib

    L = _lib.lib()
    cap = L.cb200_attn_decode_static_scratch_max_bytes()
    assert cap == 4 << 20
    a = _lib.AttnDecodeArgs()
    a.batch, a.num_qo_heads, a.num_kv_heads, a.head_dim = 8000, 64, 64, 128  # 512 000 arrival counters
    a.kv_len, a.dtype, a.sm_scale = 64, _lib.F16, 1.0
    assert L.cb200_attn_decode_workspace_bytes(C.byref(a)) > cap
    rc = L.cb200_attn_decode_static_scratch(C.byref(a), None)
    assert rc == 7
    assert b"scratch" in L.cb200_strerror(rc)
