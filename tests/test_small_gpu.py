"""Causal prefill whose key window is far shorter than its run of query rows (cleave_b200/csrc/small_attn.cu): the
operators hand such calls to one CTA per row that sees a key and one warp per row that sees none. Parity with the
oracle through the same public calls, on the shapes of the reference's captured chunks of that kind
(python/cleave/dynamic/workloads.py): a long query run over a page table of one token, dozens of requests with a few
keys each (more requests than the 32 a step of the row search covers), requests with more keys than rows beside
requests with none. The tcgen05 kernels are run on the same inputs; both must be within the operators' tolerance of
the fp32 reference."""

import numpy as np
import pytest
import torch

import cases
from _util import assert_close, assert_lse_close, dev, host
from oracle import cleave_oracle as orc

pytestmark = [pytest.mark.gpu, pytest.mark.small_kernels]


def _ops():
    from cleave_b200 import ops

    return ops


MANY_Q = [40] * 70
MANY_KV = [(3 * i) % 5 for i in range(70)]

GQA_CASES = [([1210], [1], 32, 4, 128, "bf16"),
             ([500, 0, 300, 7, 64], [2, 5, 30, 40, 20], 32, 8, 128, "bf16"),
             (MANY_Q, MANY_KV, 32, 8, 128, "f16"),
             ([900, 3], [90, 0], 8, 2, 64, "f16"),
             ([2100], [256], 32, 4, 128, "bf16")]


@pytest.mark.parametrize("paged", [False, True])
@pytest.mark.parametrize("q_lens,kv_lens,hq,hkv,d,dt", GQA_CASES)
def test_short_window_causal_prefill(paged, q_lens, kv_lens, hq, hkv, d, dt):
    """Rows before the last min(q_len, kv_len) of a request are 0 / -inf; the others see a growing prefix."""
    rng = np.random.default_rng(7)
    tq, tk = sum(q_lens), sum(kv_lens)
    assert 8 * tk <= tq and tk <= 256  # what the operators ask before they take the light kernels
    q = cases.round_to(rng.standard_normal((tq, hq, d), dtype=np.float32), dt)
    qo = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
    kv = np.concatenate([[0], np.cumsum(kv_lens)]).astype(np.int32)
    scale = d ** -0.5
    ops = _ops()
    if paged:
        pool = tk + 9
        kc = cases.round_to(rng.standard_normal((pool, 1, hkv, d), dtype=np.float32), dt)
        vc = cases.round_to(rng.standard_normal((pool, 1, hkv, d), dtype=np.float32), dt)
        idx = rng.permutation(pool)[:tk].astype(np.int32)
        args = (dev(q, dt), dev(kc, dt), dev(vc, dt), torch.from_numpy(qo).cuda(), torch.from_numpy(kv).cuda(),
                torch.from_numpy(idx).cuda(), scale)
        call = ops.gqa_paged_prefill
        want, want_lse = orc.gqa_paged_prefill(q, kc, vc, qo, kv, idx, scale, dt)
    else:
        k = cases.round_to(rng.standard_normal((tk, hkv, d), dtype=np.float32), dt)
        v = cases.round_to(rng.standard_normal((tk, hkv, d), dtype=np.float32), dt)
        args = (dev(q, dt), dev(k, dt), dev(v, dt), torch.from_numpy(qo).cuda(), torch.from_numpy(kv).cuda(), scale)
        call = ops.gqa_ragged_prefill
        want, want_lse = orc.gqa_ragged_prefill(q, k, v, qo, kv, scale, dt)
    out, lse = call(*args)
    assert_close(host(out), want)
    assert_lse_close(host(lse), want_lse)
    ops.set_small_problem_limit(0)  # the tcgen05 kernel on the same inputs
    out_t, lse_t = call(*args)
    assert_close(host(out_t), want)
    assert_lse_close(host(lse_t), want_lse)


def test_light_kernels_overwrite_every_row():
    """Every row of the output is written by one of the two kernels, whatever it held before: run twice over an output
    buffer, first poisoned, and compare."""
    ops = _ops()
    rng = np.random.default_rng(11)
    q_lens, kv_lens, hq, hkv, d, dt = [300, 120, 0, 50], [7, 0, 3, 50], 32, 8, 128, "bf16"
    tq, tk = sum(q_lens), sum(kv_lens)
    q = cases.round_to(rng.standard_normal((tq, hq, d), dtype=np.float32), dt)
    k = cases.round_to(rng.standard_normal((tk, hkv, d), dtype=np.float32), dt)
    v = cases.round_to(rng.standard_normal((tk, hkv, d), dtype=np.float32), dt)
    qo = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
    kv = np.concatenate([[0], np.cumsum(kv_lens)]).astype(np.int32)
    want, want_lse = orc.gqa_ragged_prefill(q, k, v, qo, kv, d ** -0.5, dt)
    for _ in range(3):
        torch.empty(tq * hq * d * 4, dtype=torch.bfloat16, device="cuda").fill_(float("nan"))  # dirty the allocator's blocks
        out, lse = ops.gqa_ragged_prefill(dev(q, dt), dev(k, dt), dev(v, dt), torch.from_numpy(qo).cuda(), torch.from_numpy(kv).cuda(),
                                          d ** -0.5)
        assert_close(host(out), want)
        assert_lse_close(host(lse), want_lse)


@pytest.mark.parametrize("q_lens,kv_lens,dt", [([400, 9], [3, 9], "bf16"), (MANY_Q, MANY_KV, "bf16"), ([300], [30], "f16"),
                                               ([150, 0, 600, 5, 1], [7, 30, 30, 0, 20], "f16")])
def test_short_window_paged_mla_prefill(q_lens, kv_lens, dt):
    """Against the oracle, and against the tile kernel on the same inputs (both within the operator's tolerance)."""
    ops = _ops()
    assert 8 * sum(kv_lens) <= sum(q_lens)
    inp = cases.mla_prefill_inputs(303, q_lens, kv_lens, 16, 512, 64, dt, cases.MLA_SM_SCALE)
    args = (dev(inp["q_nope"], dt), dev(inp["q_pe"], dt), dev(inp["ckv_cache"], dt), dev(inp["kpe_cache"], dt), dev(inp["qo_indptr"]),
            dev(inp["kv_indptr"]), dev(inp["kv_indices"]), inp["sm_scale"])
    out, lse = ops.mla_paged_prefill(*args)
    want, want_lse = orc.mla_paged_prefill(inp["q_nope"], inp["q_pe"], inp["ckv_cache"], inp["kpe_cache"], inp["qo_indptr"],
                                           inp["kv_indptr"], inp["kv_indices"], inp["sm_scale"], dt)
    assert_close(host(out), want)
    assert_lse_close(host(lse), want_lse)
    ops.set_small_problem_limit(0)
    out_t, lse_t = ops.mla_paged_prefill(*args)
    assert_close(host(out_t), want)
    assert_lse_close(host(lse_t), want_lse)
