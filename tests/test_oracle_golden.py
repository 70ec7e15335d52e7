"""The numpy oracle against golden outputs produced by the reference's own torch code."""

import numpy as np
import pytest

import cases
from oracle import cleave_oracle as orc

GOLDEN = cases.load_golden()

# One unit in the last place of the 16-bit storage type: the oracle and the reference both
# compute in fp32 but sum in different orders, so a value on a rounding boundary may land on
# either neighbour.
ULP = {"f16": 2.0 ** -10, "bf16": 2.0 ** -7}


def _close(got, want, dtype):
    np.testing.assert_allclose(got, want, rtol=ULP[dtype], atol=ULP[dtype] * 1e-2 + 1e-6)


def _run(name):
    family, inp, opt = cases.build(name)
    dt = opt["dtype"]
    if family == "matmul":
        return [orc.matmul(inp["x"], inp["w0"], dt)]
    if family == "rmsnorm_matmul":
        return [orc.rmsnorm_matmul(inp["x"], inp["w0"], opt["eps"], inp.get("gamma"), dt)]
    if family == "swiglu":
        return [orc.swiglu(inp["x"], inp["w0"], inp["w1"], dt)]
    if family == "attention":
        return [orc.attention(inp["q"], inp["k"], inp["v"], dt)]
    if family == "attention_exact":
        return [orc.attention_exact(inp["q"], inp["k"], inp["v"], dt)]
    if family == "matmul_matmul":
        return [orc.matmul_matmul(inp["q"], inp["k"], inp["v"], dt)]
    if family == "qknorm":
        return [orc.qknorm_attention(inp["q"], inp["k"], inp["v"], opt["eps"], dt)]
    if family == "matmul_rowsum":
        return [orc.matmul_rowsum(inp["x"], inp["w0"], dt)]
    if family == "lora":
        return [orc.lora(inp["x"], inp["w"], inp["a"], inp["b"], dt)]
    if family == "mla":
        return [orc.mla_decode(inp["q"], inp["kv"], inp["q_pe"], inp["k_pe"], opt["scale"], dt)]
    if family == "gqa_paged":
        last = inp["kv_last_page_len"] if opt["page_size"] != 1 else None
        return list(orc.gqa_paged_decode(inp["q"], inp["k_cache"], inp["v_cache"], inp["kv_indptr"],
                                         inp["kv_indices"], last, inp["sm_scale"]))
    if family == "mla_paged":
        return list(orc.mla_paged_decode(inp["q_nope"], inp["q_pe"], inp["ckv_cache"], inp["kpe_cache"],
                                         inp["kv_indptr"], inp["kv_indices"], inp["sm_scale"]))
    if family == "mla_prefill":
        return list(orc.mla_paged_prefill(inp["q_nope"], inp["q_pe"], inp["ckv_cache"], inp["kpe_cache"], inp["qo_indptr"],
                                          inp["kv_indptr"], inp["kv_indices"], inp["sm_scale"]))
    if family == "gqa_prefill":
        if opt["paged"]:
            return list(orc.gqa_paged_prefill(inp["q"], inp["k_cache"], inp["v_cache"], inp["qo_indptr"],
                                              inp["kv_indptr"], inp["kv_indices"], inp["sm_scale"]))
        return list(orc.gqa_ragged_prefill(inp["q"], inp["k"], inp["v"], inp["qo_indptr"], inp["kv_indptr"],
                                           inp["sm_scale"]))
    raise KeyError(family)


@pytest.mark.parametrize("name", sorted(cases.CASES))
def test_oracle_matches_reference_golden(name):
    family, _, opt = cases.build(name)
    got = _run(name)
    want = GOLDEN[name]
    assert len(got) == len(want)
    out_dt = "bf16" if family in ("gqa_paged", "mla_paged", "gqa_prefill", "mla_prefill") else opt["dtype"]
    _close(got[0].reshape(want[0].shape), want[0], out_dt)
    if len(want) > 1:  # base-2 lse, fp32
        assert np.array_equal(np.isneginf(got[1]), np.isneginf(want[1]))
        live = ~np.isneginf(want[1])
        np.testing.assert_allclose(got[1][live], want[1][live], rtol=1e-5, atol=1e-5)


def test_empty_request_is_zero_and_neg_inf():
    # reference: tests/graph/handwritten/test_empty_request.py:37-39 (DECODE_KV_LENS = [5, 0, 7])
    out, lse = GOLDEN["gqa_paged_ps64_empty_bf16"]
    assert np.all(out[1] == 0) and np.all(np.isneginf(lse[1]))
    got = _run("gqa_paged_ps64_empty_bf16")
    assert np.all(got[0][1] == 0) and np.all(np.isneginf(got[1][1]))


def test_valid_len_clamp():
    # reference: python/cleave/dynamic/paging/builders/slab.py:132-142
    ptr = np.array([0, 3, 3, 4, 6], dtype=np.int32)
    last = np.array([10, 5, 0, 999], dtype=np.int32)
    v = orc.valid_len(ptr, last, 64)
    assert v.tolist() == [2 * 64 + 10, 0, 0, 128]
    assert orc.valid_len(ptr, None, 1).tolist() == [3, 0, 1, 2]


@pytest.mark.parametrize("valid,split", [(0, 8), (1, 8), (64, 4), (65, 4), (1000, 8), (8192, 16), (513, 3)])
def test_split_ranges_partition_every_tile_once(valid, split):
    # reference: python/cleave/dynamic/paging/stages.py:331-347 ("every KV tile owned by exactly one split")
    tile = 64
    owned = []
    for tile0, trip, end in orc.split_ranges(valid, tile, split):
        owned += list(range(tile0, tile0 + trip))
        assert end <= valid
    assert owned == list(range(-(-valid // tile)))


def test_bf16_round_is_nearest_even():
    import torch

    x = np.random.default_rng(0).standard_normal(10000).astype(np.float32) * 100
    want = torch.from_numpy(x).to(torch.bfloat16).float().numpy()
    assert np.array_equal(orc.round_bf16(x), want)
