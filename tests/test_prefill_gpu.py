"""GPU parity of the tcgen05 unsplit-attention ("prefill") kernel, through the C ABI, against the
oracle: the reference's fixed-shift static attention without a mask, and the end-aligned causal
mask of its paged / ragged prefill definitions."""

import numpy as np
import pytest
import torch

import cases
from _util import assert_close, assert_lse_close, dev, host
from oracle import cleave_oracle as orc

pytestmark = pytest.mark.gpu


def _ops():
    from cleave_b200 import ops

    return ops


def _check_ws():
    ops = _ops()
    ops.check_workspace(ops.workspace("attn_prefill", 0, "cuda"))


GOLDEN = cases.load_golden()


@pytest.mark.parametrize("name", [n for n, c in cases.CASES.items() if c[0] == "attention" and c[1]["sq"] > 1])
def test_static_prefill_matches_reference_golden(name):
    """Golden outputs of the reference's own torch path (cleave.trace(...).reference) on the seeded case."""
    _, inp, opt = cases.build(name)
    dt = opt["dtype"]
    got = _ops().attention_prefill(dev(inp["q"], dt), dev(inp["k"], dt), dev(inp["v"], dt))
    _check_ws()
    assert_close(host(got), GOLDEN[name][0])


@pytest.mark.parametrize("name", [n for n, c in cases.CASES.items() if c[0] == "gqa_prefill"])
def test_dynamic_prefill_matches_reference_golden(name):
    """Golden outputs of python/cleave/dynamic/reference.py's ragged / paged prefill definitions."""
    _, inp, opt = cases.build(name)
    dt = opt["dtype"]
    qo, kv = torch.from_numpy(inp["qo_indptr"]).cuda(), torch.from_numpy(inp["kv_indptr"]).cuda()
    if opt["paged"]:
        out, lse = _ops().gqa_paged_prefill(dev(inp["q"], dt), dev(inp["k_cache"], dt), dev(inp["v_cache"], dt), qo, kv,
                                            torch.from_numpy(inp["kv_indices"]).cuda(), inp["sm_scale"])
    else:
        out, lse = _ops().gqa_ragged_prefill(dev(inp["q"], dt), dev(inp["k"], dt), dev(inp["v"], dt), qo, kv,
                                             inp["sm_scale"])
    _check_ws()
    assert_close(host(out), GOLDEN[name][0])
    assert_lse_close(host(lse), GOLDEN[name][1])


SHAPES = [  # hq, hkv, sq, skv, d
    (4, 4, 256, 256, 64),     # MHA, whole tiles
    (8, 2, 300, 517, 128),    # GQA, ragged in both lengths
    (4, 1, 130, 1000, 64),    # MQA
    (2, 2, 128, 128, 128),    # a single tile
    (3, 3, 1, 77, 64),        # one query row
    (2, 1, 640, 640, 128),    # five KV tiles: both S and P buffers wrap
    (160, 160, 300, 300, 64),   # more CTAs than SMs; last query tile partly filled
    (152, 8, 300, 517, 128),    # the same with grouped heads and more keys than queries
    (160, 32, 129, 260, 64),    # last query tile holds a single row
]


@pytest.mark.parametrize("dt", ["f16", "bf16"])
@pytest.mark.parametrize("hq,hkv,sq,skv,d", SHAPES)
def test_unmasked_attention_vs_oracle(hq, hkv, sq, skv, d, dt):
    """Reference: demo/attention.py:5-8 (exp(s/sqrt(d) - 50/sqrt(d)) / rowsum)."""
    inp = cases.attention_inputs(hq * 1000 + sq, hq, hkv, sq, skv, d, dt)
    got = _ops().attention_prefill(dev(inp["q"], dt), dev(inp["k"], dt), dev(inp["v"], dt))
    _check_ws()
    assert_close(host(got), orc.attention(inp["q"], inp["k"], inp["v"], dt))


@pytest.mark.parametrize("dt", ["bf16", "f16"])
@pytest.mark.parametrize("hq,hkv,sq,skv,d", [s for s in SHAPES if s[2] <= s[3]])
def test_causal_attention_vs_oracle(hq, hkv, sq, skv, d, dt):
    """Reference: python/cleave/dynamic/reference.py:85-133 (end-aligned causal mask, base-2 lse)."""
    inp = cases.attention_inputs(hq * 1000 + skv, hq, hkv, sq, skv, d, dt)
    scale = d ** -0.5
    lse = torch.empty(hq, sq, dtype=torch.float32, device="cuda")
    got = _ops().attention_prefill(dev(inp["q"], dt), dev(inp["k"], dt), dev(inp["v"], dt), scale, causal=True, lse=lse)
    _check_ws()
    want, want_lse = orc.attention_masked(inp["q"], inp["k"], inp["v"], scale, True, dt)
    assert_close(host(got), want)
    assert_lse_close(host(lse), want_lse)


@pytest.mark.parametrize("hq,hkv,sq,skv,d,dt", [(8, 2, 300, 100, 128, "bf16"), (4, 4, 513, 40, 64, "f16"), (160, 160, 257, 129, 128, "bf16")])
def test_causal_attention_with_more_queries_than_keys(hq, hkv, sq, skv, d, dt):
    """Static layout, end-aligned mask, S_Q > S_KV: the first S_Q - S_KV rows see no key (0 and -inf), whole query
    tiles among them - items the persistent CTAs only write zeros for - and, with 160 heads, more items than SMs."""
    inp = cases.attention_inputs(21, hq, hkv, sq, skv, d, dt)
    lse = torch.empty(hq, sq, dtype=torch.float32, device="cuda")
    scale = d ** -0.5
    got = _ops().attention_prefill(dev(inp["q"], dt), dev(inp["k"], dt), dev(inp["v"], dt), scale, causal=True, lse=lse)
    _check_ws()
    want, want_lse = orc.attention_masked(inp["q"], inp["k"], inp["v"], scale, True, dt)
    assert_close(host(got), want)
    assert_lse_close(host(lse), want_lse)
    assert not host(got)[:, :sq - skv].any() and np.isneginf(host(lse)[:, :sq - skv]).all()


@pytest.mark.parametrize("heads,sq_", [(2, 128), (160, 256)])
def test_large_logits_take_the_rescale_path(heads, sq_):
    """Keys whose norm grows along the sequence push the running maximum up by more than 2^8
    between tiles, so O is rescaled in tensor memory."""
    rng = np.random.default_rng(5)
    hq, sq, skv, d = heads, sq_, 512, 64
    q = cases.round_to(rng.standard_normal((hq, sq, d), dtype=np.float32), "bf16")
    step = (1.0 + 3.0 * (np.arange(skv) // 128))[None, :, None].astype(np.float32)
    k = cases.round_to(rng.standard_normal((hq, skv, d), dtype=np.float32) * step, "bf16")
    v = cases.round_to(rng.standard_normal((hq, skv, d), dtype=np.float32), "bf16")
    lse = torch.empty(hq, sq, dtype=torch.float32, device="cuda")
    got = _ops().attention_prefill(dev(q, "bf16"), dev(k, "bf16"), dev(v, "bf16"), 1.0, lse=lse)
    _check_ws()
    want, want_lse = orc.attention_masked(q, k, v, 1.0, False, "bf16")
    assert_close(host(got), want)
    assert_lse_close(host(lse), want_lse)


@pytest.mark.parametrize("hq,hkv,d,dt", [(8, 2, 128, "bf16"), (4, 4, 64, "f16"), (16, 1, 64, "bf16")])
def test_ragged_causal_prefill_vs_oracle(hq, hkv, d, dt):
    """Reference: python/cleave/dynamic/reference.py:244-278. Requests without queries, without keys,
    with more queries than keys (rows the mask leaves empty), and with several query tiles."""
    q_lens = [100, 0, 128, 5, 257, 30, 1]
    kv_lens = [300, 50, 128, 0, 1000, 20, 129]
    rng = np.random.default_rng(hq * 10 + d)
    tq, tk = sum(q_lens), sum(kv_lens)
    q = cases.round_to(rng.standard_normal((tq, hq, d), dtype=np.float32), dt)
    k = cases.round_to(rng.standard_normal((tk, hkv, d), dtype=np.float32), dt)
    v = cases.round_to(rng.standard_normal((tk, hkv, d), dtype=np.float32), dt)
    qo = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
    kv = np.concatenate([[0], np.cumsum(kv_lens)]).astype(np.int32)
    scale = d ** -0.5
    out, lse = _ops().gqa_ragged_prefill(dev(q, dt), dev(k, dt), dev(v, dt), torch.from_numpy(qo).cuda(),
                                         torch.from_numpy(kv).cuda(), scale)
    _check_ws()
    want, want_lse = orc.gqa_ragged_prefill(q, k, v, qo, kv, scale, dt)
    assert_close(host(out), want)
    assert_lse_close(host(lse), want_lse)


@pytest.mark.parametrize("hq,hkv,d,dt", [(8, 2, 128, "bf16"), (4, 4, 64, "f16")])
def test_paged_causal_prefill_vs_oracle(hq, hkv, d, dt):
    """Reference: python/cleave/dynamic/reference.py:204-241 (one token per page, pages a seeded
    permutation of the pool); the gathered rows must be exactly the indexed ones."""
    q_lens = [100, 0, 128, 5, 257, 1]
    kv_lens = [300, 50, 128, 0, 1000, 129]
    rng = np.random.default_rng(hq + d)
    tq, tk = sum(q_lens), sum(kv_lens)
    num_pages = tk + 37
    q = cases.round_to(rng.standard_normal((tq, hq, d), dtype=np.float32), dt)
    kc = cases.round_to(rng.standard_normal((num_pages, 1, hkv, d), dtype=np.float32), dt)
    vc = cases.round_to(rng.standard_normal((num_pages, 1, hkv, d), dtype=np.float32), dt)
    idx = rng.permutation(num_pages)[:tk].astype(np.int32)
    qo = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
    kv = np.concatenate([[0], np.cumsum(kv_lens)]).astype(np.int32)
    scale = d ** -0.5
    out, lse = _ops().gqa_paged_prefill(dev(q, dt), dev(kc, dt), dev(vc, dt), torch.from_numpy(qo).cuda(),
                                        torch.from_numpy(kv).cuda(), torch.from_numpy(idx).cuda(), scale)
    _check_ws()
    want, want_lse = orc.gqa_paged_prefill(q, kc, vc, qo, kv, idx, scale, dt)
    assert_close(host(out), want)
    assert_lse_close(host(lse), want_lse)
    # the same keys laid out contiguously give bit-identical results: the gather moves rows, nothing else
    out2, lse2 = _ops().gqa_ragged_prefill(dev(q, dt), dev(kc[idx, 0], dt), dev(vc[idx, 0], dt),
                                           torch.from_numpy(qo).cuda(), torch.from_numpy(kv).cuda(), scale)
    assert np.array_equal(host(out), host(out2)) and np.array_equal(host(lse), host(lse2))


def test_paged_prefill_ranges_beyond_the_page_table_are_clipped():
    """Ranges of kv_indptr that run past the entries kv_indices holds are read as shorter requests."""
    hq, hkv, d, dt = 8, 2, 128, "bf16"
    q_lens, kv_lens = [64, 130, 20], [200, 400, 300]
    rng = np.random.default_rng(91)
    tq, tk = sum(q_lens), sum(kv_lens)
    q = cases.round_to(rng.standard_normal((tq, hq, d), dtype=np.float32), dt)
    kc = cases.round_to(rng.standard_normal((tk, 1, hkv, d), dtype=np.float32), dt)
    vc = cases.round_to(rng.standard_normal((tk, 1, hkv, d), dtype=np.float32), dt)
    keep = 200 + 150                       # request 1 keeps 150 of its 400 keys, request 2 none
    idx = rng.permutation(tk)[:keep].astype(np.int32)
    qo = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
    kv = np.concatenate([[0], np.cumsum(kv_lens)]).astype(np.int32)
    scale = d ** -0.5
    out, lse = _ops().gqa_paged_prefill(dev(q, dt), dev(kc, dt), dev(vc, dt), torch.from_numpy(qo).cuda(),
                                        torch.from_numpy(kv).cuda(), torch.from_numpy(idx).cuda(), scale)
    _check_ws()
    want, want_lse = orc.gqa_paged_prefill(q, kc, vc, qo, np.minimum(kv, keep).astype(np.int32), idx, scale, dt)
    assert_close(host(out), want)
    assert_lse_close(host(lse), want_lse)
    assert (host(out)[qo[2]:] == 0).all() and np.isneginf(host(lse)[qo[2]:]).all()


def test_ragged_long_requests():
    """Requests of several hundred query rows on 32 heads: several query tiles per request, more CTAs than SMs."""
    q_lens, kv_lens = [300, 700, 256, 513], [300, 1000, 600, 513]
    hq, hkv, d, dt = 32, 8, 128, "bf16"
    rng = np.random.default_rng(77)
    tq, tk = sum(q_lens), sum(kv_lens)
    q = cases.round_to(rng.standard_normal((tq, hq, d), dtype=np.float32), dt)
    k = cases.round_to(rng.standard_normal((tk, hkv, d), dtype=np.float32), dt)
    v = cases.round_to(rng.standard_normal((tk, hkv, d), dtype=np.float32), dt)
    qo = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
    kv = np.concatenate([[0], np.cumsum(kv_lens)]).astype(np.int32)
    scale = d ** -0.5
    out, lse = _ops().gqa_ragged_prefill(dev(q, dt), dev(k, dt), dev(v, dt), torch.from_numpy(qo).cuda(),
                                         torch.from_numpy(kv).cuda(), scale)
    _check_ws()
    want, want_lse = orc.gqa_ragged_prefill(q, k, v, qo, kv, scale, dt)
    assert_close(host(out), want)
    assert_lse_close(host(lse), want_lse)


@pytest.mark.parametrize("paged", [False, True])
def test_items_dealt_among_persistent_ctas(paged):
    """45 requests (more than the 32 whose ranges a warp keeps in registers) of 0...400 rows on 32 heads: about two
    thousand (head, query tile) items, some of them blind or surplus, for at most 148 CTAs that take them from the
    counter in the workspace header. Three launches on the same workspace must agree bit for bit (the counter clears
    itself) and with the oracle."""
    rng = np.random.default_rng(2024)
    q_lens = [int(x) for x in rng.integers(0, 401, 45)]
    kv_lens = [int(max(0, ql + d)) for ql, d in zip(q_lens, rng.integers(-150, 300, 45))]
    q_lens[7], kv_lens[7] = 130, 0      # rows without any key
    q_lens[20], kv_lens[20] = 300, 40   # leading tiles blind under the end-aligned mask
    hq, hkv, d, dt = 32, 4, 128, "bf16"
    tq, tk = sum(q_lens), sum(kv_lens)
    q = cases.round_to(rng.standard_normal((tq, hq, d), dtype=np.float32), dt)
    qo = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
    kv = np.concatenate([[0], np.cumsum(kv_lens)]).astype(np.int32)
    scale = d ** -0.5
    if paged:
        pool = tk + 11
        kc = cases.round_to(rng.standard_normal((pool, 1, hkv, d), dtype=np.float32), dt)
        vc = cases.round_to(rng.standard_normal((pool, 1, hkv, d), dtype=np.float32), dt)
        idx = rng.permutation(pool)[:tk].astype(np.int32)
        args = (dev(q, dt), dev(kc, dt), dev(vc, dt), torch.from_numpy(qo).cuda(), torch.from_numpy(kv).cuda(),
                torch.from_numpy(idx).cuda(), scale)
        call = _ops().gqa_paged_prefill
        want, want_lse = orc.gqa_paged_prefill(q, kc, vc, qo, kv, idx, scale, dt)
    else:
        k = cases.round_to(rng.standard_normal((tk, hkv, d), dtype=np.float32), dt)
        v = cases.round_to(rng.standard_normal((tk, hkv, d), dtype=np.float32), dt)
        args = (dev(q, dt), dev(k, dt), dev(v, dt), torch.from_numpy(qo).cuda(), torch.from_numpy(kv).cuda(), scale)
        call = _ops().gqa_ragged_prefill
        want, want_lse = orc.gqa_ragged_prefill(q, k, v, qo, kv, scale, dt)
    runs = [tuple(host(x) for x in call(*args)) for _ in range(3)]
    _check_ws()
    assert_close(runs[0][0], want)
    assert_lse_close(runs[0][1], want_lse)
    for out, lse in runs[1:]:
        assert np.array_equal(out, runs[0][0]) and np.array_equal(lse, runs[0][1])


@pytest.mark.parametrize("paged", [False, True])
@pytest.mark.parametrize("kv_len", [1, 7, 8, 9, 33, 63, 64, 65, 127, 129])
def test_single_small_item_key_boundaries(paged, kv_len):
    """One request with a few query rows: the call has fewer items than SMs and takes the kernel's one-item form, in
    which half tiles of scores no row of a warp sees are skipped and, in the paged layout, rounds of eight rows past the
    last key are zero-filled in shared memory instead of fetched. Key counts on both sides of those boundaries; a launch
    over NaN caches runs first, so stale shared memory would show."""
    hq, hkv, d, dt = 32, 4, 128, "bf16"
    q_len = min(3, kv_len)
    rng = np.random.default_rng(kv_len)
    q = cases.round_to(rng.standard_normal((q_len, hq, d), dtype=np.float32), dt)
    qo = np.array([0, q_len], dtype=np.int32)
    kv = np.array([0, kv_len], dtype=np.int32)
    scale = d ** -0.5
    if paged:
        pool = kv_len + 5
        kc = cases.round_to(rng.standard_normal((pool, 1, hkv, d), dtype=np.float32), dt)
        vc = cases.round_to(rng.standard_normal((pool, 1, hkv, d), dtype=np.float32), dt)
        idx = rng.permutation(pool)[:kv_len].astype(np.int32)
        args = [dev(q, dt), dev(kc, dt), dev(vc, dt), torch.from_numpy(qo).cuda(), torch.from_numpy(kv).cuda(),
                torch.from_numpy(idx).cuda(), scale]
        call = _ops().gqa_paged_prefill
        want, want_lse = orc.gqa_paged_prefill(q, kc, vc, qo, kv, idx, scale, dt)
    else:
        k = cases.round_to(rng.standard_normal((kv_len, hkv, d), dtype=np.float32), dt)
        v = cases.round_to(rng.standard_normal((kv_len, hkv, d), dtype=np.float32), dt)
        args = [dev(q, dt), dev(k, dt), dev(v, dt), torch.from_numpy(qo).cuda(), torch.from_numpy(kv).cuda(), scale]
        call = _ops().gqa_ragged_prefill
        want, want_lse = orc.gqa_ragged_prefill(q, k, v, qo, kv, scale, dt)
    poisoned = list(args)
    poisoned[1], poisoned[2] = torch.full_like(args[1], float("nan")), torch.full_like(args[2], float("nan"))
    call(*poisoned)
    out, lse = call(*args)
    _check_ws()
    assert_close(host(out), want)
    assert_lse_close(host(lse), want_lse)


def test_repeat_launches_are_bit_identical():
    inp = cases.attention_inputs(9, 8, 2, 300, 517, 128, "f16")
    q, k, v = (dev(inp[n], "f16") for n in ("q", "k", "v"))
    a = host(_ops().attention_prefill(q, k, v, causal=True))
    b = host(_ops().attention_prefill(q, k, v, causal=True))
    assert np.array_equal(a, b)


def test_full_demo_shape_properties():
    """demo/gqa_prefill.py at full size (32 / 8 heads, S_Q = S_KV = 4096, D 64, fp16): with V = 1 every
    output is 1 (the weights of a row sum to one), and sampled rows match the oracle."""
    g = torch.Generator(device="cpu").manual_seed(0)
    hq, hkv, s, d = 32, 8, 4096, 64
    q = torch.randn(hq, s, d, generator=g).half()
    k = torch.randn(hkv, s, d, generator=g).half()
    v = torch.randn(hkv, s, d, generator=g).half()
    ops = _ops()
    ones = ops.attention_prefill(q.cuda(), k.cuda(), torch.ones_like(v).cuda(), causal=True)
    np.testing.assert_allclose(host(ones), 1.0, rtol=0, atol=4e-3)
    out = host(ops.attention_prefill(q.cuda(), k.cuda(), v.cuda(), causal=True))
    _check_ws()
    rows = np.array([0, 1, 127, 128, 2047, 3000, 4095])
    for h in (0, 13, 31):
        hk = h // (hq // hkv)
        logits = (q[h, rows].float() @ k[hk].float().T).numpy() * np.float32(d ** -0.5)
        logits = np.where(np.arange(s)[None, :] <= rows[:, None], logits, -np.inf).astype(np.float32)
        w, _ = orc._finish(logits)
        assert_close(out[h, rows], cases.round_to(w @ v[hk].float().numpy(), "f16"))


def test_prefill_bad_arguments():
    from cleave_b200 import Cb200Error

    ops = _ops()
    q = torch.zeros(2, 64, 96, dtype=torch.float16, device="cuda")
    k = torch.zeros(2, 64, 96, dtype=torch.float16, device="cuda")
    with pytest.raises(Cb200Error):
        ops.attention_prefill(q, k, k)  # head_dim 96
    q = torch.zeros(2, 64, 64, dtype=torch.float32, device="cuda")
    with pytest.raises((Cb200Error, ValueError, TypeError)):
        ops.attention_prefill(q, q, q)  # fp32 inputs
