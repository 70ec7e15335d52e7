"""Seeded input builders shared by the golden-vector generator and the tests.

Inputs are regenerated from the seed on both sides, so only the reference's OUTPUTS are
stored in ``golden.npz``. Every array is float32 holding values exactly representable in
the case's storage dtype; integer tables are int32.
"""

from __future__ import annotations

import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "..", ".."))
from oracle.cleave_oracle import round_to  # noqa: E402


def _randn(rng, shape, dtype, scale=1.0):
    return round_to(rng.standard_normal(shape, dtype=np.float32) * np.float32(scale), dtype)


def gemm_inputs(seed, m, n, k, dtype, n_w=1, gamma=False):
    rng = np.random.default_rng(seed)
    out = {"x": _randn(rng, (m, k), dtype)}
    for i in range(n_w):
        out[f"w{i}"] = _randn(rng, (k, n), dtype, 1.0 / np.sqrt(k))
    if gamma:
        out["gamma"] = round_to(1.0 + 0.1 * rng.standard_normal((k,), dtype=np.float32), dtype)
    return out


def attention_inputs(seed, hq, hkv, sq, skv, d, dtype):
    rng = np.random.default_rng(seed)
    return {"q": _randn(rng, (hq, sq, d), dtype), "k": _randn(rng, (hkv, skv, d), dtype),
            "v": _randn(rng, (hkv, skv, d), dtype)}


def matmul_matmul_inputs(seed, hq, hkv, sq, skv, d, dtype):
    """v is scaled by 1/sqrt(SKV * D) so that the output is O(1): the scores (magnitude sqrt(D)) are a
    16-bit operand of the second product on the GPU and their rounding must stay inside the absolute
    tolerance of the comparison."""
    rng = np.random.default_rng(seed)
    return {"q": _randn(rng, (hq, sq, d), dtype), "k": _randn(rng, (hkv, skv, d), dtype),
            "v": _randn(rng, (hkv, skv, d), dtype, 1.0 / np.sqrt(skv * d))}


def lora_inputs(seed, m, n, k, r, dtype):
    rng = np.random.default_rng(seed)
    return {"x": _randn(rng, (m, k), dtype), "w": _randn(rng, (k, n), dtype, 1.0 / np.sqrt(k)),
            "a": _randn(rng, (k, r), dtype, 1.0 / np.sqrt(k)), "b": _randn(rng, (r, n), dtype, 1.0 / np.sqrt(r))}


def mla_inputs(seed, b, h, skv, d, pe, dtype):
    rng = np.random.default_rng(seed)
    return {"q": _randn(rng, (b, h, d), dtype), "kv": _randn(rng, (b, skv, d), dtype),
            "q_pe": _randn(rng, (b, h, pe), dtype), "k_pe": _randn(rng, (b, skv, pe), dtype)}


def page_tables(rng, kv_lens, page_size, spare_pages=3):
    pages = [-(-n // page_size) for n in kv_lens]
    num_pages = sum(pages) + spare_pages
    perm = rng.permutation(num_pages).astype(np.int32)
    kv_indices = perm[:sum(pages)]
    kv_indptr = np.concatenate([[0], np.cumsum(pages)]).astype(np.int32)
    last = np.array([n - (p - 1) * page_size if p else 0 for n, p in zip(kv_lens, pages)], dtype=np.int32)
    return num_pages, kv_indptr, kv_indices, last


def gqa_paged_inputs(seed, kv_lens, hq, hkv, d, page_size, dtype):
    rng = np.random.default_rng(seed)
    num_pages, kv_indptr, kv_indices, last = page_tables(rng, kv_lens, page_size)
    return {"q": _randn(rng, (len(kv_lens), hq, d), dtype),
            "k_cache": _randn(rng, (num_pages, page_size, hkv, d), dtype),
            "v_cache": _randn(rng, (num_pages, page_size, hkv, d), dtype),
            "kv_indptr": kv_indptr, "kv_indices": kv_indices, "kv_last_page_len": last,
            "sm_scale": float(d) ** -0.5}


def mla_paged_inputs(seed, kv_lens, h, ckv, kpe, dtype, scale):
    rng = np.random.default_rng(seed)
    num_pages, kv_indptr, kv_indices, _ = page_tables(rng, kv_lens, 1)
    return {"q_nope": _randn(rng, (len(kv_lens), h, ckv), dtype),
            "q_pe": _randn(rng, (len(kv_lens), h, kpe), dtype),
            "ckv_cache": _randn(rng, (num_pages, 1, ckv), dtype),
            "kpe_cache": _randn(rng, (num_pages, 1, kpe), dtype),
            "kv_indptr": kv_indptr, "kv_indices": kv_indices, "sm_scale": float(scale)}


def gqa_prefill_inputs(seed, q_lens, kv_lens, hq, hkv, d, dtype, paged):
    """Ragged (``paged=False``) or page-size-1 paged causal prefill, argument for argument as
    python/cleave/dynamic/reference.py:204-258 lays them out."""
    rng = np.random.default_rng(seed)
    tq, tk = sum(q_lens), sum(kv_lens)
    out = {"q": _randn(rng, (tq, hq, d), dtype),
           "qo_indptr": np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32),
           "kv_indptr": np.concatenate([[0], np.cumsum(kv_lens)]).astype(np.int32),
           "sm_scale": float(d) ** -0.5}
    if paged:
        num_pages = tk + 5
        out["k_cache"] = _randn(rng, (num_pages, 1, hkv, d), dtype)
        out["v_cache"] = _randn(rng, (num_pages, 1, hkv, d), dtype)
        out["kv_indices"] = rng.permutation(num_pages)[:tk].astype(np.int32)
    else:
        out["k"] = _randn(rng, (tk, hkv, d), dtype)
        out["v"] = _randn(rng, (tk, hkv, d), dtype)
    return out


def mla_prefill_inputs(seed, q_lens, kv_lens, h, ckv, kpe, dtype, scale):
    """Paged causal MLA prefill, argument for argument as python/cleave/dynamic/reference.py:323-338."""
    rng = np.random.default_rng(seed)
    tq, tk = sum(q_lens), sum(kv_lens)
    num_pages = tk + 4
    return {"q_nope": _randn(rng, (tq, h, ckv), dtype), "q_pe": _randn(rng, (tq, h, kpe), dtype),
            "ckv_cache": _randn(rng, (num_pages, 1, ckv), dtype), "kpe_cache": _randn(rng, (num_pages, 1, kpe), dtype),
            "qo_indptr": np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32),
            "kv_indptr": np.concatenate([[0], np.cumsum(kv_lens)]).astype(np.int32),
            "kv_indices": rng.permutation(num_pages)[:tk].astype(np.int32), "sm_scale": float(scale)}


MLA_SM_SCALE = 0.1352337747812271

# name -> (family, builder kwargs)
CASES = {
    # dense GEMM family
    "matmul_f16": ("matmul", dict(seed=1, m=128, n=128, k=512, dtype="f16")),
    "matmul_bf16_ragged": ("matmul", dict(seed=2, m=40, n=72, k=320, dtype="bf16")),
    "rmsnorm_matmul_f16": ("rmsnorm_matmul", dict(seed=3, m=64, n=256, k=512, dtype="f16"), dict(eps=0.0)),
    "rmsnorm_matmul_eps_f16": ("rmsnorm_matmul", dict(seed=4, m=64, n=256, k=512, dtype="f16"), dict(eps=1e-6)),
    "rmsnorm_matmul_gamma_f16": ("rmsnorm_matmul", dict(seed=5, m=64, n=256, k=512, dtype="f16", gamma=True),
                                 dict(eps=1e-6)),
    "swiglu_f16": ("swiglu", dict(seed=6, m=128, n=256, k=512, dtype="f16", n_w=2)),
    # static decode attention, SQ = 1
    "gqa_decode_f16": ("attention", dict(seed=10, hq=32, hkv=8, sq=1, skv=1000, d=128, dtype="f16")),
    "mha_decode_f16": ("attention", dict(seed=11, hq=8, hkv=8, sq=1, skv=333, d=128, dtype="f16")),
    "mqa_decode_bf16": ("attention", dict(seed=12, hq=16, hkv=1, sq=1, skv=777, d=128, dtype="bf16")),
    "gqa_decode_d64_f16": ("attention", dict(seed=13, hq=16, hkv=4, sq=1, skv=500, d=64, dtype="f16")),
    # static MLA decode
    "mla_decode_bf16": ("mla", dict(seed=20, b=1, h=128, skv=300, d=512, pe=64, dtype="bf16"),
                        dict(scale=192 ** -0.5)),
    "mla_decode_h16_bf16": ("mla", dict(seed=21, b=3, h=16, skv=130, d=512, pe=64, dtype="bf16"),
                            dict(scale=MLA_SM_SCALE)),
    # paged GQA decode (lengths follow the reference's own end-to-end and empty-request tests)
    "gqa_paged_ps64_bf16": ("gqa_paged", dict(seed=30, kv_lens=[700, 1, 129, 64], hq=32, hkv=8, d=128,
                                              page_size=64, dtype="bf16")),
    "gqa_paged_ps1_bf16": ("gqa_paged", dict(seed=31, kv_lens=[700, 1, 129, 64], hq=32, hkv=8, d=128,
                                             page_size=1, dtype="bf16")),
    "gqa_paged_ps64_empty_bf16": ("gqa_paged", dict(seed=32, kv_lens=[5, 0, 7], hq=32, hkv=8, d=128,
                                                    page_size=64, dtype="bf16")),
    "gqa_paged_ps1_empty_kv4_bf16": ("gqa_paged", dict(seed=33, kv_lens=[5, 0, 7], hq=32, hkv=4, d=128,
                                                       page_size=1, dtype="bf16")),
    "gqa_paged_ps16_f16": ("gqa_paged", dict(seed=34, kv_lens=[100, 33, 16, 250], hq=32, hkv=8, d=128,
                                             page_size=16, dtype="f16")),
    # unsplit static attention with many query rows (demo/{mha,gqa}_prefill.py at test size)
    "gqa_prefill_d64_f16": ("attention", dict(seed=14, hq=8, hkv=2, sq=130, skv=130, d=64, dtype="f16")),
    "mha_prefill_d128_bf16": ("attention", dict(seed=15, hq=2, hkv=2, sq=200, skv=333, d=128, dtype="bf16")),
    # ragged / paged causal prefill (requests without queries, without keys, with several query tiles)
    "gqa_ragged_prefill_bf16": ("gqa_prefill", dict(seed=50, q_lens=[100, 0, 128, 5, 257], kv_lens=[300, 50, 128, 0, 600],
                                                    hq=8, hkv=2, d=128, dtype="bf16", paged=False)),
    "gqa_paged_prefill_bf16": ("gqa_prefill", dict(seed=51, q_lens=[100, 0, 128, 5, 257], kv_lens=[300, 50, 128, 0, 600],
                                                   hq=8, hkv=2, d=64, dtype="bf16", paged=True)),
    "mla_paged_prefill_bf16": ("mla_prefill", dict(seed=52, q_lens=[20, 0, 30, 5, 1], kv_lens=[70, 30, 30, 0, 129], h=16,
                                                  ckv=512, kpe=64, dtype="bf16", scale=MLA_SM_SCALE)),
    # the remaining fused operators of the reference's demo set
    "mha_decode_exact_f16": ("attention_exact", dict(seed=60, hq=4, hkv=4, sq=64, skv=256, d=64, dtype="f16")),
    "matmul_matmul_f16": ("matmul_matmul", dict(seed=61, hq=4, hkv=4, sq=130, skv=300, d=64, dtype="f16")),
    "matmul_matmul_gqa_bf16": ("matmul_matmul", dict(seed=62, hq=4, hkv=2, sq=64, skv=256, d=128, dtype="bf16")),
    "qknorm_f16": ("qknorm", dict(seed=63, hq=8, hkv=2, sq=200, skv=333, d=128, dtype="f16"), dict(eps=1e-6)),
    "qknorm_d64_bf16": ("qknorm", dict(seed=64, hq=4, hkv=4, sq=128, skv=128, d=64, dtype="bf16"), dict(eps=1e-6)),
    "matmul_rowsum_f16": ("matmul_rowsum", dict(seed=65, m=200, n=512, k=64, dtype="f16")),
    "matmul_rowsum_bf16": ("matmul_rowsum", dict(seed=66, m=33, n=72, k=320, dtype="bf16")),
    "lora_f16": ("lora", dict(seed=67, m=16, n=512, k=1024, r=16, dtype="f16")),
    "lora_bf16": ("lora", dict(seed=68, m=200, n=264, k=320, r=8, dtype="bf16")),
    # paged MLA decode
    "mla_paged_bf16": ("mla_paged", dict(seed=40, kv_lens=[5, 0, 7, 300], h=16, ckv=512, kpe=64,
                                         dtype="bf16", scale=MLA_SM_SCALE)),
}


def build(name):
    entry = CASES[name]
    family, kw = entry[0], entry[1]
    extra = entry[2] if len(entry) > 2 else {}
    if family in ("matmul", "rmsnorm_matmul", "swiglu"):
        return family, gemm_inputs(**kw), dict(extra, dtype=kw["dtype"])
    if family in ("attention", "attention_exact", "qknorm"):
        return family, attention_inputs(**kw), dict(extra, dtype=kw["dtype"])
    if family == "matmul_matmul":
        return family, matmul_matmul_inputs(**kw), dict(extra, dtype=kw["dtype"])
    if family == "matmul_rowsum":
        return family, gemm_inputs(**kw), dict(extra, dtype=kw["dtype"])
    if family == "lora":
        return family, lora_inputs(**kw), dict(extra, dtype=kw["dtype"])
    if family == "mla":
        return family, mla_inputs(**kw), dict(extra, dtype=kw["dtype"])
    if family == "gqa_paged":
        return family, gqa_paged_inputs(**kw), dict(extra, dtype=kw["dtype"], page_size=kw["page_size"],
                                                    kv_lens=kw["kv_lens"])
    if family == "mla_paged":
        return family, mla_paged_inputs(**kw), dict(extra, dtype=kw["dtype"], kv_lens=kw["kv_lens"])
    if family == "mla_prefill":
        return family, mla_prefill_inputs(**kw), dict(extra, dtype=kw["dtype"], q_lens=kw["q_lens"], kv_lens=kw["kv_lens"])
    if family == "gqa_prefill":
        return family, gqa_prefill_inputs(**kw), dict(extra, dtype=kw["dtype"], q_lens=kw["q_lens"],
                                                      kv_lens=kw["kv_lens"], paged=kw["paged"])
    raise KeyError(family)


def load_golden(path=None):
    """``{case: [float32 arrays]}`` decoded from ``golden.npz``."""
    path = path or os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden.npz")
    raw = np.load(path)
    out = {}
    for key in raw.files:
        ident, kind = key.rsplit(":", 1)
        name, idx = ident.rsplit("/", 1)
        a = raw[key]
        if kind == "bf16":
            a = (a.astype(np.uint32) << 16).view(np.float32)
        else:
            a = a.astype(np.float32)
        out.setdefault(name, {})[int(idx)] = a
    return {k: [v[i] for i in sorted(v)] for k, v in out.items()}
