"""CPU oracle: a numpy restatement of the reference's torch fp32 semantics for the fused
operators this library implements on the GPU.

THIS IS TEST INFRASTRUCTURE. Only the test-suite, the smoke check and the benchmark's CPU
baseline import it; no product code path may route through it.

Every function restates one reference definition (paths are relative to the reference
project root):

* ``matmul``            - ``python/cleave/frontend/program.py:296-321`` (``Program.reference``:
                          inputs ``.float()``, eager fp32 ops, output cast to the program dtype)
                          applied to ``demo/matmul.py:11-13``.
* ``rmsnorm_matmul``    - ``python/cleave/frontend/composites.py:48-53`` (``x * rsqrt(mean(x*x)+eps)``)
                          followed by ``@ w`` (``demo/rmsnorm_matmul.py:11-13``).
* ``swiglu``            - ``demo/swiglu.py:6-10``.
* ``attention``         - ``demo/attention.py:5-8`` with ``composites.softmax`` (``:56-64``, fixed
                          shift ``-50/sqrt(d)``) and the grouped batch broadcast of
                          ``frontend/program.py:351-363`` (``repeat_interleave``).
* ``mla_decode``        - ``demo/mla_decode.py:8-13`` with a caller-chosen scale.
* ``attention_exact``   - ``demo/attention.py:11-13`` (``exp(s - max(s)) / sum``; ``demo/mha_decode_exact.py``).
* ``matmul_matmul``     - ``demo/matmul_matmul.py:11-13`` (``(q @ k.mT) @ v``).
* ``qknorm_attention``  - ``demo/qknorm.py:17-24`` (``x * rsqrt(mean(x*x) + eps)`` on q and k, then ``attention``).
* ``matmul_rowsum``     - ``demo/matmul_rowsum.py:6-8`` (``(x @ w).sum(-1, keepdim=True)``).
* ``lora``              - ``demo/lora.py:11-18`` (``x @ w + (x @ a) @ b``).
* ``gqa_paged_decode``  - ``python/cleave/dynamic/reference.py:180-200`` (+ ``_paged_tokens`` ``:143-152``,
                          ``_attend`` ``:85-105``, ``_finish`` ``:68-82``).
* ``mla_paged_decode``  - ``python/cleave/dynamic/reference.py:297-320`` (+ ``_mla_attend_rows`` ``:108-128``).
* ``valid_len`` / ``split_ranges`` - the integer page arithmetic of
                          ``python/cleave/dynamic/paging/builders/slab.py:132-142`` and
                          ``python/cleave/dynamic/paging/stages.py:331-347``.

Parity pin: the functions here are checked, bit for bit where they are integer and to fp32
round-off where they are floating point, against outputs produced by importing the reference
itself (fixtures under ``tests/golden``; generator ``tests/golden/make_golden.py``).

Storage types: low-precision tensors travel as float32 arrays whose values are exactly
representable in the storage type ("f16" or "bf16"); ``round_to`` performs the
round-to-nearest-even cast a torch ``.to(dtype)`` performs.
"""

from __future__ import annotations

import numpy as np

LOG2E = 1.4426950408889634  # python/cleave/dynamic/paging/stages.py:29
NEG_INF = float("-inf")


# --------------------------------------------------------------------------- storage casts
def round_bf16(x: np.ndarray) -> np.ndarray:
    """float32 -> nearest-even bfloat16 -> float32 (NaN stays NaN)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32)
    lsb = (bits >> np.uint32(16)) & np.uint32(1)
    rounded = (bits + np.uint32(0x7FFF) + lsb) & np.uint32(0xFFFF0000)
    out = rounded.view(np.float32).copy()
    nan = np.isnan(x)
    if nan.any():
        out[nan] = np.nan
    return out


def round_f16(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)


def round_to(x: np.ndarray, dtype: str) -> np.ndarray:
    if dtype == "f16":
        return round_f16(x)
    if dtype == "bf16":
        return round_bf16(x)
    if dtype == "f32":
        return np.asarray(x, dtype=np.float32)
    raise ValueError(f"unknown storage dtype {dtype!r}")


def f32(x) -> np.ndarray:
    return np.asarray(x, dtype=np.float32)


# --------------------------------------------------------------------------- dense GEMM family
def matmul(x, w, dtype: str = "f16") -> np.ndarray:
    """``Y = X @ W`` in fp32, cast to ``dtype``. X (M,K), W (K,N) row-major."""
    return round_to(f32(x) @ f32(w), dtype)


def matmul_splitk_partials(x, w, split: int) -> np.ndarray:
    """The ``(S, M, N)`` fp32 partial products a split-K plan sums:
    ``P[s] = X[:, sK/S:(s+1)K/S] @ W[sK/S:(s+1)K/S, :]``."""
    x, w = f32(x), f32(w)
    k = x.shape[1]
    assert k % split == 0
    step = k // split
    return np.stack([x[:, s * step:(s + 1) * step] @ w[s * step:(s + 1) * step] for s in range(split)])


def rms_norm(x, eps: float = 0.0, gamma=None) -> np.ndarray:
    """``x * (1 / sqrt(mean(x*x) + eps))`` along the last axis, fp32 statistics; an optional
    per-column weight ``gamma`` multiplies the normalised row."""
    x = f32(x)
    ms = np.mean(x * x, axis=-1, keepdims=True, dtype=np.float32)
    if eps:
        ms = ms + np.float32(eps)
    y = x * (np.float32(1.0) / np.sqrt(ms))
    if gamma is not None:
        y = y * f32(gamma)
    return y.astype(np.float32)


def rmsnorm_matmul(x, w, eps: float = 0.0, gamma=None, dtype: str = "f16") -> np.ndarray:
    return round_to(rms_norm(x, eps, gamma) @ f32(w), dtype)


def silu(x) -> np.ndarray:
    x = f32(x)
    return x / (np.float32(1.0) + np.exp(-x))


def swiglu(x, w0, w1, dtype: str = "f16") -> np.ndarray:
    x = f32(x)
    return round_to(silu(x @ f32(w0)) * (x @ f32(w1)), dtype)


# --------------------------------------------------------------------------- static attention
def _grouped(a: np.ndarray, b: np.ndarray):
    """Broadcast leading batch axes the way the tile IR does: the smaller extent is
    ``repeat_interleave``d up to the larger."""
    for i in range(a.ndim - 2):
        ea, eb = a.shape[i], b.shape[i]
        if ea > eb:
            b = np.repeat(b, ea // eb, axis=i)
        elif eb > ea:
            a = np.repeat(a, eb // ea, axis=i)
    return a, b


def attention(q, k, v, dtype: str = "f16", scale: float | None = None) -> np.ndarray:
    """Static attention ``softmax(Q K^T / sqrt(d)) V`` written, as the reference writes it, with
    the fixed shift ``exp(s/n - 50/n) / sum``. ``q`` (HQ, SQ, D); ``k``, ``v`` (HKV, SKV, D);
    query head ``h`` reads kv head ``h // (HQ/HKV)``. ``scale`` overrides ``1/sqrt(D)``."""
    q, k, v = f32(q), f32(k), f32(v)
    n = np.float32(q.shape[-1] ** 0.5)
    qq, kk = _grouped(q, k)
    if scale is None:
        s = (qq @ np.swapaxes(kk, -1, -2)) / n
        shift = np.float32(-50.0 / float(n))
    else:
        s = (qq @ np.swapaxes(kk, -1, -2)) * np.float32(scale)
        shift = np.float32(-50.0 * scale)
    e = np.exp(s + shift)
    p = e / e.sum(axis=-1, keepdims=True, dtype=np.float32)
    pp, vv = _grouped(p, v)
    return round_to(pp @ vv, dtype)


def attention_exact(q, k, v, dtype: str = "f16") -> np.ndarray:
    """``softmax(Q K^T / sqrt(d)) V`` with the exact row maximum (demo/attention.py:11-13;
    ``composites.softmax`` without a shift subtracts ``max`` along the axis)."""
    q, k, v = f32(q), f32(k), f32(v)
    qq, kk = _grouped(q, k)
    s = (qq @ np.swapaxes(kk, -1, -2)) / np.float32(q.shape[-1] ** 0.5)
    e = np.exp(s - s.max(axis=-1, keepdims=True))
    p = e / e.sum(axis=-1, keepdims=True, dtype=np.float32)
    pp, vv = _grouped(p, v)
    return round_to(pp @ vv, dtype)


def matmul_matmul(q, k, v, dtype: str = "f16") -> np.ndarray:
    """``(Q K^T) V`` in fp32, no softmax and no scale (demo/matmul_matmul.py:11-13); grouped heads
    broadcast as in ``attention``."""
    q, k, v = f32(q), f32(k), f32(v)
    qq, kk = _grouped(q, k)
    s = qq @ np.swapaxes(kk, -1, -2)
    ss, vv = _grouped(s, v)
    return round_to(ss @ vv, dtype)


def qknorm_attention(q, k, v, eps: float = 1e-6, dtype: str = "f16") -> np.ndarray:
    """``attention(rms(q), rms(k), v)`` with ``rms(x) = x * rsqrt(mean(x*x, -1) + eps)`` written out in
    primitives as demo/qknorm.py:17-24 does (mean = sum / extent, python/cleave/frontend/tensor.py:273-274)."""
    q, k = f32(q), f32(k)
    d = np.float32(q.shape[-1])
    qn = q * (np.float32(1) / np.sqrt((q * q).sum(-1, keepdims=True, dtype=np.float32) / d + np.float32(eps)))
    kn = k * (np.float32(1) / np.sqrt((k * k).sum(-1, keepdims=True, dtype=np.float32) / d + np.float32(eps)))
    return attention(qn.astype(np.float32), kn.astype(np.float32), v, dtype)


def matmul_rowsum(x, w, dtype: str = "f16") -> np.ndarray:
    """``(X @ W).sum(-1, keepdim=True)`` in fp32 (demo/matmul_rowsum.py:6-8); shape (M, 1)."""
    return round_to((f32(x) @ f32(w)).sum(-1, keepdims=True, dtype=np.float32), dtype)


def lora(x, w, a, b, dtype: str = "f16") -> np.ndarray:
    """``X @ W + (X @ A) @ B`` in fp32 (demo/lora.py:11-18)."""
    x = f32(x)
    return round_to(x @ f32(w) + (x @ f32(a)) @ f32(b), dtype)


def attention_masked(q, k, v, scale: float, causal: bool, dtype: str = "bf16"):
    """Attention with the end-aligned causal mask of the paged and ragged prefill operators
    (python/cleave/dynamic/reference.py:85-133: keep ``kv_pos <= kv_len - q_len + q_pos``, fp32
    softmax through ``_finish``, base-2 lse). q (HQ, SQ, D); k, v (HKV, SKV, D).
    Returns (out (HQ, SQ, D), lse (HQ, SQ))."""
    q, k, v = f32(q), f32(k), f32(v)
    hq, sq, _ = q.shape
    hkv, skv, _ = k.shape
    g = hq // hkv
    kk, vv = np.repeat(k, g, axis=0), np.repeat(v, g, axis=0)
    logits = np.einsum("hqd,hkd->hqk", q, kk, optimize=True).astype(np.float32) * np.float32(scale)
    if causal:
        keep = np.arange(skv)[None, :] <= (skv - sq) + np.arange(sq)[:, None]
        logits = np.where(keep[None], logits, -np.inf).astype(np.float32)
    w, l = _finish(logits)
    return round_to(np.einsum("hqk,hkd->hqd", w, vv, optimize=True), dtype), l


def gqa_ragged_prefill(q, k, v, qo_indptr, kv_indptr, scale: float, dtype: str = "bf16", causal: bool = True):
    """Ragged causal prefill (python/cleave/dynamic/reference.py:244-278): per request r, rows
    ``qo_indptr[r]:qo_indptr[r+1]`` of q (total_q, HQ, D) attend keys ``kv_indptr[r]:kv_indptr[r+1]`` of
    k, v (total_kv, HKV, D) under the end-aligned causal mask; requests without queries or keys keep the
    preallocated 0 / -inf. Returns (out (total_q, HQ, D), lse (total_q, HQ))."""
    q, k, v = f32(q), f32(k), f32(v)
    total_q, hq, d = q.shape
    out = np.zeros((total_q, hq, d), dtype=np.float32)
    lse = np.full((total_q, hq), NEG_INF, dtype=np.float32)
    for r in range(len(qo_indptr) - 1):
        qs, qe, ks, ke = int(qo_indptr[r]), int(qo_indptr[r + 1]), int(kv_indptr[r]), int(kv_indptr[r + 1])
        if qe <= qs or ke <= ks:
            continue
        o, l = attention_masked(q[qs:qe].transpose(1, 0, 2), k[ks:ke].transpose(1, 0, 2), v[ks:ke].transpose(1, 0, 2),
                                scale, causal, dtype)
        out[qs:qe] = o.transpose(1, 0, 2)
        lse[qs:qe] = l.T
    return out, lse


def gqa_paged_prefill(q, k_cache, v_cache, qo_indptr, kv_indptr, kv_indices, scale: float, dtype: str = "bf16"):
    """Paged causal prefill over page-size-1 caches (python/cleave/dynamic/reference.py:204-241): request r
    attends the rows ``kv_indices[kv_indptr[r]:kv_indptr[r+1]]`` of caches (num_pages, 1, HKV, D)."""
    q, kc, vc = f32(q), f32(k_cache), f32(v_cache)
    total_q, hq, d = q.shape
    out = np.zeros((total_q, hq, d), dtype=np.float32)
    lse = np.full((total_q, hq), NEG_INF, dtype=np.float32)
    for r in range(len(qo_indptr) - 1):
        qs, qe, ks, ke = int(qo_indptr[r]), int(qo_indptr[r + 1]), int(kv_indptr[r]), int(kv_indptr[r + 1])
        if qe <= qs or ke <= ks:
            continue
        pages = np.asarray(kv_indices[ks:ke], dtype=np.int64)
        o, l = attention_masked(q[qs:qe].transpose(1, 0, 2), kc[pages, 0].transpose(1, 0, 2),
                                vc[pages, 0].transpose(1, 0, 2), scale, True, dtype)
        out[qs:qe] = o.transpose(1, 0, 2)
        lse[qs:qe] = l.T
    return out, lse


def mla_decode(q, kv, q_pe, k_pe, scale: float, dtype: str = "bf16") -> np.ndarray:
    """Absorbed-latent MLA decode: ``S = (Q KV^T + Qpe Kpe^T) * scale``; ``O = softmax(S) KV``.
    q (B,H,D), kv (B,SKV,D), q_pe (B,H,PE), k_pe (B,SKV,PE)."""
    q, kv, q_pe, k_pe = f32(q), f32(kv), f32(q_pe), f32(k_pe)
    s = (q @ np.swapaxes(kv, -1, -2) + q_pe @ np.swapaxes(k_pe, -1, -2)) * np.float32(scale)
    shift = np.float32(-50.0 * scale)
    e = np.exp(s + shift)
    p = e / e.sum(axis=-1, keepdims=True, dtype=np.float32)
    return round_to(p @ kv, dtype)


# --------------------------------------------------------------------------- paged decode
def _finish(logits: np.ndarray):
    """Softmax weights and base-2 log-sum-exp of a logit block; a row with no live column
    gets zero weights and a -inf lse."""
    m = logits.max(axis=-1, keepdims=True)
    safe_m = np.where(np.isneginf(m), np.float32(0), m)
    e = np.exp(logits - safe_m)
    tot = e.sum(axis=-1, keepdims=True, dtype=np.float32)
    with np.errstate(divide="ignore"):
        lse = (np.log(tot) + safe_m)[..., 0] / np.float32(np.log(2.0))
    lse = np.where(np.isneginf(m[..., 0]), np.float32(NEG_INF), lse).astype(np.float32)
    w = e / np.where(tot == 0, np.float32(1), tot)
    w = np.where(np.isneginf(m), np.float32(0), w)
    return w.astype(np.float32), lse


def paged_tokens(kv_indices: np.ndarray, base: int, kv_len: int, page_size: int):
    """(page id, slot) of every live token of one request, in order."""
    n_pages = -(-kv_len // page_size)
    pages = np.asarray(kv_indices[base:base + n_pages], dtype=np.int64)
    if page_size == 1:
        return pages, np.zeros_like(pages)
    page_of = np.repeat(pages, page_size)[:kv_len]
    slot_of = np.tile(np.arange(page_size, dtype=np.int64), pages.size)[:kv_len]
    return page_of, slot_of


def valid_len(kv_indptr, kv_last_page_len, page_size: int) -> np.ndarray:
    """Tokens each request attends to, from page counts and the last page's fill:
    ``min(max(n_pages-1,0)*page + max(last,0), n_pages*page)``; with one token per page it is
    the page count itself."""
    ptr = np.asarray(kv_indptr, dtype=np.int64)
    n_pages = ptr[1:] - ptr[:-1]
    if page_size == 1 or kv_last_page_len is None:
        return (n_pages * page_size).astype(np.int32)
    last = np.asarray(kv_last_page_len, dtype=np.int64)
    v = np.minimum(np.maximum(n_pages - 1, 0) * page_size + np.maximum(last, 0), n_pages * page_size)
    return v.astype(np.int32)


def split_ranges(valid: int, kv_tile: int, split: int):
    """``[(tile0, my_trip, split_end)]`` per split index: tiles are dealt ``ceil(n_tiles/split)``
    per split, a trailing split may own none."""
    n_tiles = -(-valid // kv_tile)
    per = -(-n_tiles // split)
    out = []
    for s in range(split):
        out.append((s * per, max(min(per, n_tiles - s * per), 0), min(valid, kv_tile * (s * per + per))))
    return out


def gqa_paged_decode(q, k_cache, v_cache, kv_indptr, kv_indices, kv_last_page_len, sm_scale: float,
                     out_dtype: str = "bf16"):
    """Paged GQA decode. q (batch, HQ, D); caches (num_pages, page, HKV, D); ``kv_indptr`` in
    page units. Returns ``(out, lse)``: ``out`` rounded to ``out_dtype`` (the reference always
    returns bf16), ``lse`` base-2 fp32. An empty request gives 0 / -inf."""
    q, k_cache, v_cache = f32(q), f32(k_cache), f32(v_cache)
    batch, hq, d = q.shape
    page_size, hkv = k_cache.shape[1], k_cache.shape[2]
    group = hq // hkv
    lens = valid_len(kv_indptr, kv_last_page_len, page_size)
    out = np.zeros((batch, hq, d), dtype=np.float32)
    lse = np.full((batch, hq), NEG_INF, dtype=np.float32)
    for b in range(batch):
        n = int(lens[b])
        if n <= 0:
            continue
        page_of, slot_of = paged_tokens(kv_indices, int(kv_indptr[b]), n, page_size)
        kk = k_cache[page_of, slot_of]  # (n, HKV, D)
        vv = v_cache[page_of, slot_of]
        qg = q[b].reshape(hkv, group, d)
        logits = np.einsum("hgd,khd->hgk", qg, kk, optimize=True).astype(np.float32) * np.float32(sm_scale)
        w, l = _finish(logits)
        o = np.einsum("hgk,khd->hgd", w, vv, optimize=True)
        out[b] = round_to(o.reshape(hq, d), out_dtype)
        lse[b] = l.reshape(hq)
    return out, lse


def mla_paged_decode(q_nope, q_pe, ckv_cache, kpe_cache, kv_indptr, kv_indices, sm_scale: float,
                     out_dtype: str = "bf16"):
    """Paged MLA decode, one token per page. q_nope (batch,H,CKV), q_pe (batch,H,KPE),
    ckv_cache (pages,1,CKV), kpe_cache (pages,1,KPE)."""
    qn, qp, ckv, kpe = f32(q_nope), f32(q_pe), f32(ckv_cache), f32(kpe_cache)
    batch, h, c = qn.shape
    out = np.zeros((batch, h, c), dtype=np.float32)
    lse = np.full((batch, h), NEG_INF, dtype=np.float32)
    ptr = np.asarray(kv_indptr, dtype=np.int64)
    for b in range(batch):
        n = int(ptr[b + 1] - ptr[b])
        if n <= 0:
            continue
        pages = np.asarray(kv_indices[ptr[b]:ptr[b] + n], dtype=np.int64)
        kc, kp = ckv[pages, 0], kpe[pages, 0]
        logits = (qn[b] @ kc.T + qp[b] @ kp.T).astype(np.float32) * np.float32(sm_scale)
        w, l = _finish(logits)
        out[b] = round_to(w @ kc, out_dtype)
        lse[b] = l
    return out, lse


def mla_paged_prefill(q_nope, q_pe, ckv_cache, kpe_cache, qo_indptr, kv_indptr, kv_indices, scale: float,
                      dtype: str = "bf16"):
    """Paged causal MLA prefill (python/cleave/dynamic/reference.py:324-365): per request, rows
    ``qo_indptr[r]:qo_indptr[r+1]`` attend the latent rows ``kv_indices[kv_indptr[r]:kv_indptr[r+1]]`` under the
    end-aligned causal mask; ``S = (Qn CKV^T + Qp KPE^T) scale``, ``O = softmax(S) CKV``."""
    qn, qp, ckv, kpe = f32(q_nope), f32(q_pe), f32(ckv_cache), f32(kpe_cache)
    total_q, h, c = qn.shape
    out = np.zeros((total_q, h, c), dtype=np.float32)
    lse = np.full((total_q, h), NEG_INF, dtype=np.float32)
    for r in range(len(qo_indptr) - 1):
        qs, qe, ks, ke = int(qo_indptr[r]), int(qo_indptr[r + 1]), int(kv_indptr[r]), int(kv_indptr[r + 1])
        if qe <= qs or ke <= ks:
            continue
        pages = np.asarray(kv_indices[ks:ke], dtype=np.int64)
        kv, kp = ckv[pages, 0], kpe[pages, 0]
        logits = (np.einsum("qhc,kc->qhk", qn[qs:qe], kv, optimize=True) +
                  np.einsum("qhp,kp->qhk", qp[qs:qe], kp, optimize=True)).astype(np.float32) * np.float32(scale)
        keep = np.arange(ke - ks)[None, :] <= (ke - ks) - (qe - qs) + np.arange(qe - qs)[:, None]
        logits = np.where(keep[:, None, :], logits, -np.inf).astype(np.float32)
        w, l = _finish(logits)
        out[qs:qe] = round_to(np.einsum("qhk,kc->qhc", w, kv, optimize=True), dtype)
        lse[qs:qe] = l
    return out, lse


def attention_lse(q, k, v, scale: float, dtype: str = "f16"):
    """Decode attention plus base-2 lse for contiguous caches, used to check the split-KV
    log-sum-exp combine: q (B,HQ,D), k/v (B,HKV,SKV,D)."""
    q, k, v = f32(q), f32(k), f32(v)
    b, hq, d = q.shape
    hkv = k.shape[1]
    g = hq // hkv
    qg = q.reshape(b, hkv, g, d)
    logits = np.einsum("bhgd,bhkd->bhgk", qg, k, optimize=True).astype(np.float32) * np.float32(scale)
    w, l = _finish(logits)
    o = np.einsum("bhgk,bhkd->bhgd", w, v, optimize=True)
    return round_to(o.reshape(b, hq, d), dtype), l.reshape(b, hq)
