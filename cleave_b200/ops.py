"""Tensor-level entry to the kernel library: torch CUDA tensors in, torch CUDA tensors out.

Torch is plumbing here (device memory, the current stream); every operator body is a
hand-written sm_100a kernel reached through the C ABI of ``include/cleave_b200.h``.
"""

from __future__ import annotations

import ctypes as C

import torch

from . import _lib

_DT = {torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}
_workspaces: dict = {}


def _dtype_code(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported storage dtype {t.dtype}; use float16 or bfloat16") from None


def _cuda(t: torch.Tensor, name: str) -> torch.Tensor:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    return t


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def workspace(kind: str, nbytes: int, device) -> torch.Tensor:
    """A zero-initialised scratch buffer cached per (kind, device, stream); launches on one
    stream run in order, so they can share it. It is allocated once per size, never per call
    (the reference's split wrappers do the same, python/cleave/runtime/autotune.py:191-222)."""
    index = torch.device(device).index
    if index is None:
        index = torch.cuda.current_device()
    key = (kind, index, _stream())
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 256), dtype=torch.uint8, device=device)  # never smaller than the status header
        _workspaces[key] = ws
    return ws


def set_small_problem_limit(tokens: int) -> int:
    """Causal prefill with at most ``tokens`` keys (default 256) and at least eight times as many query rows runs on
    two light kernels (one CTA per row that sees a key, one warp per row that sees none) instead of the tcgen05
    kernels; 0 = never. Returns the previous value. Process-wide."""
    return int(_lib.lib().cb200_set_small_problem_limit(int(tokens)))


def check_workspace(ws: torch.Tensor) -> None:
    """Synchronise and raise ``Cb200Error`` (status 6) if a kernel recorded a bounded-wait timeout in
    ``ws``. The launch that gave up left arrival counters behind, so the workspace is zero-filled again
    before the error is raised: the next launch on it starts clean."""
    try:
        _lib.check(_lib.lib().cb200_workspace_status(ws.data_ptr(), _stream()))
    except _lib.Cb200Error as exc:
        if exc.status == _lib.ERR_DEVICE_TIMEOUT:
            _lib.check(_lib.lib().cb200_workspace_reset(ws.data_ptr(), ws.numel(), _stream()))
        raise


def _attn_args(q, k_cache, v_cache, out, lse, ws, *, batch, hq, hkv, d, sm_scale, q_rows=1,
               kv_indptr=None, kv_indices=None, kv_last_page_len=None, page_size=0, num_pages=0,
               kv_len=0, max_ctas=0):
    a = _lib.AttnDecodeArgs()
    a.q, a.k_cache, a.v_cache = q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr()
    a.kv_indptr = None if kv_indptr is None else kv_indptr.data_ptr()
    a.kv_indices = None if kv_indices is None else kv_indices.data_ptr()
    a.kv_last_page_len = None if kv_last_page_len is None else kv_last_page_len.data_ptr()
    a.out = out.data_ptr()
    a.lse = None if lse is None else lse.data_ptr()
    a.workspace = None if ws is None else ws.data_ptr()
    a.workspace_bytes = 0 if ws is None else ws.numel()
    a.batch, a.num_qo_heads, a.num_kv_heads, a.head_dim = batch, hq, hkv, d
    a.page_size, a.num_pages = page_size, num_pages
    a.num_kv_indices = 0 if kv_indices is None else kv_indices.numel()
    a.kv_len, a.q_rows, a.dtype, a.max_ctas = kv_len, q_rows, _dtype_code(q), max_ctas
    a.sm_scale = float(sm_scale)
    return a


def _paged_decode_args(q, k_cache, v_cache, kv_indptr, kv_indices, kv_last_page_len, sm_scale, out, lse, max_ctas):
    """Argument checks shared by the two paged decode entry points; returns the filled argument struct.
    The kernel trusts nothing in the tables (page ids and ranges are clipped on the device), but shapes,
    dtypes and devices are the caller's contract and are refused here."""
    q, k_cache, v_cache = _cuda(q, "q"), _cuda(k_cache, "k_cache"), _cuda(v_cache, "v_cache")
    if q.dim() != 3 or k_cache.dim() != 4:
        raise ValueError("q must be (batch, HQ, D) and the caches (num_pages, page_size, HKV, D)")
    batch, hq, d = q.shape
    num_pages, page_size, hkv, d2 = k_cache.shape
    if d2 != d or v_cache.shape != k_cache.shape:
        raise ValueError("k_cache / v_cache must be (num_pages, page_size, HKV, D) with q's D")
    if k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
        raise TypeError("q and the caches must share one storage dtype")
    if kv_indptr.dtype != torch.int32 or kv_indices.dtype != torch.int32:
        raise TypeError("kv_indptr / kv_indices must be int32")
    if kv_indptr.numel() != batch + 1:
        raise ValueError("kv_indptr must have batch + 1 entries")
    _cuda(kv_indptr, "kv_indptr"), _cuda(kv_indices, "kv_indices")
    if page_size != 1 and kv_last_page_len is None:
        raise TypeError("missing input 'kv_last_page_len'")
    if kv_last_page_len is not None:
        if _cuda(kv_last_page_len, "kv_last_page_len").dtype != torch.int32 or kv_last_page_len.numel() != batch:
            raise TypeError("kv_last_page_len must hold batch int32 values")
    if tuple(_cuda(out, "out").shape) != tuple(q.shape) or out.dtype != q.dtype or out.device != q.device:
        raise ValueError("out must have q's shape, dtype and device")
    if tuple(_cuda(lse, "lse").shape) != (batch, hq) or lse.dtype != torch.float32 or lse.device != q.device:
        raise ValueError("lse must be (batch, HQ) float32 on q's device")
    return _attn_args(q, k_cache, v_cache, out, lse, None, batch=batch, hq=hq, hkv=hkv, d=d,
                      sm_scale=sm_scale, kv_indptr=kv_indptr, kv_indices=kv_indices,
                      kv_last_page_len=kv_last_page_len, page_size=page_size, num_pages=num_pages,
                      max_ctas=max_ctas)


def gqa_paged_decode(q, k_cache, v_cache, kv_indptr, kv_indices, kv_last_page_len, sm_scale, *,
                     out=None, lse=None, max_ctas=0):
    """Paged GQA/MHA/MQA decode. Argument order and meaning follow the reference's operator
    (python/cleave/dynamic/reference.py:156-200): q (batch, HQ, D); caches
    (num_pages, page_size, HKV, D); ``kv_indptr`` in pages; ``kv_last_page_len`` may be None
    when page_size is 1. Returns ``(out, lse)`` with ``lse`` base 2."""
    if out is None:
        out = torch.empty_like(q)
    if lse is None:
        lse = torch.empty(tuple(q.shape[:2]), dtype=torch.float32, device=q.device)
    probe = _paged_decode_args(q, k_cache, v_cache, kv_indptr, kv_indices, kv_last_page_len, sm_scale, out, lse,
                               max_ctas)
    need = _lib.lib().cb200_attn_decode_workspace_bytes(C.byref(probe))
    if need == 0:
        _lib.check(_lib.lib().cb200_attn_decode(C.byref(probe), _stream()))  # raises the real status
    ws = workspace("attn_decode", need, q.device)
    probe.workspace, probe.workspace_bytes = ws.data_ptr(), ws.numel()
    _lib.check(_lib.lib().cb200_attn_decode(C.byref(probe), _stream()))
    return out, lse


def attention_decode(q, k, v, sm_scale=None, *, out=None, lse=None, max_ctas=0):
    """Static decode attention over contiguous caches. ``q`` (HQ, SQ, D) with a small SQ;
    ``k``, ``v`` (HKV, SKV, D); query head h reads kv head h // (HQ/HKV)
    (reference: demo/attention.py:5-8, demo/{mha,gqa,mqa}_decode.py). Returns ``out`` (HQ, SQ, D);
    pass ``lse`` (HQ, SQ) fp32 to also get the base-2 log-sum-exp."""
    q, k, v = _cuda(q, "q"), _cuda(k, "k"), _cuda(v, "v")
    hq, sq, d = q.shape
    hkv, skv, d2 = k.shape
    if d2 != d or v.shape != k.shape or hq % hkv:
        raise ValueError("shapes: q (HQ,SQ,D), k/v (HKV,SKV,D), HQ a multiple of HKV")
    if sm_scale is None:
        sm_scale = float(d) ** -0.5
    if out is None:
        out = torch.empty_like(q)
    # the C ABI sees batch = HKV requests of one kv head each with HQ/HKV query heads
    probe = _attn_args(q, k, v, out, lse, None, batch=hkv, hq=hq // hkv, hkv=1, d=d,
                       sm_scale=sm_scale, q_rows=sq, kv_len=skv, max_ctas=max_ctas)
    need = _lib.lib().cb200_attn_decode_workspace_bytes(C.byref(probe))
    if need == 0:
        _lib.check(_lib.lib().cb200_attn_decode(C.byref(probe), _stream()))
    ws = workspace("attn_decode", need, q.device)
    probe.workspace, probe.workspace_bytes = ws.data_ptr(), ws.numel()
    _lib.check(_lib.lib().cb200_attn_decode(C.byref(probe), _stream()))
    return out


def attention_prefill(q, k, v, sm_scale=None, *, causal=False, out=None, lse=None, linear=False, qk_norm_eps=None):
    """Unsplit attention with many query rows (reference: demo/attention.py:5-8 at the shapes of
    demo/{mha,gqa,mqa}_prefill.py). ``q`` (HQ, SQ, D); ``k``, ``v`` (HKV, SKV, D); D 64 or 128; query
    head h reads kv head h // (HQ/HKV). ``causal`` applies the end-aligned mask of the paged and
    ragged prefill operators (python/cleave/dynamic/reference.py:129-133). Returns ``out``
    (HQ, SQ, D); pass ``lse`` (HQ, SQ) fp32 to also get the base-2 log-sum-exp. ``linear`` drops the
    softmax (``O = (sm_scale * Q K^T) V``, see :func:`matmul_matmul`); ``qk_norm_eps`` RMS-normalises the
    rows of q and k first (see :func:`qknorm_attention`)."""
    q, k, v = _cuda(q, "q"), _cuda(k, "k"), _cuda(v, "v")
    hq, sq, d = q.shape
    hkv, skv, d2 = k.shape
    if d2 != d or v.shape != k.shape or hq % hkv:
        raise ValueError("shapes: q (HQ,SQ,D), k/v (HKV,SKV,D), HQ a multiple of HKV")
    if sm_scale is None:
        sm_scale = float(d) ** -0.5
    if out is None:
        out = torch.empty_like(q)
    a = _lib.AttnPrefillArgs()
    a.score_mode = _lib.SCORE_LINEAR if linear else _lib.SCORE_SOFTMAX
    if qk_norm_eps is not None:
        a.qk_norm, a.norm_eps = 1, float(qk_norm_eps)
    a.q, a.k, a.v, a.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    a.lse = lse.data_ptr() if lse is not None else None
    a.num_qo_heads, a.num_kv_heads, a.q_len, a.kv_len, a.head_dim = hq, hkv, sq, skv, d
    a.dtype, a.causal, a.sm_scale = _dtype_code(q), int(bool(causal)), float(sm_scale)
    need = _lib.lib().cb200_attn_prefill_workspace_bytes(C.byref(a))
    if need == 0:
        _lib.check(_lib.lib().cb200_attn_prefill(C.byref(a), _stream()))  # reports why the plan is refused
    ws = workspace("attn_prefill", need, q.device)
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    _lib.check(_lib.lib().cb200_attn_prefill(C.byref(a), _stream()))
    return out


def matmul_matmul(q, k, v, *, out=None, impl="auto"):
    """``O = (Q K^T) V`` without softmax (reference operator: demo/matmul_matmul.py:11-13): q (HQ, SQ, D);
    k, v (HKV, SKV, D); D 64 or 128. ``impl``: "scores_first" evaluates (Q K^T) V on the tcgen05 attention
    kernel (scores rounded to the storage dtype before the second product); "chain" evaluates Q (K^T V),
    a D x D intermediate per kv head and one pass over every input; "auto" takes the chain when it saves
    at least four times the FLOPs (32 times at the demo's S = 4096, D = 64)."""
    q, k, v = _cuda(q, "q"), _cuda(k, "k"), _cuda(v, "v")
    hq, sq, d = q.shape
    hkv, skv, d2 = k.shape
    if d2 != d or v.shape != k.shape or hq % hkv:
        raise ValueError("shapes: q (HQ,SQ,D), k/v (HKV,SKV,D), HQ a multiple of HKV")
    if out is None:
        out = torch.empty_like(q)
    a = _lib.MatmulMatmulArgs()
    a.q, a.k, a.v, a.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    a.num_qo_heads, a.num_kv_heads, a.q_len, a.kv_len, a.head_dim = hq, hkv, sq, skv, d
    a.dtype, a.impl = _dtype_code(q), _lib.MM_IMPL[impl]
    need = _lib.lib().cb200_matmul_matmul_workspace_bytes(C.byref(a))
    if need == 0:
        _lib.check(_lib.lib().cb200_matmul_matmul(C.byref(a), _stream()))  # reports why the plan is refused
    # the scores-first order shares the attention kernel's workspace (its status word)
    chain = bool(_lib.lib().cb200_matmul_matmul_uses_chain(C.byref(a)))
    ws = workspace("matmul_chain" if chain else "attn_prefill", need, q.device)
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    _lib.check(_lib.lib().cb200_matmul_matmul(C.byref(a), _stream()))
    return out


def qknorm_attention(q, k, v, sm_scale=None, *, eps=1e-6, out=None, lse=None):
    """Attention over RMS-normalised queries and keys (reference operator: demo/qknorm.py:17-24):
    ``softmax(rms(q) rms(k)^T * scale) v`` with ``rms(x) = x * rsqrt(mean(x^2) + eps)`` along D, fp32
    statistics. The query factor is folded into the score scale inside the kernel; K is normalised once."""
    return attention_prefill(q, k, v, sm_scale, out=out, lse=lse, qk_norm_eps=eps)


def matmul_rowsum(x, w, *, out=None):
    """``Y = rowsum(X @ W)``, shape (M, 1) (reference operator: demo/matmul_rowsum.py:6-8), computed as
    ``X @ rowsum(W)``: every input byte is read once and the (M, N) product is never formed."""
    x, w = _cuda(x, "x"), _cuda(w, "w")
    m, k = x.shape
    k2, n = w.shape
    if k2 != k or w.dtype != x.dtype:
        raise ValueError(f"shapes/dtypes: x {tuple(x.shape)} {x.dtype}, w {tuple(w.shape)} {w.dtype}")
    if out is None:
        out = torch.empty((m, 1), dtype=x.dtype, device=x.device)
    if out.numel() != m or not out.is_contiguous():
        raise ValueError("out must hold M contiguous values")
    a = _lib.MatmulRowsumArgs()
    a.x, a.w, a.y = x.data_ptr(), w.data_ptr(), out.data_ptr()
    a.m, a.n, a.k, a.dtype = m, n, k, _dtype_code(x)
    need = _lib.lib().cb200_matmul_rowsum_workspace_bytes(C.byref(a))
    if need == 0:
        _lib.check(_lib.lib().cb200_matmul_rowsum(C.byref(a), _stream()))  # raises the real status
    ws = workspace("matmul_rowsum", need, x.device)
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    _lib.check(_lib.lib().cb200_matmul_rowsum(C.byref(a), _stream()))
    return out


def lora(x, w, a, b, *, out=None):
    """``Y = X @ W + (X @ A) @ B`` (reference operator: demo/lora.py:11-18): x (M, K), w (K, N), a (K, R),
    b (R, N). Two tcgen05 GEMM launches: ``T = X @ A``, then ``[X | T] @ [W ; B]`` as one product that streams
    W while T is computed."""
    x, w, a, b = _cuda(x, "x"), _cuda(w, "w"), _cuda(a, "a"), _cuda(b, "b")
    m, k = x.shape
    n, r = w.shape[1], a.shape[1]
    if w.shape[0] != k or a.shape[0] != k or tuple(b.shape) != (r, n) or len({x.dtype, w.dtype, a.dtype, b.dtype}) != 1:
        raise ValueError("shapes: x (M,K), w (K,N), a (K,R), b (R,N), one storage dtype")
    if out is None:
        out = torch.empty((m, n), dtype=x.dtype, device=x.device)
    g = _lib.LoraArgs()
    g.x, g.w, g.a, g.b, g.y = x.data_ptr(), w.data_ptr(), a.data_ptr(), b.data_ptr(), out.data_ptr()
    g.m, g.n, g.k, g.r, g.dtype = m, n, k, r, _dtype_code(x)
    need = _lib.lib().cb200_lora_workspace_bytes(C.byref(g))
    if need == 0:
        _lib.check(_lib.lib().cb200_lora(C.byref(g), _stream()))  # raises the real status
    ws = workspace("lora", need, x.device)
    g.workspace, g.workspace_bytes = ws.data_ptr(), ws.numel()
    _lib.check(_lib.lib().cb200_lora(C.byref(g), _stream()))
    return out


def gqa_ragged_prefill(q, k, v, qo_indptr, kv_indptr, sm_scale, *, causal=True, out=None, lse=None, kv_indices=None):
    """Ragged causal prefill (reference: python/cleave/dynamic/reference.py:244-278, builders/ragged.py).
    ``q`` (total_q, HQ, D); ``k``, ``v`` (total_kv, HKV, D); ``qo_indptr`` / ``kv_indptr`` (batch + 1)
    int32 on the device. Returns ``(out, lse)``: out (total_q, HQ, D), lse (total_q, HQ) fp32 base 2;
    rows of requests without queries or keys are 0 / -inf."""
    q, k, v = _cuda(q, "q"), _cuda(k, "k"), _cuda(v, "v")
    total_q, hq, d = q.shape
    total_kv, hkv, d2 = k.shape
    if d2 != d or v.shape != k.shape or hq % hkv:
        raise ValueError("shapes: q (total_q,HQ,D), k/v (total_kv,HKV,D), HQ a multiple of HKV")
    if qo_indptr.dtype != torch.int32 or kv_indptr.dtype != torch.int32 or qo_indptr.numel() != kv_indptr.numel():
        raise ValueError("qo_indptr and kv_indptr: int32 tensors of batch + 1 entries")
    if out is None:
        out = torch.zeros_like(q)
    if lse is None:
        lse = torch.full((total_q, hq), float("-inf"), dtype=torch.float32, device=q.device)
    a = _lib.AttnPrefillRaggedArgs()
    a.q, a.k, a.v, a.out, a.lse = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr()
    a.qo_indptr, a.kv_indptr = _cuda(qo_indptr, "qo_indptr").data_ptr(), _cuda(kv_indptr, "kv_indptr").data_ptr()
    a.kv_indices = kv_indices.data_ptr() if kv_indices is not None else None
    if kv_indices is not None:
        if kv_indices.dtype != torch.int32 or not kv_indices.is_contiguous() or kv_indices.device != q.device:
            raise ValueError("kv_indices: a contiguous int32 tensor on q's device")
        a.num_kv_indices = kv_indices.numel()  # ranges of kv_indptr are clipped to it on the device
    a.batch, a.total_q, a.total_kv = qo_indptr.numel() - 1, total_q, total_kv
    a.num_qo_heads, a.num_kv_heads, a.head_dim = hq, hkv, d
    a.dtype, a.causal, a.sm_scale = _dtype_code(q), int(bool(causal)), float(sm_scale)
    need = _lib.lib().cb200_attn_prefill_ragged_workspace_bytes(C.byref(a))
    if need == 0:
        _lib.check(_lib.lib().cb200_attn_prefill_ragged(C.byref(a), _stream()))  # reports why the plan is refused
    ws = workspace("attn_prefill", need, q.device)
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    _lib.check(_lib.lib().cb200_attn_prefill_ragged(C.byref(a), _stream()))
    return out, lse


def gqa_paged_prefill(q, k_cache, v_cache, qo_indptr, kv_indptr, kv_indices, sm_scale, *, causal=True, out=None,
                      lse=None):
    """Paged causal prefill over page-size-1 caches (reference: python/cleave/dynamic/reference.py:204-241,
    builders/prefill.py). ``q`` (total_q, HQ, D); caches (num_pages, 1, HKV, D); request r attends the
    tokens ``kv_indices[kv_indptr[r] : kv_indptr[r+1]]``. Returns ``(out, lse)`` as gqa_ragged_prefill."""
    k_cache, v_cache = _cuda(k_cache, "k_cache"), _cuda(v_cache, "v_cache")
    if k_cache.dim() != 4 or k_cache.shape[1] != 1 or v_cache.shape != k_cache.shape:
        raise ValueError("caches: (num_pages, 1, HKV, D), one token per page")
    if kv_indices.dtype != torch.int32:
        raise ValueError("kv_indices: int32")
    return gqa_ragged_prefill(q, k_cache[:, 0], v_cache[:, 0], qo_indptr, kv_indptr, sm_scale, causal=causal, out=out,
                              lse=lse, kv_indices=_cuda(kv_indices, "kv_indices"))


def gqa_paged_decode_static_scratch(q, k_cache, v_cache, kv_indptr, kv_indices, kv_last_page_len, sm_scale,
                                    *, out, lse, max_ctas=0):
    """Paged decode for hosts that may not allocate device memory (a server that gave this
    library only tensors from its own arena, a runtime that bans allocation after start-up, a
    GPU already filled by the KV cache). The split-KV scratch is a fixed 4 MiB array inside the
    library instead of a torch buffer, so the caller must pass ``out`` and ``lse`` too: nothing is
    allocated here. Same results as :func:`gqa_paged_decode`. Problems that need more scratch
    than the array holds raise ``Cb200Error`` (status 7). All calls on a device share the array:
    keep them on one stream, or order them, or they race. The first call on a device resolves
    the array's address; make it before any stream capture."""
    a = _paged_decode_args(q, k_cache, v_cache, kv_indptr, kv_indices, kv_last_page_len, sm_scale, out, lse, max_ctas)
    _lib.check(_lib.lib().cb200_attn_decode_static_scratch(C.byref(a), _stream()))
    return out, lse


def check_static_scratch() -> None:
    """Synchronise and raise ``Cb200Error`` (status 6) if a bounded wait of the most recent
    :func:`gqa_paged_decode_static_scratch` call on the current device gave up."""
    _lib.check(_lib.lib().cb200_attn_decode_static_scratch_status(_stream()))


def _gemm(op, x, w, w1=None, gamma=None, eps=0.0, split_k=0, out=None, max_ctas=0, addend=None, x2=None, w2=None,
          dependent_launch=1, peers=None):
    if not x.is_cuda or not w.is_cuda:
        raise ValueError("x and w must be CUDA tensors (there is no CPU path)")
    ldx = 0
    if op == _lib.GEMM_MATMUL and x.dim() == 2 and not x.is_contiguous() and x.stride(1) == 1:
        ldx = x.stride(0)   # a K slice of a wider matrix: the kernel reads it in place with X's row pitch
    else:
        x = _cuda(x, "x")
    w = _cuda(w, "w")
    m, k = x.shape
    k2, n = w.shape
    if k2 != k or w.dtype != x.dtype:
        raise ValueError(f"shapes/dtypes: x {tuple(x.shape)} {x.dtype}, w {tuple(w.shape)} {w.dtype}")
    if w1 is not None and (_cuda(w1, "w1").shape != w.shape or w1.dtype != x.dtype):
        raise ValueError("w1 must match w")
    if gamma is not None and (_cuda(gamma, "gamma").numel() != k or gamma.dtype != x.dtype):
        raise ValueError("gamma must hold K values of x's dtype")
    if out is None:
        out = torch.empty((m, n), dtype=x.dtype, device=x.device)
    elif tuple(out.shape) != (m, n) or out.dtype != x.dtype or not out.is_cuda or out.stride(1) != 1:
        raise ValueError("out must be an (M, N) CUDA tensor of x's dtype with unit column stride")
    a = _lib.GemmArgs()
    a.x, a.w, a.y = x.data_ptr(), w.data_ptr(), out.data_ptr()
    if out.stride(0) != n:
        a.ldy = out.stride(0)  # a column slice of a wider result (the N-sharded form)
    if peers:
        if len(peers) > 7:
            raise ValueError("at most seven peer copies")
        a.n_peers = len(peers)
        for i, ptr in enumerate(peers):
            a.y_peers[i] = int(ptr)
    a.w1 = None if w1 is None else w1.data_ptr()
    a.gamma = None if gamma is None else gamma.data_ptr()
    a.m, a.n, a.k, a.op, a.dtype = m, n, k, op, _dtype_code(x)
    a.split_k, a.max_ctas, a.eps = int(split_k), int(max_ctas), float(eps)
    a.dependent_launch = int(dependent_launch)
    a.ldx = int(ldx)
    if addend is not None:
        if tuple(_cuda(addend, "addend").shape) != (m, n) or addend.dtype != x.dtype:
            raise ValueError("addend must be (M, N) of x's dtype")
        a.addend = addend.data_ptr()
    if (x2 is None) != (w2 is None):
        raise ValueError("x2 and w2 go together")
    if x2 is not None:
        if _cuda(x2, "x2").shape[0] != m or tuple(_cuda(w2, "w2").shape) != (x2.shape[1], n) or x2.dtype != x.dtype or w2.dtype != x.dtype:
            raise ValueError("x2 must be (M, K2) and w2 (K2, N), of x's dtype")
        a.x2, a.w2, a.k2 = x2.data_ptr(), w2.data_ptr(), x2.shape[1]
    need = _lib.lib().cb200_gemm_workspace_bytes(C.byref(a))
    if need == 0:
        _lib.check(_lib.lib().cb200_gemm(C.byref(a), _stream()))  # raises the real status
    ws = workspace("gemm", need, x.device)
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    _lib.check(_lib.lib().cb200_gemm(C.byref(a), _stream()))
    return out


def peer_scatter_cols(src, ld_dst: int, dsts) -> None:
    """Copies the dense (M, N) CUDA tensor ``src`` into column slices of several (M, ld_dst)-pitched matrices:
    ``dsts`` are device pointers to element [0, first column of the slice] of each - this GPU's copy of a result
    sharded along N and the peer GPUs' copies (symmetric memory). One kernel of plain stores on the current stream;
    the caller orders the GPUs before anyone reads (:func:`cleave_b200.sharding.gemm_n_sharded_fused`)."""
    src = _cuda(src, "src")
    m, n = src.shape
    arr = (C.c_void_p * len(dsts))(*[int(d) for d in dsts])
    _lib.check(_lib.lib().cb200_peer_scatter_cols(src.data_ptr(), m, n, int(ld_dst), arr, len(dsts), _dtype_code(src), _stream()))


def matmul(x, w, *, split_k=0, out=None, max_ctas=0, addend=None, x2=None, w2=None, dependent_launch=1, peers=None):
    """``Y = X @ W`` (reference operator: demo/matmul.py:11-13); ``split_k`` is the plan's K split.
    ``addend`` (M, N) is added in the epilogue; ``x2`` (M, K2) and ``w2`` (K2, N) extend the contraction:
    ``Y = X @ W + X2 @ W2`` in one accumulator (the low-rank term of LoRA). ``dependent_launch`` 1 (the
    default of this layer) lets the grid be scheduled while the preceding kernel of the stream drains; it
    waits for that kernel before it reads or writes anything, so ordering is unchanged and only the set-up
    (barriers, tensor memory, descriptor prefetch) overlaps: 8.5 -> 7.2 us on back-to-back 128 x 128 x 4096
    products. 0 gives an ordinary launch."""
    return _gemm(_lib.GEMM_MATMUL, x, w, split_k=split_k, out=out, max_ctas=max_ctas, addend=addend, x2=x2, w2=w2,
                 dependent_launch=dependent_launch, peers=peers)


def rmsnorm_matmul(x, w, *, eps=0.0, gamma=None, split_k=0, out=None, max_ctas=0, dependent_launch=1, peers=None):
    """``Y = (X * rsqrt(mean(X^2) + eps) [* gamma]) @ W`` (reference operator:
    demo/rmsnorm_matmul.py:11-13 with python/cleave/frontend/composites.py:48-53)."""
    return _gemm(_lib.GEMM_RMSNORM, x, w, gamma=gamma, eps=eps, split_k=split_k, out=out, max_ctas=max_ctas,
                 dependent_launch=dependent_launch, peers=peers)


def swiglu(x, w0, w1, *, split_k=0, out=None, max_ctas=0, peers=None):
    """``Y = silu(X @ W0) * (X @ W1)`` (reference operator: demo/swiglu.py:6-10).

    For all three GEMM operators ``out`` may be a column slice of a wider (M, N_total) tensor, and ``peers`` a list
    of device pointers to the same element of that tensor's copies on other GPUs (symmetric memory): the kernel
    then also stores every finished tile into those copies while it computes the next one
    (:func:`cleave_b200.sharding.gemm_n_sharded_fused`)."""
    return _gemm(_lib.GEMM_SWIGLU, x, w0, w1=w1, split_k=split_k, out=out, max_ctas=max_ctas, peers=peers)


def _mla(q_nope, q_pe, ckv, kpe, sm_scale, *, kv_indptr=None, kv_indices=None, out=None, lse=None, max_ctas=0,
         impl="auto", kv_start=None, kv_lens=None):
    q_nope, q_pe, ckv, kpe = _cuda(q_nope, "q_nope"), _cuda(q_pe, "q_pe"), _cuda(ckv, "ckv"), _cuda(kpe, "kpe")
    batch, heads, dc = q_nope.shape
    dp = q_pe.shape[2]
    if q_pe.shape[:2] != (batch, heads) or ckv.shape[-1] != dc or kpe.shape[-1] != dp:
        raise ValueError("shapes: q_nope (B,H,CKV), q_pe (B,H,KPE), caches (..., CKV) / (..., KPE)")
    if out is None:
        out = torch.empty_like(q_nope)
    a = _lib.MlaDecodeArgs()
    a.q_nope, a.q_pe, a.ckv_cache, a.kpe_cache = q_nope.data_ptr(), q_pe.data_ptr(), ckv.data_ptr(), kpe.data_ptr()
    a.out = out.data_ptr()
    a.lse = None if lse is None else lse.data_ptr()
    a.batch, a.num_heads, a.ckv_dim, a.kpe_dim = batch, heads, dc, dp
    a.dtype, a.max_ctas, a.sm_scale = _dtype_code(q_nope), max_ctas, float(sm_scale)
    a.impl = _lib.MLA_IMPL[impl]
    if kv_indptr is not None:
        if kv_indptr.dtype != torch.int32 or kv_indices.dtype != torch.int32:
            raise TypeError("kv_indptr / kv_indices must be int32")
        a.kv_indptr, a.kv_indices = kv_indptr.data_ptr(), kv_indices.data_ptr()
        a.page_size, a.num_pages, a.num_kv_indices = ckv.shape[1], ckv.shape[0], kv_indices.numel()
        if kv_start is not None:
            a.kv_start, a.kv_lens = kv_start.data_ptr(), kv_lens.data_ptr()
    else:
        a.kv_len = ckv.shape[1]
    need = _lib.lib().cb200_mla_decode_workspace_bytes(C.byref(a))
    if need == 0:
        _lib.check(_lib.lib().cb200_mla_decode(C.byref(a), _stream()))  # raises the real status
    ws = workspace("mla_decode", need, q_nope.device)
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    _lib.check(_lib.lib().cb200_mla_decode(C.byref(a), _stream()))
    return out


def mla_decode(q, kv, q_pe, k_pe, sm_scale, *, out=None, lse=None, max_ctas=0, impl="auto"):
    """Static absorbed-latent MLA decode (reference operator: demo/mla_decode.py:8-13):
    q (B,H,512), kv (B,SKV,512), q_pe (B,H,64), k_pe (B,SKV,64) -> out (B,H,512).
    ``impl``: "auto", "tcgen05" (tensor-memory kernel) or "mma_sync" (the warp-MMA kernel that also
    serves paged caches)."""
    return _mla(q, q_pe, kv, k_pe, sm_scale, out=out, lse=lse, max_ctas=max_ctas, impl=impl)


def mla_paged_decode(q_nope, q_pe, ckv_cache, kpe_cache, kv_indptr, kv_indices, sm_scale, *, out=None, lse=None,
                     max_ctas=0, impl="auto"):
    """Paged MLA decode, one token per page; argument order follows the reference's operator
    (python/cleave/dynamic/reference.py:282-320). Returns ``(out, lse)``, ``lse`` base 2. ``impl``: "auto" takes
    the tcgen05 kernel (tokens as MMA rows) for at most 16 heads and the warp-MMA kernel otherwise; "tcgen05" /
    "mma_sync" force one of them."""
    batch, heads = q_nope.shape[:2]
    if lse is None:
        lse = torch.empty((batch, heads), dtype=torch.float32, device=q_nope.device)
    out = _mla(q_nope, q_pe, ckv_cache, kpe_cache, sm_scale, kv_indptr=kv_indptr, kv_indices=kv_indices,
               out=out, lse=lse, max_ctas=max_ctas, impl=impl)
    return out, lse


def mla_paged_prefill(q_nope, q_pe, ckv_cache, kpe_cache, qo_indptr, kv_indptr, kv_indices, sm_scale, *, out=None,
                      lse=None, impl="auto"):
    """Paged causal MLA prefill (reference: python/cleave/dynamic/reference.py:324-365, builders/mla.py):
    q_nope (total_q, H, 512), q_pe (total_q, H, 64), caches (num_pages, 1, 512 / 64), per-request query
    and key offsets. ``impl`` "tile" is the tcgen05 query-tile kernel (128 / H query tokens times their heads
    are the rows of every MMA; H must divide 128), "per_token" runs every query token as one request of the
    paged MLA decode kernel over the prefix the mask lets it see (any H; the prefix is re-read per token);
    "auto" takes the tile kernel whenever H divides 128. Returns ``(out, lse)``; rows without visible keys
    are 0 / -inf."""
    q_nope, qo_indptr, kv_indptr = _cuda(q_nope, "q_nope"), _cuda(qo_indptr, "qo_indptr"), _cuda(kv_indptr, "kv_indptr")
    q_pe, ckv_cache, kpe_cache = _cuda(q_pe, "q_pe"), _cuda(ckv_cache, "ckv_cache"), _cuda(kpe_cache, "kpe_cache")
    total_q, heads, dc = q_nope.shape
    batch = qo_indptr.numel() - 1
    dev = q_nope.device
    if qo_indptr.dtype != torch.int32 or kv_indptr.dtype != torch.int32 or kv_indices.dtype != torch.int32:
        raise TypeError("qo_indptr / kv_indptr / kv_indices must be int32")
    if kv_indptr.numel() != batch + 1:
        raise ValueError("qo_indptr and kv_indptr must both hold batch + 1 entries")
    if lse is None:
        lse = torch.empty(total_q, heads, dtype=torch.float32, device=dev)
    tile_ok = heads <= 128 and 128 % heads == 0 and dc == 512 and q_pe.shape[2] == 64
    if impl == "tile" and not tile_ok:
        raise ValueError("the tile kernel needs a head count that divides 128 and the 512 + 64 latent layout")
    if impl == "tile" or (impl == "auto" and tile_ok):
        if out is None:
            out = torch.empty_like(q_nope)
        a = _lib.MlaPrefillArgs()
        a.q_nope, a.q_pe, a.ckv_cache, a.kpe_cache = q_nope.data_ptr(), q_pe.data_ptr(), ckv_cache.data_ptr(), kpe_cache.data_ptr()
        a.qo_indptr, a.kv_indptr, a.kv_indices = qo_indptr.data_ptr(), kv_indptr.data_ptr(), _cuda(kv_indices, "kv_indices").data_ptr()
        a.out, a.lse = out.data_ptr(), lse.data_ptr()
        a.batch, a.total_q, a.num_heads, a.ckv_dim, a.kpe_dim = batch, total_q, heads, dc, q_pe.shape[2]
        a.num_pages, a.num_kv_indices, a.dtype, a.sm_scale = ckv_cache.shape[0], kv_indices.numel(), _dtype_code(q_nope), float(sm_scale)
        need = _lib.lib().cb200_mla_prefill_workspace_bytes(C.byref(a))
        if need == 0:
            _lib.check(_lib.lib().cb200_mla_prefill(C.byref(a), _stream()))  # raises the real status
        ws = workspace("mla_prefill", need, dev)
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        _lib.check(_lib.lib().cb200_mla_prefill(C.byref(a), _stream()))
        return out, lse
    q_lens = (qo_indptr[1:] - qo_indptr[:-1]).long().clamp(min=0)
    kv_lens = (kv_indptr[1:] - kv_indptr[:-1]).long().clamp(min=0)
    req = torch.repeat_interleave(torch.arange(batch, device=dev), q_lens, output_size=total_q)
    pos = torch.arange(total_q, device=dev) - qo_indptr.long()[req]
    seen = torch.minimum((kv_lens[req] - q_lens[req] + pos + 1).clamp(min=0), kv_lens[req]).to(torch.int32)
    start = kv_indptr[:-1][req].to(torch.int32).contiguous()
    out = _mla(q_nope, q_pe, ckv_cache, kpe_cache, sm_scale, kv_indptr=start, kv_indices=_cuda(kv_indices, "kv_indices"),
               out=out, lse=lse, impl="mma_sync", kv_start=start, kv_lens=seen.contiguous())
    return out, lse


# ---------------------------------------------------------------------------- two-stage split (compatibility)
def split_combine(num, den=None, *, axis, out=None):
    """The combine stage of a split pair (reference kernels: tests/graph/handwritten/expected_kernels/
    matmul_splitk_combine.py, mha_split_combine.py): ``out = sum(num, axis)`` in fp32, divided row by row by
    ``sum(den, axis)`` when ``den`` is given (``den`` has ``num``'s leading axes up to and including ``axis``
    and then either nothing, unit axes, or ``num``'s trailing axes)."""
    num = _cuda(num, "num")
    axis = axis % num.dim()
    outer = int(torch.tensor(num.shape[:axis]).prod()) if axis else 1
    inner = int(torch.tensor(num.shape[axis + 1:]).prod()) if axis + 1 < num.dim() else 1
    splits = num.shape[axis]
    if out is None:
        out = torch.empty(tuple(num.shape[:axis]) + tuple(num.shape[axis + 1:]), dtype=num.dtype, device=num.device)
    if out.numel() != outer * inner or out.dtype != num.dtype or not out.is_contiguous():
        raise ValueError("out must hold the reduced tensor, contiguous, in num's dtype")
    a = _lib.SplitCombineArgs()
    a.num, a.out, a.outer, a.inner, a.splits, a.dtype = num.data_ptr(), out.data_ptr(), outer, inner, splits, _dtype_code(num)
    if den is not None:
        den = _cuda(den, "den")
        if den.dtype != num.dtype or den.numel() not in (outer * splits, outer * splits * inner):
            raise ValueError("den must be (outer, splits) or (outer, splits, inner) in num's dtype")
        a.den, a.den_inner = den.data_ptr(), 1 if den.numel() == outer * splits else inner
    _lib.check(_lib.lib().cb200_split_combine(C.byref(a), _stream()))
    return out


def matmul_split_partial(x, w, split, *, out=None):
    """The partial stage of a split-K matmul (reference kernel: tests/graph/handwritten/expected_kernels/
    matmul_splitk_partial.py): ``out[s] = x[:, s K/S : (s+1) K/S] @ w[s K/S : (s+1) K/S, :]`` for every split,
    (S, M, N) in the storage dtype. One tcgen05 GEMM launch per split, reading the K slices in place."""
    x, w = _cuda(x, "x"), _cuda(w, "w")
    m, k = x.shape
    n = w.shape[1]
    if k % split or (k // split) % 8:
        raise ValueError(f"K = {k} does not cut into {split} slices of a multiple of 8 columns")
    kc = k // split
    if out is None:
        out = torch.empty((split, m, n), dtype=x.dtype, device=x.device)
    flat = out.view(split, m, n)
    for s in range(split):
        _gemm(_lib.GEMM_MATMUL, x[:, s * kc:(s + 1) * kc], w[s * kc:(s + 1) * kc], out=flat[s], split_k=1, dependent_launch=0)
    return out


def attention_split_partial(q, k, v, split, sm_scale=None, *, shift=None, o_part=None, l_part=None):
    """The partial stage of a split-KV decode (reference kernels: tests/graph/handwritten/expected_kernels/
    {gqa,mha,mqa}_split_partial.py): for every split s of the KV axis ``o_part[h, s] = sum_j e_j v_j`` and
    ``l_part[h, s] = sum_j e_j`` with ``e_j = exp(q_h . k_j * scale + shift)`` over the split's tokens
    (``shift`` defaults to the demos' -50 * scale). q (HQ, 1, D), k / v (HKV, SKV, D). The decode kernel runs
    once over the cache viewed as HKV * S requests; a second small kernel rescales its normalised results."""
    q, k, v = _cuda(q, "q"), _cuda(k, "k"), _cuda(v, "v")
    hq, sq, d = q.shape
    hkv, skv, _ = k.shape
    if sq != 1:
        raise ValueError("the two-stage partial is built for decode (one query row per head)")
    if skv % split:
        raise ValueError(f"KV length {skv} does not cut into {split} equal splits")
    g = hq // hkv
    scale = float(d) ** -0.5 if sm_scale is None else float(sm_scale)
    shift = -50.0 * scale if shift is None else float(shift)
    # query head (hkv, j) attends every split of its kv head: one copy of its row per split
    q_rep = q.view(hkv, 1, g, 1, d).expand(hkv, split, g, 1, d).reshape(hkv * split * g, 1, d).contiguous()
    k_view, v_view = k.view(hkv * split, skv // split, d), v.view(hkv * split, skv // split, d)
    out = torch.empty_like(q_rep)
    lse = torch.empty((hkv * split * g, 1), dtype=torch.float32, device=q.device)
    attention_decode(q_rep, k_view, v_view, scale, out=out, lse=lse)
    if o_part is None:
        o_part = torch.empty((hq, split, d), dtype=q.dtype, device=q.device)
    if l_part is None:
        l_part = torch.empty((hq, split), dtype=q.dtype, device=q.device)
    a = _lib.AttnUnnormaliseArgs()
    a.out, a.lse, a.o_part, a.l_part = out.data_ptr(), lse.data_ptr(), o_part.data_ptr(), l_part.data_ptr()
    a.kv_heads, a.group, a.splits, a.head_dim, a.dtype, a.shift = hkv, g, split, d, _dtype_code(q), shift
    _lib.check(_lib.lib().cb200_attn_unnormalise(C.byref(a), _stream()))
    return o_part, l_part
