"""Torch fp32 references the runtime validates every kernel against, and seeded inputs.

This is the checker of the validate stage, as in the reference (python/cleave/runtime/reference.py:280-445
for static graphs, python/cleave/dynamic/reference.py for paged operators): inputs are upcast to
fp32, evaluated eagerly on the kernel's device and cast to the storage dtype. It is never the
product path.
"""

from __future__ import annotations

import hashlib
import json

import torch

TORCH_DTYPES = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32,
                "int32": torch.int32}


def torch_dtype(name: str):
    return TORCH_DTYPES[str(name)]


def fingerprint_seed(spec) -> int:
    """A seed derived from the kernel's structure (family, dims, dtype), so that every
    candidate of one operator is validated on the same inputs (python/cleave/runtime/reference.py:86-106)."""
    text = json.dumps({"family": spec.family, "dims": spec.dims, "dtype": spec.dtype}, sort_keys=True)
    return int.from_bytes(hashlib.sha256(text.encode()).digest()[:4], "little")


def _grouped(a, b):
    for i in range(a.ndim - 2):
        ea, eb = a.shape[i], b.shape[i]
        if ea > eb:
            b = b.repeat_interleave(ea // eb, dim=i)
        elif eb > ea:
            a = a.repeat_interleave(eb // ea, dim=i)
    return a, b


def matmul(x, w):
    return x.float() @ w.float()


def rmsnorm_matmul(x, w, eps=0.0, gamma=None):
    x = x.float()
    ms = (x * x).mean(-1, keepdim=True)
    if eps:
        ms = ms + eps
    y = x * (1.0 / torch.sqrt(ms))
    if gamma is not None:
        y = y * gamma.float()
    return y @ w.float()


def swiglu(x, w0, w1):
    x = x.float()
    return torch.nn.functional.silu(x @ w0.float()) * (x @ w1.float())


def attention(q, k, v, scale=None):
    q, k, v = q.float(), k.float(), v.float()
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    qq, kk = _grouped(q, k)
    p = torch.softmax((qq @ kk.mT) * scale, dim=-1)
    pp, vv = _grouped(p, v)
    return pp @ vv


def matmul_matmul(q, k, v):
    """``(q @ k.mT) @ v`` (demo/matmul_matmul.py), grouped heads broadcast like the attention operators."""
    q, k, v = q.float(), k.float(), v.float()
    qq, kk = _grouped(q, k)
    s = qq @ kk.mT
    ss, vv = _grouped(s, v)
    return ss @ vv


def _rms(x, eps):
    return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps)


def qknorm_attention(q, k, v, eps=0.0, scale=None):
    """Attention over RMS-normalised q and k (demo/qknorm.py)."""
    return attention(_rms(q.float(), eps), _rms(k.float(), eps), v, scale)


def matmul_rowsum(x, w):
    """``(x @ w).sum(-1, keepdim=True)`` (demo/matmul_rowsum.py)."""
    return (x.float() @ w.float()).sum(-1, keepdim=True)


def lora(x, w, a, b):
    """``x @ w + (x @ a) @ b`` (demo/lora.py)."""
    x = x.float()
    return x @ w.float() + (x @ a.float()) @ b.float()


def mla_decode(q, kv, q_pe, k_pe, scale):
    q, kv, q_pe, k_pe = q.float(), kv.float(), q_pe.float(), k_pe.float()
    p = torch.softmax((q @ kv.mT + q_pe @ k_pe.mT) * scale, dim=-1)
    return p @ kv


def _finish(logits):
    lse = torch.logsumexp(logits, dim=-1) / torch.log(torch.tensor(2.0))
    w = torch.softmax(logits, dim=-1)
    blind = torch.isneginf(lse)
    if blind.any():
        w = w.masked_fill(blind[..., None], 0.0)
    return w, lse


def valid_lens(kv_indptr, kv_last_page_len, page_size):
    n_pages = (kv_indptr[1:] - kv_indptr[:-1]).long()
    if page_size == 1 or kv_last_page_len is None:
        return n_pages * page_size
    last = kv_last_page_len.long().clamp(min=0)
    return torch.minimum((n_pages - 1).clamp(min=0) * page_size + last, n_pages * page_size)


def gqa_paged_decode(q, k_cache, v_cache, kv_indptr, kv_indices, kv_last_page_len, sm_scale):
    """``(out, lse)``; out in q's dtype, lse base 2; empty request -> 0 / -inf."""
    batch, hq, d = q.shape
    page_size, hkv = k_cache.shape[1], k_cache.shape[2]
    group = hq // hkv
    lens = valid_lens(kv_indptr, kv_last_page_len, page_size).tolist()
    ptr = kv_indptr.tolist()
    out = torch.zeros(batch, hq, d, device=q.device, dtype=torch.float32)
    lse = torch.full((batch, hq), float("-inf"), device=q.device, dtype=torch.float32)
    for b, n in enumerate(lens):
        if n <= 0:
            continue
        n_pages = -(-n // page_size)
        pages = kv_indices[ptr[b]:ptr[b] + n_pages].long()
        kk = k_cache[pages].reshape(-1, hkv, d)[:n].float()
        vv = v_cache[pages].reshape(-1, hkv, d)[:n].float()
        qg = q[b].float().reshape(hkv, group, d)
        logits = torch.einsum("hgd,khd->hgk", qg, kk) * sm_scale
        w, l = _finish(logits)
        out[b] = torch.einsum("hgk,khd->hgd", w, vv).reshape(hq, d)
        lse[b] = l.reshape(hq)
    return out.to(q.dtype), lse


def mla_paged_decode(q_nope, q_pe, ckv_cache, kpe_cache, kv_indptr, kv_indices, sm_scale):
    batch, h, c = q_nope.shape
    ptr = kv_indptr.tolist()
    out = torch.zeros(batch, h, c, device=q_nope.device, dtype=torch.float32)
    lse = torch.full((batch, h), float("-inf"), device=q_nope.device, dtype=torch.float32)
    for b in range(batch):
        n = ptr[b + 1] - ptr[b]
        if n <= 0:
            continue
        pages = kv_indices[ptr[b]:ptr[b] + n].long()
        kc, kp = ckv_cache[pages, 0].float(), kpe_cache[pages, 0].float()
        logits = (q_nope[b].float() @ kc.T + q_pe[b].float() @ kp.T) * sm_scale
        w, l = _finish(logits)
        out[b] = w @ kc
        lse[b] = l
    return out.to(q_nope.dtype), lse


def _causal_attend(q, k, v, sm_scale):
    """One request: q (n_q, HQ, D), k / v (n_kv, HKV, D); end-aligned causal mask
    (python/cleave/dynamic/reference.py:85-133). Returns (out fp32, lse base 2)."""
    n_q, hq, d = q.shape
    n_kv, hkv, _ = k.shape
    group = hq // hkv
    qg = q.float().reshape(n_q, hkv, group, d)
    logits = torch.einsum("qhgd,khd->hgqk", qg, k.float()) * sm_scale
    keep = torch.arange(n_kv, device=q.device)[None, :] <= (n_kv - n_q) + torch.arange(n_q, device=q.device)[:, None]
    logits = logits.masked_fill(~keep[None, None], float("-inf"))
    w, l = _finish(logits)
    out = torch.einsum("hgqk,khd->qhgd", w, v.float()).reshape(n_q, hq, d)
    return out, l.permute(2, 0, 1).reshape(n_q, hq)


def gqa_ragged_prefill(q, k, v, qo_indptr, kv_indptr, sm_scale):
    """``(out, lse)`` of the ragged causal prefill (python/cleave/dynamic/reference.py:244-278)."""
    total_q, hq, d = q.shape
    out = torch.zeros(total_q, hq, d, device=q.device, dtype=torch.float32)
    lse = torch.full((total_q, hq), float("-inf"), device=q.device, dtype=torch.float32)
    qo, kv = qo_indptr.tolist(), kv_indptr.tolist()
    for r in range(len(qo) - 1):
        if qo[r + 1] <= qo[r] or kv[r + 1] <= kv[r]:
            continue
        o, l = _causal_attend(q[qo[r]:qo[r + 1]], k[kv[r]:kv[r + 1]], v[kv[r]:kv[r + 1]], sm_scale)
        out[qo[r]:qo[r + 1]], lse[qo[r]:qo[r + 1]] = o, l
    return out.to(q.dtype), lse


def gqa_paged_prefill(q, k_cache, v_cache, qo_indptr, kv_indptr, kv_indices, sm_scale):
    """``(out, lse)`` of the paged causal prefill over page-size-1 caches
    (python/cleave/dynamic/reference.py:204-241)."""
    total_q, hq, d = q.shape
    out = torch.zeros(total_q, hq, d, device=q.device, dtype=torch.float32)
    lse = torch.full((total_q, hq), float("-inf"), device=q.device, dtype=torch.float32)
    qo, kv = qo_indptr.tolist(), kv_indptr.tolist()
    for r in range(len(qo) - 1):
        if qo[r + 1] <= qo[r] or kv[r + 1] <= kv[r]:
            continue
        pages = kv_indices[kv[r]:kv[r + 1]].long()
        o, l = _causal_attend(q[qo[r]:qo[r + 1]], k_cache[pages, 0], v_cache[pages, 0], sm_scale)
        out[qo[r]:qo[r + 1]], lse[qo[r]:qo[r + 1]] = o, l
    return out.to(q.dtype), lse


def mla_paged_prefill(q_nope, q_pe, ckv_cache, kpe_cache, qo_indptr, kv_indptr, kv_indices, sm_scale):
    """``(out, lse)`` of the paged causal MLA prefill (python/cleave/dynamic/reference.py:324-365): per request
    the latent rows are both keys (with the rope part) and values, under the end-aligned causal mask."""
    total_q, h, c = q_nope.shape
    out = torch.zeros(total_q, h, c, device=q_nope.device, dtype=torch.float32)
    lse = torch.full((total_q, h), float("-inf"), device=q_nope.device, dtype=torch.float32)
    qo, kv = qo_indptr.tolist(), kv_indptr.tolist()
    for r in range(len(qo) - 1):
        n_q, n_kv = qo[r + 1] - qo[r], kv[r + 1] - kv[r]
        if n_q <= 0 or n_kv <= 0:
            continue
        pages = kv_indices[kv[r]:kv[r + 1]].long()
        kc, kp = ckv_cache[pages, 0].float(), kpe_cache[pages, 0].float()
        qn, qp = q_nope[qo[r]:qo[r + 1]].float(), q_pe[qo[r]:qo[r + 1]].float()
        logits = (torch.einsum("qhc,kc->qhk", qn, kc) + torch.einsum("qhp,kp->qhk", qp, kp)) * sm_scale
        keep = torch.arange(n_kv, device=logits.device)[None, :] <= (n_kv - n_q) + torch.arange(n_q, device=logits.device)[:, None]
        logits = logits.masked_fill(~keep[:, None, :], float("-inf"))
        w, l = _finish(logits)
        out[qo[r]:qo[r + 1]] = torch.einsum("qhk,kc->qhc", w, kc)
        lse[qo[r]:qo[r + 1]] = l
    return out.to(q_nope.dtype), lse


def order_inputs_for_kernel(inputs_by_name: dict, kernel) -> list:
    """The tensors of ``inputs_by_name`` in the kernel's parameter order (by buffer name), as the
    reference orders them (python/cleave/runtime/reference.py:448-479)."""
    adapter = kernel.adapter
    outs = {i % len(adapter.params) for i in (adapter.result_idx or [])}
    order = []
    for i, param in enumerate(adapter.prim_func.params):
        if i in outs:
            continue
        name = adapter.prim_func.buffer_map[param].name
        if name not in inputs_by_name:
            raise KeyError(f"kernel parameter {name!r} has no input; have {sorted(inputs_by_name)}")
        order.append(inputs_by_name[name])
    return order


def reconcile_output_layout(ref, shape):
    """View a reference as the kernel's physical output shape when only unit axes differ."""
    shape = tuple(shape)
    if tuple(ref.shape) == shape or ref.numel() != torch.Size(shape).numel():
        return ref
    return ref.reshape(shape)
