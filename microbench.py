"""Per-operator timing of the kernel library on the benchmark configurations.

    python microbench.py                      # every configuration, one line each
    python microbench.py --op rmsnorm_matmul --m 4096 --n 14336 --k 4096 --launches 3

Timing follows the reference's protocol (python/cleave/runtime/timer.py:76-108,
python/cleave/runtime/autotune.py:36-43): CUDA events around CUDA-graph replays, minimum over
rounds. Successive launches of a graph read different copies of the inputs (enough copies to
cover 2.5x the 126 MB L2) unless one copy is already larger than L2, so no launch is served from
the cache lines of the one before. ``--launches N`` instead runs N plain launches after a warm-up (what a profiler capture
wants) and prints nothing but a completion line.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from cleave_b200 import ops  # noqa: E402
from cleave_b200.runtime.timer import min_launch_us  # noqa: E402

NOMINAL_HBM_GBS, NOMINAL_TFLOPS = 8000.0, 2250.0


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    except Exception:  # noqa: BLE001
        return 6650.0, 1590.0, "fallback"


def _gen(seed=0):
    return torch.Generator(device="cpu").manual_seed(seed)


L2_BYTES = 126 * 1024 * 1024


def _rotating(make_call, tensors, max_sets=8):
    """Successive launches read different copies of the inputs, so that no launch finds its
    operands in L2 from the one before: as many copies as it takes to cover 2.5x the L2 (at most
    ``max_sets``; a working set that is already larger than L2 keeps one copy).
    ``make_call(tensors)`` returns the zero-argument launch for one copy."""
    per_set = sum(t.numel() * t.element_size() for t in tensors if t is not None)
    n = max(1, min(max_sets, -(-int(2.5 * L2_BYTES) // max(per_set, 1)))) if per_set < L2_BYTES else 1
    calls = [make_call(tensors)]
    for _ in range(n - 1):
        calls.append(make_call([None if t is None else t.clone() for t in tensors]))
    state = {"i": 0}

    def fn():
        calls[state["i"] % n]()
        state["i"] += 1

    fn.n_sets = n
    return fn


def gemm_case(op, m, n, k, dtype=torch.float16, gamma=True, split_k=0):
    """(callable, flops, algorithmic bytes) for one GEMM-family configuration."""
    g = _gen()
    x = torch.randn(m, k, generator=g).to(dtype).cuda()
    w0 = (torch.randn(k, n, generator=g) / k ** 0.5).to(dtype).cuda()
    out = torch.empty(m, n, dtype=dtype, device="cuda")
    esz = 2
    if op == "matmul":
        fn = _rotating(lambda t: (lambda: ops.matmul(t[0], t[1], split_k=split_k, out=t[2])), [x, w0, out])
        return fn, 2 * m * n * k, (m * k + k * n + m * n) * esz
    if op == "rmsnorm_matmul":
        gm = (1 + 0.1 * torch.randn(k, generator=g)).to(dtype).cuda() if gamma else None
        fn = _rotating(lambda t: (lambda: ops.rmsnorm_matmul(t[0], t[1], eps=1e-6, gamma=t[3], split_k=split_k, out=t[2])),
                       [x, w0, out, gm])
        return fn, 2 * m * n * k, (m * k + k * n + m * n + (k if gamma else 0)) * esz
    if op == "swiglu":
        w1 = (torch.randn(k, n, generator=g) / k ** 0.5).to(dtype).cuda()
        fn = _rotating(lambda t: (lambda: ops.swiglu(t[0], t[1], t[3], split_k=split_k, out=t[2])), [x, w0, out, w1])
        return fn, 4 * m * n * k, (m * k + 2 * k * n + m * n) * esz
    raise KeyError(op)


def gqa_decode_case(batch=8, hq=32, hkv=8, d=128, skv=8192, dtype=torch.float16):
    g = _gen()
    q = torch.randn(batch * hq, 1, d, generator=g).to(dtype).cuda()
    k = torch.randn(batch * hkv, skv, d, generator=g).to(dtype).cuda()
    v = torch.randn(batch * hkv, skv, d, generator=g).to(dtype).cuda()
    out = torch.empty_like(q)
    byts = (2 * k.numel() + 2 * q.numel()) * 2
    fn = _rotating(lambda t: (lambda: ops.attention_decode(t[0], t[1], t[2], out=t[3])), [q, k, v, out])
    return fn, 4 * batch * hq * skv * d, byts


def mla_decode_case(batch=16, heads=128, skv=4096, dtype=torch.bfloat16):
    g = _gen()
    q = torch.randn(batch, heads, 512, generator=g).to(dtype).cuda()
    qp = torch.randn(batch, heads, 64, generator=g).to(dtype).cuda()
    kv = torch.randn(batch, skv, 512, generator=g).to(dtype).cuda()
    kp = torch.randn(batch, skv, 64, generator=g).to(dtype).cuda()
    out = torch.empty_like(q)
    flops = 2 * batch * heads * skv * (576 + 512)
    byts = (kv.numel() + kp.numel() + q.numel() + qp.numel() + out.numel()) * 2
    fn = _rotating(lambda t: (lambda: ops.mla_decode(t[0], t[1], t[2], t[3], 192 ** -0.5, out=t[4])), [q, kv, qp, kp, out])
    return fn, flops, byts


def attn_prefill_case(hq=32, hkv=32, s=4096, d=64, dtype=torch.float16, causal=False):
    g = _gen()
    q = torch.randn(hq, s, d, generator=g).to(dtype).cuda()
    k = torch.randn(hkv, s, d, generator=g).to(dtype).cuda()
    v = torch.randn(hkv, s, d, generator=g).to(dtype).cuda()
    out = torch.empty_like(q)
    flops = 4 * hq * s * s * d // (2 if causal else 1)
    byts = (2 * q.numel() + 2 * k.numel()) * 2
    fn = _rotating(lambda t: (lambda: ops.attention_prefill(t[0], t[1], t[2], causal=causal, out=t[3])), [q, k, v, out])
    return fn, flops, byts


def fused_attn_case(kind, hq, hkv, s, d, dtype=torch.float16, impl="auto"):
    """(Q K^T) V without softmax (demo/matmul_matmul.py) or QK-norm attention (demo/qknorm.py) at demo size."""
    g = _gen()
    q = torch.randn(hq, s, d, generator=g).to(dtype).cuda()
    k = torch.randn(hkv, s, d, generator=g).to(dtype).cuda()
    v = (torch.randn(hkv, s, d, generator=g) / (s * d) ** 0.5 if kind == "matmul_matmul" else torch.randn(hkv, s, d, generator=g)).to(dtype).cuda()
    out = torch.empty_like(q)
    byts = (2 * q.numel() + 2 * k.numel()) * 2
    if kind == "matmul_matmul":
        fn = _rotating(lambda t: (lambda: ops.matmul_matmul(t[0], t[1], t[2], out=t[3], impl=impl)), [q, k, v, out])
        if impl != "scores_first":  # the chain order Q (K^T V) does 2 (HKV SKV + HQ SQ) D^2 FLOPs, not 4 HQ SQ SKV D
            return fn, 2 * (hkv * s + hq * s) * d * d, byts
    else:
        fn = _rotating(lambda t: (lambda: ops.qknorm_attention(t[0], t[1], t[2], eps=1e-6, out=t[3])), [q, k, v, out])
    return fn, 4 * hq * s * s * d, byts


def rowsum_case(m=4096, n=4096, k=64, dtype=torch.float16):
    """rowsum(X @ W) (demo/matmul_rowsum.py); FLOPs are the operator's nominal 2 M N K, bytes X + W + y."""
    g = _gen()
    x = torch.randn(m, k, generator=g).to(dtype).cuda()
    w = (torch.randn(k, n, generator=g) / k ** 0.5).to(dtype).cuda()
    out = torch.empty(m, 1, dtype=dtype, device="cuda")
    fn = _rotating(lambda t: (lambda: ops.matmul_rowsum(t[0], t[1], out=t[2])), [x, w, out], max_sets=16)
    return fn, 2 * m * n * k, (m * k + k * n + m) * 2


def lora_case(m=16, n=4096, k=4096, r=16, dtype=torch.float16):
    """LoRA (demo/lora.py): bytes X + W + A + B + Y, FLOPs 2 M K N + 2 M K R + 2 M R N."""
    g = _gen()
    x = torch.randn(m, k, generator=g).to(dtype).cuda()
    w = (torch.randn(k, n, generator=g) / k ** 0.5).to(dtype).cuda()
    a = (torch.randn(k, r, generator=g) / k ** 0.5).to(dtype).cuda()
    b = (torch.randn(r, n, generator=g) / r ** 0.5).to(dtype).cuda()
    out = torch.empty(m, n, dtype=dtype, device="cuda")
    fn = _rotating(lambda t: (lambda: ops.lora(t[0], t[1], t[2], t[3], out=t[4])), [x, w, a, b, out])
    return fn, 2 * m * k * n + 2 * m * k * r + 2 * m * r * n, (m * k + k * n + k * r + r * n + m * n) * 2


def attn_prefill_case_rect(hq, hkv, sq, skv, d, dtype=torch.float16):
    """Unsplit attention with S_Q != S_KV (demo/mha_decode_exact.py: 64 query rows over 256 keys)."""
    g = _gen()
    q = torch.randn(hq, sq, d, generator=g).to(dtype).cuda()
    k = torch.randn(hkv, skv, d, generator=g).to(dtype).cuda()
    v = torch.randn(hkv, skv, d, generator=g).to(dtype).cuda()
    out = torch.empty_like(q)
    fn = _rotating(lambda t: (lambda: ops.attention_prefill(t[0], t[1], t[2], out=t[3])), [q, k, v, out], max_sets=16)
    return fn, 4 * hq * sq * skv * d, (2 * q.numel() + 2 * k.numel()) * 2


def paged_decode_case(page_size=1, batch=64, hi=8192, lo=512):
    """Paged GQA decode (32 / 8 heads, d 128, bf16) over a cache far larger than L2; page size 1 takes
    the row-gather path. Small ``batch`` and ``hi`` give the batches of a few short requests on which the fixed
    cost of a launch is all there is to see."""
    from cleave_b200.workloads import paged_decode_workload

    w = paged_decode_workload(batch=batch, page_size=page_size, lo=lo, hi=hi, dtype=torch.bfloat16)
    out = torch.empty_like(w.q)
    lse = torch.empty(w.q.shape[0], w.q.shape[1], dtype=torch.float32, device="cuda")
    last = None if page_size == 1 else w.kv_last_page_len
    fn = lambda: ops.gqa_paged_decode(w.q, w.k_cache, w.v_cache, w.kv_indptr, w.kv_indices, last, w.sm_scale,  # noqa: E731
                                      out=out, lse=lse)
    return fn, w.flops(), w.algorithmic_bytes()


def gqa_dynamic_prefill_case(paged, batch=8, q_len=2048, hq=32, hkv=8, d=128, dtype=torch.bfloat16, kv_len=None, light=True):
    """Ragged or paged (one token per page) causal prefill: whole prompts, or with ``kv_len`` far below ``q_len`` a
    chunk whose key window is much shorter than its run of query rows (only the last kv_len rows of a request see a
    key); ``light=False`` keeps such a chunk on the tcgen05 kernel."""
    g = _gen()
    kv_len = q_len if kv_len is None else kv_len
    tq, tk = batch * q_len, batch * kv_len
    q = torch.randn(tq, hq, d, generator=g).to(dtype).cuda()
    qo = (torch.arange(batch + 1, dtype=torch.int32) * q_len).cuda()
    kv = (torch.arange(batch + 1, dtype=torch.int32) * kv_len).cuda()
    out = torch.empty_like(q)
    lse = torch.empty(tq, hq, dtype=torch.float32, device="cuda")
    vis = min(q_len, kv_len)
    flops = 4 * batch * hq * (vis * (vis + 1) // 2 + vis * (kv_len - vis)) * d
    if paged:
        num_pages = tk + 8
        kc = torch.randn(num_pages, 1, hkv, d, generator=g).to(dtype).cuda()
        vc = torch.randn(num_pages, 1, hkv, d, generator=g).to(dtype).cuda()
        idx = torch.randperm(num_pages, generator=g)[:tk].to(torch.int32).cuda()
        call = lambda: ops.gqa_paged_prefill(q, kc, vc, qo, kv, idx, d ** -0.5, out=out, lse=lse)  # noqa: E731
        byts = (q.numel() + q.numel() * vis // q_len + 2 * kc.numel()) * 2  # out, the rows of Q that see a key, the caches
    else:
        k = torch.randn(tk, hkv, d, generator=g).to(dtype).cuda()
        v = torch.randn(tk, hkv, d, generator=g).to(dtype).cuda()
        call = lambda: ops.gqa_ragged_prefill(q, k, v, qo, kv, d ** -0.5, out=out, lse=lse)  # noqa: E731
        byts = (q.numel() + q.numel() * vis // q_len + 2 * k.numel()) * 2
    if light:
        return call, flops, byts

    def tile_kernels_only():
        old = ops.set_small_problem_limit(0)
        try:
            return call()
        finally:
            ops.set_small_problem_limit(old)

    return tile_kernels_only, flops, byts


def mla_paged_decode_case(batch=64, heads=16, lo=512, hi=8192, dtype=torch.bfloat16, impl="auto"):
    """Paged MLA decode (one token per page, 16 heads as the reference's shipped operator)."""
    g = _gen()
    lens = torch.randint(lo, hi + 1, (batch,), generator=g)
    total = int(lens.sum())
    num_pages = total + 8
    qn = torch.randn(batch, heads, 512, generator=g).to(dtype).cuda()
    qp = torch.randn(batch, heads, 64, generator=g).to(dtype).cuda()
    ckv = torch.randn(num_pages, 1, 512, dtype=dtype, device="cuda")
    kpe = torch.randn(num_pages, 1, 64, dtype=dtype, device="cuda")
    ptr = torch.cat([torch.zeros(1, dtype=torch.int64), lens.cumsum(0)]).to(torch.int32).cuda()
    idx = torch.randperm(num_pages, generator=g)[:total].to(torch.int32).cuda()
    out = torch.empty_like(qn)
    flops = 2 * heads * total * (576 + 512)
    byts = total * 576 * 2 + (qn.numel() + qp.numel() + out.numel()) * 2
    fn = lambda: ops.mla_paged_decode(qn, qp, ckv, kpe, ptr, idx, 0.1352337747812271, out=out, impl=impl)  # noqa: E731
    return fn, flops, byts


def mla_prefill_case(batch=4, q_len=512, heads=16, dtype=torch.bfloat16, impl="auto"):
    """Paged causal MLA prefill, whole prompts (q_len = kv_len), one token per page."""
    g = _gen()
    tq = batch * q_len
    num_pages = tq + 8
    qn = torch.randn(tq, heads, 512, generator=g).to(dtype).cuda()
    qp = torch.randn(tq, heads, 64, generator=g).to(dtype).cuda()
    ckv = torch.randn(num_pages, 1, 512, generator=g).to(dtype).cuda()
    kpe = torch.randn(num_pages, 1, 64, generator=g).to(dtype).cuda()
    ptr = (torch.arange(batch + 1, dtype=torch.int32) * q_len).cuda()
    idx = torch.randperm(num_pages, generator=g)[:tq].to(torch.int32).cuda()
    out = torch.empty_like(qn)
    lse = torch.empty(tq, heads, dtype=torch.float32, device="cuda")
    flops = 2 * batch * heads * (q_len * (q_len + 1) // 2) * (576 + 512)
    byts = (qn.numel() + qp.numel() + ckv.numel() + kpe.numel() + out.numel()) * 2
    fn = lambda: ops.mla_paged_prefill(qn, qp, ckv, kpe, ptr, ptr, idx, 0.1352337747812271, out=out, lse=lse, impl=impl)  # noqa: E731
    return fn, flops, byts


CONFIGS = {
    "cfg1_matmul_128x128x4096": lambda: gemm_case("matmul", 128, 128, 4096),
    "cfg2_rmsnorm_matmul_64x11008x4096": lambda: gemm_case("rmsnorm_matmul", 64, 11008, 4096),
    "demo_rmsnorm_matmul_4096x14336x4096": lambda: gemm_case("rmsnorm_matmul", 4096, 14336, 4096, gamma=False),
    "demo_matmul_4096x14336x4096": lambda: gemm_case("matmul", 4096, 14336, 4096),
    "demo_swiglu_4096x14336x4096": lambda: gemm_case("swiglu", 4096, 14336, 4096),
    "cfg3_gqa_decode_b8_h32_kv8_d128_s8192": lambda: gqa_decode_case(),
    "cfg4_mla_decode_b16_h128_s4096": lambda: mla_decode_case(),
    "demo_mha_prefill_h32_s4096_d64": lambda: attn_prefill_case(32, 32, 4096, 64),
    "demo_gqa_prefill_h32_kv8_s4096_d64": lambda: attn_prefill_case(32, 8, 4096, 64),
    "gqa_prefill_causal_h32_kv8_s4096_d128": lambda: attn_prefill_case(32, 8, 4096, 128, torch.bfloat16, True),
    "gqa_prefill_h32_kv8_s4096_d128": lambda: attn_prefill_case(32, 8, 4096, 128, torch.bfloat16, False),
    "demo_matmul_matmul_bh32_s4096_d64": lambda: fused_attn_case("matmul_matmul", 32, 32, 4096, 64),
    "demo_matmul_matmul_scores_first_bh32_s4096_d64": lambda: fused_attn_case("matmul_matmul", 32, 32, 4096, 64, impl="scores_first"),
    "demo_qknorm_h64_kv8_s4096_d128": lambda: fused_attn_case("qknorm", 64, 8, 4096, 128),
    "demo_mha_decode_exact_h32_sq64_skv256_d64": lambda: attn_prefill_case_rect(32, 32, 64, 256, 64),
    "demo_matmul_rowsum_4096x4096x64": lambda: rowsum_case(),
    "demo_lora_16x4096x4096_r16": lambda: lora_case(),
    "gqa_ragged_prefill_causal_h32_kv8_d128_b8_q2048": lambda: gqa_dynamic_prefill_case(False),
    "gqa_paged_prefill_causal_h32_kv8_d128_ps1_b8_q2048": lambda: gqa_dynamic_prefill_case(True),
    "mla_paged_decode_h16_ps1_b64_kv512_8192": lambda: mla_paged_decode_case(),
    "mla_paged_decode_h16_ps1_b64_kv512_8192_mma_sync": lambda: mla_paged_decode_case(impl="mma_sync"),
    "mla_paged_prefill_causal_h16_b4_q512": lambda: mla_prefill_case(),
    "mla_paged_prefill_causal_h16_b4_q512_per_token": lambda: mla_prefill_case(impl="per_token"),
    "mla_paged_prefill_causal_h16_b8_q2048": lambda: mla_prefill_case(batch=8, q_len=2048),
    "gqa_paged_decode_ps1_b64_kv512_8192": lambda: paged_decode_case(1),
    "gqa_paged_decode_ps16_b64_kv512_8192": lambda: paged_decode_case(16),
    "gqa_paged_decode_ps32_b64_kv512_8192": lambda: paged_decode_case(32),
    "gqa_paged_decode_ps64_b64_kv512_8192": lambda: paged_decode_case(64),
    # fixed cost: a handful of short requests, and a prefill chunk of 16384 query rows over a page table of 64 tokens
    "gqa_paged_decode_ps1_b1_kv8": lambda: paged_decode_case(1, batch=1, lo=8, hi=8),
    "gqa_paged_decode_ps1_b16_kv32_128": lambda: paged_decode_case(1, batch=16, lo=32, hi=128),
    "mla_paged_decode_h16_ps1_b16_kv16_64": lambda: mla_paged_decode_case(batch=16, lo=16, hi=64),
    "gqa_paged_prefill_causal_h32_kv4_d128_ps1_b32_q512_kv2": lambda: gqa_dynamic_prefill_case(True, batch=32, q_len=512, hkv=4, kv_len=2),
    "gqa_paged_prefill_causal_h32_kv4_d128_ps1_b32_q512_kv2_tile_kernels": lambda: gqa_dynamic_prefill_case(
        True, batch=32, q_len=512, hkv=4, kv_len=2, light=False),
}


def measure(name, build):
    fn, flops, byts = build()
    us = min_launch_us(fn, [], batch=20, repeats=5)
    hbm, tf, kind = _peaks()
    gbs, tfs = byts / us / 1e3, flops / us / 1e6
    return {"config": name, "us": us, "input_sets": getattr(fn, "n_sets", 1), "GB/s": gbs, "TFLOP/s": tfs,
            "hbm_frac": gbs / hbm, "tensor_frac": tfs / tf, "peaks": f"of {kind}",
            "hbm_frac_nominal": gbs / NOMINAL_HBM_GBS, "tensor_frac_nominal": tfs / NOMINAL_TFLOPS}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default=None, choices=["matmul", "rmsnorm_matmul", "swiglu", "gqa_decode", "mla_decode", "attn_prefill", "gqa_paged_ps1",
                                             "mla_paged_decode", "mla_prefill", "matmul_matmul", "qknorm", "matmul_rowsum", "lora"])
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--split-k", type=int, default=0)
    ap.add_argument("--no-gamma", action="store_true")
    ap.add_argument("--launches", type=int, default=0)
    ap.add_argument("--only", default=None, help="substring filter on the configuration names")
    a = ap.parse_args()
    if a.op:
        if a.op == "gqa_decode":
            build = gqa_decode_case
        elif a.op == "mla_decode":
            build = mla_decode_case
        elif a.op == "gqa_paged_ps1":
            build = lambda: paged_decode_case(1)  # noqa: E731
        elif a.op == "mla_paged_decode":
            build = mla_paged_decode_case
        elif a.op == "mla_prefill":
            build = lambda: mla_prefill_case(batch=8, q_len=2048)  # noqa: E731
        elif a.op == "matmul_matmul":
            build = lambda: fused_attn_case("matmul_matmul", 32, 32, 4096, 64)  # noqa: E731
        elif a.op == "qknorm":
            build = lambda: fused_attn_case("qknorm", 64, 8, 4096, 128)  # noqa: E731
        elif a.op == "matmul_rowsum":
            build = rowsum_case
        elif a.op == "lora":
            build = lora_case
        elif a.op == "attn_prefill":
            build = lambda: attn_prefill_case(32, 8, a.m, a.k if a.k in (64, 128) else 128, torch.bfloat16, False)  # noqa: E731
        else:
            build = lambda: gemm_case(a.op, a.m, a.n, a.k, gamma=not a.no_gamma, split_k=a.split_k)  # noqa: E731
        if a.launches:
            fn, _, _ = build()
            for _ in range(3 + a.launches):
                fn()
            torch.cuda.synchronize()
            print(f"ran {a.launches} launches of {a.op}")
            return
        print(json.dumps(measure(f"{a.op}_{a.m}x{a.n}x{a.k}", build)))
        return
    for name, build in CONFIGS.items():
        if a.only and a.only not in name:
            continue
        print(json.dumps(measure(name, build)), flush=True)
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
