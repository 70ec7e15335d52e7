"""Generate ``golden.npz`` by running the REFERENCE's own torch code on the seeded cases.

Run where the reference checkout is available::

    python tests/golden/make_golden.py /path/to/reference

Static operators go through ``cleave.trace(...).reference`` (``python/cleave/frontend/program.py:296``),
paged operators through the closures of ``python/cleave/dynamic/reference.py`` (loaded by file
path, because importing ``cleave.dynamic`` needs the TileLang fork). The reference tree is only
read; nothing from it is copied. Outputs are stored in their own 16-bit storage type (lse as float32).
"""


import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import cases  # noqa: E402


def _t(a, dtype):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if t.dtype == torch.float32:
        return t.to({"f16": torch.float16, "bf16": torch.bfloat16}[dtype])
    return t


def main(ref_root):
    sys.path.insert(0, os.path.join(ref_root, "python"))
    import cleave
    import cleave.lang as cl

    spec = importlib.util.spec_from_file_location(
        "_ref_dynamic_reference", os.path.join(ref_root, "python/cleave/dynamic/reference.py"))
    dyn = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(dyn)

    cdt = {"f16": cl.f16, "bf16": cl.bf16}

    def matmul(x: cl.Tensor["M", "K"], w: cl.Tensor["K", "N"]):
        return x @ w

    def swiglu(x: cl.Tensor["M", "K"], w0: cl.Tensor["K", "N"], w1: cl.Tensor["K", "N"]):
        gate, up = x @ w0, x @ w1
        return cl.silu(gate) * up

    def attention(q: cl.Tensor["HQ", "SQ", "D"], k: cl.Tensor["HKV", "SKV", "D"],
                  v: cl.Tensor["HKV", "SKV", "D"]):
        n = q.shape[-1] ** 0.5
        return cl.softmax((q @ k.mT) / n, dim=-1, shift=-50 / n) @ v

    out = {}
    for name in cases.CASES:
        family, inp, opt = cases.build(name)
        dt = opt["dtype"]
        if family == "matmul":
            m, k = inp["x"].shape
            prog = cleave.trace(matmul, shapes=dict(M=m, K=k, N=inp["w0"].shape[1]), dtype=cdt[dt])
            res = prog.reference(_t(inp["x"], dt), _t(inp["w0"], dt))
        elif family == "rmsnorm_matmul":
            m, k = inp["x"].shape
            eps = opt["eps"]
            if "gamma" in inp:
                def fn(x: cl.Tensor["M", "K"], g: cl.Tensor[1, "K"], w: cl.Tensor["K", "N"]):
                    return (cl.rms_norm(x, dim=-1, eps=eps) * g) @ w
                prog = cleave.trace(fn, shapes=dict(M=m, K=k, N=inp["w0"].shape[1]), dtype=cdt[dt])
                res = prog.reference(_t(inp["x"], dt), _t(inp["gamma"][None, :], dt), _t(inp["w0"], dt))
            else:
                def fn(x: cl.Tensor["M", "K"], w: cl.Tensor["K", "N"]):
                    return cl.rms_norm(x, dim=-1, eps=eps) @ w
                prog = cleave.trace(fn, shapes=dict(M=m, K=k, N=inp["w0"].shape[1]), dtype=cdt[dt])
                res = prog.reference(_t(inp["x"], dt), _t(inp["w0"], dt))
        elif family == "swiglu":
            m, k = inp["x"].shape
            prog = cleave.trace(swiglu, shapes=dict(M=m, K=k, N=inp["w0"].shape[1]), dtype=cdt[dt])
            res = prog.reference(_t(inp["x"], dt), _t(inp["w0"], dt), _t(inp["w1"], dt))
        elif family == "attention":
            hq, sq, d = inp["q"].shape
            hkv, skv, _ = inp["k"].shape
            prog = cleave.trace(attention, shapes=dict(HQ=hq, HKV=hkv, SQ=sq, SKV=skv, D=d), dtype=cdt[dt])
            res = prog.reference(_t(inp["q"], dt), _t(inp["k"], dt), _t(inp["v"], dt))
        elif family == "attention_exact":
            def fn(q: cl.Tensor["H", "SQ", "D"], k: cl.Tensor["H", "SKV", "D"], v: cl.Tensor["H", "SKV", "D"]):
                return cl.softmax((q @ k.mT) / q.shape[-1] ** 0.5, dim=-1) @ v
            h, sq, d = inp["q"].shape
            prog = cleave.trace(fn, shapes=dict(H=h, SQ=sq, SKV=inp["k"].shape[1], D=d), dtype=cdt[dt])
            res = prog.reference(_t(inp["q"], dt), _t(inp["k"], dt), _t(inp["v"], dt))
        elif family == "matmul_matmul":
            def fn(q: cl.Tensor["HQ", "SQ", "D"], k: cl.Tensor["HKV", "SKV", "D"], v: cl.Tensor["HKV", "SKV", "D"]):
                return (q @ k.mT) @ v
            hq, sq, d = inp["q"].shape
            hkv, skv, _ = inp["k"].shape
            prog = cleave.trace(fn, shapes=dict(HQ=hq, HKV=hkv, SQ=sq, SKV=skv, D=d), dtype=cdt[dt])
            res = prog.reference(_t(inp["q"], dt), _t(inp["k"], dt), _t(inp["v"], dt))
        elif family == "qknorm":
            eps = opt["eps"]

            def fn(q: cl.Tensor["HQ", "SQ", "D"], k: cl.Tensor["HKV", "SKV", "D"], v: cl.Tensor["HKV", "SKV", "D"]):
                q_sq, k_sq = q * q, k * k
                q_ms, k_ms = q_sq.mean(-1, keepdim=True), k_sq.mean(-1, keepdim=True)
                qn = q * cl.rsqrt(q_ms + eps)
                kn = k * cl.rsqrt(k_ms + eps)
                n = qn.shape[-1] ** 0.5
                return cl.softmax((qn @ kn.mT) / n, dim=-1, shift=-50 / n) @ v
            hq, sq, d = inp["q"].shape
            hkv, skv, _ = inp["k"].shape
            prog = cleave.trace(fn, shapes=dict(HQ=hq, HKV=hkv, SQ=sq, SKV=skv, D=d), dtype=cdt[dt])
            res = prog.reference(_t(inp["q"], dt), _t(inp["k"], dt), _t(inp["v"], dt))
        elif family == "matmul_rowsum":
            def fn(x: cl.Tensor["M", "K"], w: cl.Tensor["K", "N"]):
                return (x @ w).sum(-1, keepdim=True)
            m, k = inp["x"].shape
            prog = cleave.trace(fn, shapes=dict(M=m, K=k, N=inp["w0"].shape[1]), dtype=cdt[dt])
            res = prog.reference(_t(inp["x"], dt), _t(inp["w0"], dt))
        elif family == "lora":
            m, k = inp["x"].shape
            prog = cleave.Program("lora", dtype=cdt[dt])
            M, K, N, R = prog.dims(M=m, K=k, N=inp["w"].shape[1], R=inp["a"].shape[1])
            x, w = prog.input("x", (M, K)), prog.input("w", (K, N))
            a, b = prog.input("a", (K, R)), prog.input("b", (R, N))
            prog.output(x @ w + (x @ a) @ b, name="y")
            res = prog.reference(*[_t(inp[n], dt) for n in ("x", "w", "a", "b")])
        elif family == "mla":
            scale = opt["scale"]

            def fn(q: cl.Tensor["B", "H", "D"], kv: cl.Tensor["B", "SKV", "D"],
                   q_pe: cl.Tensor["B", "H", "PE"], k_pe: cl.Tensor["B", "SKV", "PE"]):
                s = (q @ kv.mT + q_pe @ k_pe.mT) * scale
                return cl.softmax(s, dim=-1, shift=-50 * scale) @ kv
            b, h, d = inp["q"].shape
            prog = cleave.trace(fn, shapes=dict(B=b, H=h, D=d, SKV=inp["kv"].shape[1],
                                                PE=inp["q_pe"].shape[2]), dtype=cdt[dt])
            res = prog.reference(*[_t(inp[n], dt) for n in ("q", "kv", "q_pe", "k_pe")])
        elif family == "gqa_paged":
            batch, hq, d = inp["q"].shape
            num_pages, ps, hkv, _ = inp["k_cache"].shape
            dims = (batch, hq, hkv, d, num_pages, inp["kv_indices"].size)
            ref = dyn.gqa_paged_decode_reference(dims, opt["kv_lens"], page_size=ps)
            args = [_t(inp["q"], dt), _t(inp["k_cache"], dt), _t(inp["v_cache"], dt),
                    _t(inp["kv_indptr"], dt), _t(inp["kv_indices"], dt)]
            if ps != 1:
                args.append(_t(inp["kv_last_page_len"], dt))
            args.append(inp["sm_scale"])
            res = ref(*args)
        elif family == "mla_paged":
            batch, h, ckv = inp["q_nope"].shape
            dims = (batch, h, ckv, inp["q_pe"].shape[2], inp["ckv_cache"].shape[0], inp["kv_indices"].size)
            ref = dyn.mla_paged_decode_reference(dims, opt["kv_lens"])
            res = ref(_t(inp["q_nope"], dt), _t(inp["q_pe"], dt), _t(inp["ckv_cache"], dt),
                      _t(inp["kpe_cache"], dt), _t(inp["kv_indptr"], dt), _t(inp["kv_indices"], dt),
                      inp["sm_scale"])
        elif family == "mla_prefill":
            tq, h, ckv = inp["q_nope"].shape
            dims = (h, ckv, inp["q_pe"].shape[2], inp["ckv_cache"].shape[0], inp["kv_indices"].size, tq)
            ref = dyn.mla_paged_prefill_reference(dims, opt["q_lens"], opt["kv_lens"])
            res = ref(_t(inp["q_nope"], dt), _t(inp["q_pe"], dt), _t(inp["ckv_cache"], dt), _t(inp["kpe_cache"], dt),
                      _t(inp["qo_indptr"], dt), _t(inp["kv_indptr"], dt), _t(inp["kv_indices"], dt), inp["sm_scale"])
        elif family == "gqa_prefill":
            tq, hq, d = inp["q"].shape
            if opt["paged"]:
                num_pages, _, hkv, _ = inp["k_cache"].shape
                dims = (hq, hkv, d, num_pages, inp["kv_indices"].size, tq)
                ref = dyn.gqa_paged_prefill_reference(dims, opt["q_lens"], opt["kv_lens"])
                res = ref(_t(inp["q"], dt), _t(inp["k_cache"], dt), _t(inp["v_cache"], dt), _t(inp["qo_indptr"], dt),
                          _t(inp["kv_indptr"], dt), _t(inp["kv_indices"], dt), inp["sm_scale"])
            else:
                tk, hkv, _ = inp["k"].shape
                dims = (hq, hkv, d, tq, tk)
                ref = dyn.gqa_ragged_prefill_reference(dims, opt["q_lens"], opt["kv_lens"])
                res = ref(_t(inp["q"], dt), _t(inp["k"], dt), _t(inp["v"], dt), _t(inp["qo_indptr"], dt),
                          _t(inp["kv_indptr"], dt), inp["sm_scale"])
        else:
            raise KeyError(family)
        for i, r in enumerate(res):
            # bf16 / f16 outputs are stored as their 16-bit patterns (see cases.load_golden)
            if r.dtype == torch.bfloat16:
                out[f"{name}/{i}:bf16"] = (r.float().numpy().view(np.uint32) >> 16).astype(np.uint16)
            elif r.dtype == torch.float16:
                out[f"{name}/{i}:f16"] = r.numpy()
            else:
                out[f"{name}/{i}:f32"] = r.float().numpy()
        print(name, [tuple(r.shape) for r in res])
    np.savez_compressed(os.path.join(HERE, "golden.npz"), **out)
    print("wrote", os.path.join(HERE, "golden.npz"), os.path.getsize(os.path.join(HERE, "golden.npz")), "bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/reference")
    main(sys.argv[1])
