"""Generates ``plans.json``: structural records of REAL scheduled plans of the reference.

    python tests/golden/make_plans.py [case ...]        # default: every case; merges into plans.json

For each program below the reference's own producer is run (``superoptimize`` -> ``schedule``,
python/cleave/pipeline/compile.py:124-128) inside the environment of ``reference_env.py``; every resulting
``Plan`` (python/cleave/pipeline/plans.py:16-41) is reduced to what a code generator reads off it - node class
names, node names, shapes, dtypes, the constants of element-wise nodes, matmul flags, reduction axes, the
edges, and the plan's variant / role / split factor / input binding - and plans that agree in all of that
(they differ in tile hints only) are stored once with a count. ``plans.py`` rebuilds light objects with the
same attribute surface from the file, so tests of the plan -> kernel-text seam run where the reference is
absent. Nothing but these structural records leaves the reference.
"""

import json
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "plans.json")
NODE_ATTRS = ("const", "const_on_left", "axis", "transpose_A", "transpose_B", "M", "N", "K", "keepdims")


def programs(cleave, cl):
    """name -> (program or jit function, shapes, dtype, split, superopt keywords, schedule keywords)."""

    @cleave.jit
    def matmul(x: cl.Tensor["M", "K"], w: cl.Tensor["K", "N"]):
        return x @ w

    @cleave.jit
    def rmsnorm_matmul(x: cl.Tensor["M", "K"], w: cl.Tensor["K", "N"]):
        return cl.rms_norm(x, dim=-1, eps=1e-6) @ w

    @cleave.jit
    def swiglu(x: cl.Tensor["M", "K"], w0: cl.Tensor["K", "N"], w1: cl.Tensor["K", "N"]):
        gate, up = x @ w0, x @ w1
        return cl.silu(gate) * up

    def attention(q, k, v):
        n = q.shape[-1] ** 0.5
        return cl.softmax((q @ k.mT) / n, dim=-1, shift=-50 / n) @ v

    @cleave.jit
    def gqa_decode(q: cl.Tensor["HQ", "SQ", "D"], k: cl.Tensor["HKV", "SKV", "D"], v: cl.Tensor["HKV", "SKV", "D"]):
        return attention(q, k, v)

    @cleave.jit
    def mla_decode(q: cl.Tensor["B", "H", "D"], kv: cl.Tensor["B", "SKV", "D"],
                   q_pe: cl.Tensor["B", "H", "PE"], k_pe: cl.Tensor["B", "SKV", "PE"]):
        n = 192 ** 0.5
        s = (q @ kv.mT + q_pe @ k_pe.mT) / n
        return cl.softmax(s, dim=-1, shift=-50 / n) @ kv

    @cleave.jit
    def matmul_matmul(q: cl.Tensor["BH", "SQ", "D"], k: cl.Tensor["BH", "SKV", "D"], v: cl.Tensor["BH", "SKV", "D"]):
        return (q @ k.mT) @ v

    @cleave.jit
    def matmul_rowsum(x: cl.Tensor["M", "K"], w: cl.Tensor["K", "N"]):
        return (x @ w).sum(-1, keepdim=True)

    @cleave.jit
    def mha_decode_exact(q: cl.Tensor["H", "SQ", "D"], k: cl.Tensor["H", "SKV", "D"], v: cl.Tensor["H", "SKV", "D"]):
        return cl.softmax((q @ k.mT) / q.shape[-1] ** 0.5, dim=-1) @ v

    def lora():
        p = cleave.Program("lora", dtype=cl.f16)
        M, K, N, R = p.dims(M=16, K=4096, N=4096, R=16)
        x, w = p.input("x", (M, K)), p.input("w", (K, N))
        a, b = p.input("a", (K, R)), p.input("b", (R, N))
        p.output(x @ w + (x @ a) @ b, name="y")
        return p

    S = cl.Split
    return {
        "cfg1_matmul": (matmul, dict(M=128, N=128, K=4096), cl.f16, S("K", (4, 8, 16)), {}, {}),
        "cfg2_rmsnorm_matmul_eps": (rmsnorm_matmul, dict(M=64, N=11008, K=4096), cl.f16, S("K", (4, 8, 16)), {}, {}),
        "swiglu": (swiglu, dict(M=64, N=11008, K=4096), cl.f16, None, {}, {}),
        "cfg3_gqa_decode": (gqa_decode, dict(HQ=256, HKV=64, SQ=1, SKV=8192, D=128), cl.f16, S("SKV", (4, 8, 16)),
                            dict(max_ops=14), {}),
        "cfg4_mla_decode": (mla_decode, dict(B=16, H=128, SKV=4096, D=512, PE=64), cl.bf16, None, dict(max_ops=13), {}),
        "demo_matmul_matmul": (matmul_matmul, dict(BH=32, SQ=4096, SKV=4096, D=64), cl.f16, None, {}, {}),
        "demo_matmul_rowsum": (matmul_rowsum, dict(M=4096, N=4096, K=64), cl.f16, None, {}, {}),
        "demo_mha_decode_exact": (mha_decode_exact, dict(H=32, SQ=64, SKV=256, D=64), cl.f16, False, dict(max_ops=14), {}),
        "demo_lora": (lora(), None, None, None, {}, {}),
    }


def node_record(n):
    rec = {"type": type(n).__name__, "name": getattr(n, "name", None)}
    try:
        rec["shape"] = [int(s) for s in n.get_shape(0)]
    except Exception:  # noqa: BLE001
        rec["shape"] = None
    try:
        rec["dtype"] = str(n.get_dtype(0))
    except Exception:  # noqa: BLE001
        rec["dtype"] = None
    for a in NODE_ATTRS:
        if hasattr(n, a):
            v = getattr(n, a)
            if v is None or isinstance(v, (bool, int, float, str)):
                rec[a] = v
    rec["inputs"] = [getattr(getattr(e, "src_node", None), "name", None) for e in getattr(n, "inputs", [])]
    return rec


def plan_record(plan):
    return {"variant": plan.variant, "role": plan.role, "split_factor": plan.split_factor,
            "inputs": None if plan.inputs is None else list(plan.inputs),
            "nodes": [node_record(n) for n in plan.tile.flat_graph.nodes]}


def run_case(cleave, cl, entry):
    from cleave.pipeline.compile import as_program, resolve_configs
    from cleave.pipeline.config import ScheduleConfig, SuperoptConfig
    from cleave.pipeline.plans import schedule
    from cleave.pipeline.superopt import superoptimize

    fn, shapes, dtype, split, so_kw, sc_kw = entry
    program = as_program(fn, shapes, dtype)
    so, sc, _ = resolve_configs(program, preset="default", superopt=SuperoptConfig(**so_kw) if so_kw else None,
                                schedule=ScheduleConfig(**sc_kw) if sc_kw else None, eval=None, split=split)
    t0 = time.time()
    graphs = superoptimize(program, so.replace(cache=False))
    plans = schedule(graphs, sc)
    distinct, counts = {}, {}
    for p in plans:
        rec = plan_record(p)
        key = json.dumps(rec, sort_keys=True)
        counts[key] = counts.get(key, 0) + 1
        distinct.setdefault(key, rec)
    out = []
    for key, rec in distinct.items():
        rec["count"] = counts[key]
        out.append(rec)
    return {"program_inputs": [[s.name, [int(d) for d in s.shape]] for s in program.inputs],
            "dtype": str(program.dtype), "graphs": len(graphs), "plans": len(plans),
            "refused": len(plans.refused), "seconds": round(time.time() - t0, 1), "records": out}


def main(argv):
    sys.path.insert(0, HERE)
    import reference_env

    cleave = reference_env.activate()
    import cleave.lang as cl

    catalogue = programs(cleave, cl)
    wanted = argv or list(catalogue)
    data = json.load(open(OUT)) if os.path.exists(OUT) else {}
    for name in wanted:
        print(f"[make_plans] {name} ...", flush=True)
        data[name] = run_case(cleave, cl, catalogue[name])
        print(f"[make_plans] {name}: {data[name]['plans']} plans, {len(data[name]['records'])} distinct, "
              f"{data[name]['seconds']} s", flush=True)
        with open(OUT, "w") as f:
            json.dump(data, f, indent=1, sort_keys=True)


if __name__ == "__main__":
    main(sys.argv[1:])
