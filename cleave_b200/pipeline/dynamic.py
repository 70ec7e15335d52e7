"""Paged (dynamic-shape) operators: validate over workloads, time, return a ``PagedKernel``
(the call surface of python/cleave/pipeline/dynamic.py:246-504).

The reference searches tilings of a dense attention body, wraps each in a paged access layer,
validates every candidate on every workload and calibrates a split-vs-single dispatch
threshold. Here one persistent kernel deals KV tiles evenly to the SMs whatever the length
distribution. ``calibrate_dispatch`` still measures the reference's question on it - does a
workload with short requests run better on a small grid whose CTAs keep whole items than on
the full grid that cuts them - and the report carries the answer with the reference's field
names; the threshold is applied only if the hybrid beats the full grid by a margin.
"""

from __future__ import annotations

import json
import math
import time
from dataclasses import dataclass, field

from ..codegen import B200CodeGen, make_spec
from ..core.errors import CleaveError, PagingRefusal
from ..runtime.validate import PAGED_TOLERANCE
from .config import resolve_eval
from .kernel import Kernel, Stage

# operator name -> (family, names of the traced signature in order, the dims a caller must give)
OPERATORS = {
    "gqa_paged_decode": ("gqa_paged_decode",
                         ("q", "k_cache", "v_cache", "kv_indptr", "kv_indices", "kv_last_page_len", "sm_scale"),
                         ("num_qo_heads", "num_kv_heads", "head_dim", "page_size")),
    "mla_paged_decode": ("mla_paged_decode",
                         ("q_nope", "q_pe", "ckv_cache", "kpe_cache", "kv_indptr", "kv_indices", "sm_scale"),
                         ("num_qo_heads", "head_dim_ckv", "head_dim_kpe")),
    "gqa_ragged_prefill_causal": ("gqa_ragged_prefill",
                                  ("q", "k", "v", "qo_indptr", "kv_indptr", "sm_scale"),
                                  ("num_qo_heads", "num_kv_heads", "head_dim")),
    "gqa_paged_prefill_causal": ("gqa_paged_prefill",
                                 ("q", "k_cache", "v_cache", "qo_indptr", "kv_indptr", "kv_indices", "sm_scale"),
                                 ("num_qo_heads", "num_kv_heads", "head_dim")),
    "mla_paged_prefill_causal": ("mla_paged_prefill",
                                 ("q_nope", "q_pe", "ckv_cache", "kpe_cache", "qo_indptr", "kv_indptr", "kv_indices", "sm_scale"),
                                 ("num_qo_heads", "head_dim_ckv", "head_dim_kpe")),
}
PREFILL_FAMILIES = ("gqa_ragged_prefill", "gqa_paged_prefill", "mla_paged_prefill")


def paged_decode_workloads(batches=(1, 7, 64), kv_points=6, kv_max=8192, seed=0):
    """``[(key, kv_lens)]``: batch sizes x log-spaced KV lengths in [1, kv_max], ragged around each
    point - the reference's own synthetic generator (python/cleave/frontend/paged.py:575-614) stands in
    for its captured benchmark axes, whose trace files cannot be redistributed."""
    import random

    rnd = random.Random(seed)
    out = []
    for b in batches:
        for i in range(kv_points):
            centre = max(1, round(kv_max ** (i / (kv_points - 1))))
            lens = [max(1, min(kv_max, round(centre * rnd.uniform(0.5, 1.0)))) for _ in range(b)]
            if b > 1:
                lens[rnd.randrange(b)] = centre
            out.append((f"wl_{b}_{centre}", lens))
    return out


def paged_prefill_workloads(batches=(1, 5), kv_points=4, kv_max=2048, seed=0):
    """``[(key, (q_lens, kv_lens))]``: whole-prompt prefill (q_len = kv_len) and chunked prefill (a query
    suffix of an existing context), with an empty request in every batch larger than one - the lengths
    python/cleave/dynamic/workloads.py draws for the prefill operators, generated here."""
    import random

    rnd = random.Random(seed)
    out = []
    for b in batches:
        for i in range(kv_points):
            centre = max(2, round(kv_max ** ((i + 1) / kv_points)))
            kv = [max(1, round(centre * rnd.uniform(0.5, 1.0))) for _ in range(b)]
            ql = [n if rnd.random() < 0.5 else max(1, n // rnd.choice((2, 3, 8))) for n in kv]
            if b > 1:
                ql[rnd.randrange(b)] = 0
            out.append((f"b{b}_kv{centre}", (ql, kv)))
    return out


def make_inputs(family, dims, kv_lens, dtype, device="cuda", seed=0):
    """The operator's tensors in its declared order (reference: python/cleave/dynamic/reference.py:156-177,
    282-294): random permutation page table, N(0,1) tensors, pool three pages larger than needed."""
    import torch

    from ..runtime.reference import torch_dtype

    dt = torch_dtype(dtype)
    g = torch.Generator(device="cpu").manual_seed(seed)
    if family in PREFILL_FAMILIES:
        q_lens, kv_lens = kv_lens
        rn = lambda *s: torch.randn(*s, generator=g).to(dt).to(device)  # noqa: E731
        ptr = lambda ls: torch.tensor([0] + list(torch.tensor(ls).cumsum(0).tolist()), dtype=torch.int32, device=device)  # noqa: E731
        tq, tk = max(1, sum(q_lens)), sum(kv_lens)
        if family == "mla_paged_prefill":
            h, c, k = dims["num_qo_heads"], dims["head_dim_ckv"], dims["head_dim_kpe"]
            num_pages = tk + 3
            idx = torch.randperm(num_pages, generator=g)[:tk].to(torch.int32).to(device)
            return [rn(tq, h, c), rn(tq, h, k), rn(num_pages, 1, c), rn(num_pages, 1, k), ptr(q_lens), ptr(kv_lens), idx,
                    0.1352337747812271]
        hq, hkv, d = dims["num_qo_heads"], dims["num_kv_heads"], dims["head_dim"]
        if family == "gqa_ragged_prefill":
            return [rn(tq, hq, d), rn(tk, hkv, d), rn(tk, hkv, d), ptr(q_lens), ptr(kv_lens), float(d) ** -0.5]
        num_pages = tk + 3
        idx = torch.randperm(num_pages, generator=g)[:tk].to(torch.int32).to(device)
        return [rn(tq, hq, d), rn(num_pages, 1, hkv, d), rn(num_pages, 1, hkv, d), ptr(q_lens), ptr(kv_lens), idx,
                float(d) ** -0.5]
    batch = len(kv_lens)
    ps = int(dims.get("page_size", 1))
    pages = [-(-n // ps) for n in kv_lens]
    num_pages = sum(pages) + 3
    idx = torch.randperm(num_pages, generator=g)[:sum(pages)].to(torch.int32)
    indptr = torch.tensor([0] + list(torch.tensor(pages).cumsum(0).tolist()), dtype=torch.int32)
    rn = lambda *s: torch.randn(*s, generator=g).to(dt).to(device)  # noqa: E731
    if family == "gqa_paged_decode":
        hq, hkv, d = dims["num_qo_heads"], dims["num_kv_heads"], dims["head_dim"]
        args = [rn(batch, hq, d), rn(num_pages, ps, hkv, d), rn(num_pages, ps, hkv, d), indptr.to(device), idx.to(device)]
        last = torch.tensor([n - (p - 1) * ps if p else 0 for n, p in zip(kv_lens, pages)], dtype=torch.int32)
        args.append(last.to(device) if ps != 1 else None)
        args.append(float(d) ** -0.5)
        return args
    h, c, k = dims["num_qo_heads"], dims["head_dim_ckv"], dims["head_dim_kpe"]
    return [rn(batch, h, c), rn(batch, h, k), rn(num_pages, 1, c), rn(num_pages, 1, k), indptr.to(device),
            idx.to(device), float(c + k) ** -0.5]


def reference(family, args):
    from ..runtime import reference as R

    fn = {"gqa_paged_decode": R.gqa_paged_decode, "mla_paged_decode": R.mla_paged_decode,
          "gqa_ragged_prefill": R.gqa_ragged_prefill, "gqa_paged_prefill": R.gqa_paged_prefill,
          "mla_paged_prefill": R.mla_paged_prefill}[family]
    return fn(*args)


@dataclass
class WorkloadCandidate:
    label: str
    source: str
    origin: str = "library"
    split: int | None = None
    eligible: bool = True
    kernel: object = None
    checked: int = 0
    correct: bool = False
    failure: str | None = None
    latency_us: dict = field(default_factory=dict)

    @property
    def geomean_us(self):
        vals = [v for v in self.latency_us.values() if v]
        return math.exp(sum(math.log(v) for v in vals) / len(vals)) if vals else None


SMALL_GRID_CTAS = 32        # the "single" candidate of the dispatch question: a grid that rarely cuts a short item
DISPATCH_MARGIN = 0.05      # the hybrid must beat the full grid's geomean by this much to be applied


def calibrate_dispatch(pair, solo, tiles: dict, *, kv_tile: int = 64, page_size: int = 1, indptr_index: int = 3) -> dict:
    """The smallest ``min_tiles`` threshold with the best hybrid geomean: a workload whose longest request
    has at least ``min_tiles`` KV tiles runs ``pair`` (here: the full grid, items cut across CTAs and
    combined), a shorter one runs ``solo`` (here: a small grid). Same rule, tie-break and result fields as
    the reference (python/cleave/pipeline/dynamic.py:209-242); ``pair`` / ``solo`` are candidates whose
    ``latency_us`` maps workload key -> microseconds, ``tiles`` maps workload key -> KV tiles of its longest
    request. ``applied`` says whether the hybrid beats ``pair`` alone by ``DISPATCH_MARGIN``."""
    keys = [k for k in tiles if pair.latency_us.get(k) and solo.latency_us.get(k)]
    if not keys:
        raise CleaveError("calibrate_dispatch: no workload was timed on both candidates")

    def geomean(vals):
        return math.exp(sum(math.log(v) for v in vals) / len(vals))

    def hybrid(t):
        return geomean([(pair if tiles[k] >= t else solo).latency_us[k] for k in keys])

    thresholds = sorted({tiles[k] for k in keys} | {1, max(tiles[k] for k in keys) + 1})
    best_us, min_tiles = min((hybrid(t), t) for t in thresholds)   # ties go to the smallest threshold
    split_us = geomean([pair.latency_us[k] for k in keys])
    return {
        "split_label": pair.label, "single_label": solo.label, "min_tiles": int(min_tiles),
        "kv_tile": int(kv_tile), "page_size": int(page_size), "indptr_index": int(indptr_index),
        "geomean_us": {"hybrid": best_us, "split": split_us, "single": geomean([solo.latency_us[k] for k in keys])},
        "n_workloads": len(keys), "split_runs": sum(tiles[k] >= min_tiles for k in keys),
        "applied": bool(best_us < split_us * (1.0 - DISPATCH_MARGIN)),
        "rule": "run the full grid when the longest request has at least min_tiles KV tiles "
                "(indptr units x page_size tokens / kv_tile), else the small grid",
    }


class DynamicReport:
    def __init__(self, candidates, errors, *, workloads, timings, dispatch=None):
        self.candidates, self.errors = list(candidates), list(errors)
        self.n_workloads, self.timings, self.dispatch = workloads, dict(timings), dispatch
        self.dispatch_note = ("one persistent kernel splits the KV tile stream evenly over the SMs for every "
                              "length distribution; the measured split / single threshold is recorded and "
                              "applied only when it pays")

    correct = property(lambda self: [c for c in self.candidates if c.correct])
    timed = property(lambda self: [c for c in self.correct if c.latency_us])
    failures = property(lambda self: [c for c in self.candidates if not c.correct])

    def best(self, split=None):
        pool = [c for c in self.timed if c.eligible and (split is None or bool(c.split) == split)]
        return min(pool, key=lambda c: c.geomean_us) if pool else None

    def summary(self) -> str:
        rows = [f"validate      {len(self.correct)} of {len(self.candidates)} correct over {self.n_workloads} workloads"
                f"  {self.timings.get('validate', 0):.2f} s"]
        rows += [f"  FAILS: {c.label}: {c.failure}" for c in self.failures]
        b = self.best()
        if b is not None:
            rows.append(f"benchmark     best {b.geomean_us:.2f} us geomean  {b.label}  {self.timings.get('benchmark', 0):.2f} s")
        if self.dispatch:
            d = self.dispatch
            rows.append(f"dispatch      min_tiles {d['min_tiles']}  hybrid {d['geomean_us']['hybrid']:.2f} us, full grid "
                        f"{d['geomean_us']['split']:.2f} us, small grid {d['geomean_us']['single']:.2f} us  "
                        f"({'applied' if d['applied'] else 'not applied: within the margin of the full grid'})")
        else:
            rows.append(f"dispatch      none: {self.dispatch_note}")
        return "\n".join(rows)

    def to_dict(self) -> dict:
        return {"candidates": len(self.candidates), "correct": len(self.correct),
                "failures": {c.label: c.failure for c in self.failures}, "timings_s": self.timings,
                "latency_us": {c.label: c.geomean_us for c in self.timed},
                "per_workload_us": {c.label: c.latency_us for c in self.timed}, "dispatch": self.dispatch}

    def __str__(self):
        return self.summary()


class PagedKernel(Kernel):
    """``k(*inputs)`` in the operator's declared order (or by name) -> ``(out, lse)``; outputs are
    allocated per call, the split-KV workspace once per device and stream."""

    def __init__(self, op_name, spec, source, compiled=None, **kw):
        self.op_name, self.spec = op_name, spec
        self.param_names = list(OPERATORS[op_name][1])
        self.dispatch, self.dispatch_sources = None, {}
        super().__init__([Stage("main", source, [], [], kw.get("label", ""), kw.get("latency_us"))],
                         name=op_name, input_names=self.param_names, input_shapes=[], **kw)
        if compiled is not None:
            from ..runtime.scratch import with_scratch

            compiled = with_scratch(compiled)
        self._compiled = compiled

    def compile(self) -> "PagedKernel":
        if self._compiled is None:
            from ..runtime.compile import _compile, _load_main_kernel_from_code
            from ..runtime.scratch import with_scratch

            self._compiled = with_scratch(_compile(_load_main_kernel_from_code(self.source), None))
        return self

    def save(self, path):
        p = super().save(path)
        meta = json.loads((p / "kernel.json").read_text())
        meta["paged"] = self.op_name
        (p / "kernel.json").write_text(json.dumps(meta, indent=1, default=str))
        if self.dispatch:   # the reference keeps the calibrated threshold beside the kernel (dispatch.json)
            (p / "dispatch.json").write_text(json.dumps(self.dispatch, indent=1, default=str))
        return p

    @classmethod
    def _load(cls, p, m) -> "PagedKernel":
        from ..runtime.compile import _load_main_kernel_from_code

        source = (p / m["stages"][0]["file"]).read_text()
        spec = _load_main_kernel_from_code(source)
        kernel = cls(m["paged"], spec, source, label=m["label"], variant=m["variant"], latency_us=m["latency_us"],
                     meta=dict(m.get("meta") or {}, loaded_from=str(p)))
        if (p / "dispatch.json").exists():
            kernel.dispatch = json.loads((p / "dispatch.json").read_text())
        return kernel

    def __call__(self, *args, **named):
        import torch

        from ..runtime.reference import torch_dtype

        names = self.param_names
        kept = [p.name.replace("PlaceHolder_", "") for p in self.spec.inputs]
        if args and named:
            raise TypeError("pass inputs either positionally or by name, not both")
        if named:
            unknown = sorted(set(named) - set(names))
            if unknown:
                raise TypeError(f"{self.name}: unexpected inputs {unknown}")
            bound = {n: named.get(n) for n in names}
        elif len(args) in (len(names), len(kept)):
            bound = dict(zip(names if len(args) == len(names) else kept, args))
        else:
            raise TypeError(f"{self.name}: expected inputs ({', '.join(names)})")
        for n in names:
            if n not in kept and bound.get(n) is not None:
                raise ValueError(f"{self.name}: page_size=1 reads no {n}; pass None")
            if n in kept and bound.get(n) is None:
                raise TypeError(f"{self.name}: missing input {n!r}")
        self.compile()
        sizes = {}
        for p in self.spec.inputs:
            if p.role == "input":
                for d, n in zip(p.dims, bound[p.name.replace("PlaceHolder_", "")].shape):
                    if isinstance(d, str):
                        sizes.setdefault(d, int(n))
        device = bound[kept[0]].device
        outs = [torch.empty([sizes[d] if isinstance(d, str) else int(d) for d in p.dims], dtype=torch_dtype(p.dtype),
                            device=device) for p in self.spec.outputs]
        self._compiled(*[bound[n] for n in kept], *outs)
        return outs[0] if len(outs) == 1 else tuple(outs)


def compile_dynamic(op_name, *, dtype=None, preset="default", eval=None, workloads=None, tolerance=None,  # noqa: A002
                    max_workloads: int = 6, progress=None, **dims) -> PagedKernel:
    """Validate the operator's kernel on every workload (outputs NaN-poisoned first, so an unwritten
    element fails), time it on ``max_workloads`` stratified samples, return the ``PagedKernel``."""
    import torch

    if op_name not in OPERATORS:
        raise CleaveError(f"unknown paged operator {op_name!r}; have {sorted(OPERATORS)}")
    family, _, need = OPERATORS[op_name]
    missing = [d for d in need if d not in dims]
    if missing:
        raise TypeError(f"{op_name}: missing dims {missing}")
    dt = getattr(dtype, "name", dtype) or "bfloat16"
    dims = {k: int(v) for k, v in dims.items()}
    if family in ("gqa_paged_decode", "gqa_ragged_prefill", "gqa_paged_prefill"):
        if dims["head_dim"] not in (64, 128):
            raise PagingRefusal(f"{op_name}: head_dim {dims['head_dim']} is not built (64 or 128)")
        if dims["num_qo_heads"] % dims["num_kv_heads"]:
            raise PagingRefusal(f"{op_name}: query heads must be a multiple of kv heads")
    elif (dims["head_dim_ckv"], dims["head_dim_kpe"]) != (512, 64):
        raise PagingRefusal(f"{op_name}: only the 512 + 64 latent layout is built")
    cfg = resolve_eval(preset, eval)
    tol = tolerance or PAGED_TOLERANCE
    spec = make_spec(family, dt, dims)
    source = B200CodeGen().gen(spec)
    from ..runtime.compile import _compile, _load_main_kernel_from_code
    from ..runtime.timer import min_launch_us

    cand = WorkloadCandidate(label=f"{op_name} " + ("tcgen05 query-tile" if family in PREFILL_FAMILIES else "persistent tile-stream"),
                             source=source)
    cand.kernel = _compile(_load_main_kernel_from_code(source), None)
    wls = list(workloads) if workloads is not None else (
        paged_prefill_workloads() if family in PREFILL_FAMILIES else paged_decode_workloads())
    errors, t0 = [], time.perf_counter()
    cand.correct = True
    for key, lens in wls:
        args = make_inputs(family, dims, lens, dt)
        want = reference(family, args)
        kept = [a for a in args if a is not None]
        outs = [torch.full_like(w, float("nan")) for w in want]
        try:
            cand.kernel(*kept, *outs)
            torch.testing.assert_close([o.float() for o in outs], [w.float() for w in want], rtol=tol.rtol,
                                       atol=tol.atol, equal_nan=False)
            cand.checked += 1
        except Exception as exc:  # noqa: BLE001 - reported, not raised: the report carries every failure
            cand.correct, cand.failure = False, f"{key}: {type(exc).__name__}: {str(exc).strip().splitlines()[0][:160]}"
            errors.append((cand, exc))
            break
    t1 = time.perf_counter()
    if cand.correct:
        step = max(1, len(wls) // max(1, max_workloads))
        for key, lens in wls[::step][:max_workloads]:
            args = make_inputs(family, dims, lens, dt)
            kept = [a for a in args if a is not None]
            outs = [torch.empty_like(w) for w in reference(family, args)]
            cand.latency_us[key] = min_launch_us(cand.kernel, [*kept, *outs], batch=20, repeats=5)
    dispatch, cands = None, [cand]
    if cand.correct and family in ("gqa_paged_decode", "mla_paged_decode"):
        # the reference's dispatch question on this kernel: full grid against a small grid, per workload
        small_spec = make_spec(family, dt, dims, attrs={"max_ctas": SMALL_GRID_CTAS})
        small = WorkloadCandidate(label=f"{op_name} persistent tile-stream, {SMALL_GRID_CTAS} CTAs",
                                  source=B200CodeGen().gen(small_spec), eligible=False, correct=True)
        small.kernel = _compile(_load_main_kernel_from_code(small.source), None)
        tiles = {}
        ps = int(dims.get("page_size", 1))
        for key, lens in wls[::step][:max_workloads]:
            args = make_inputs(family, dims, lens, dt)
            kept = [a for a in args if a is not None]
            outs = [torch.empty_like(w) for w in reference(family, args)]
            small.latency_us[key] = min_launch_us(small.kernel, [*kept, *outs], batch=20, repeats=5)
            tiles[key] = -(-max(-(-n // ps) for n in lens) * ps // 64)
        dispatch = calibrate_dispatch(cand, small, tiles, kv_tile=64, page_size=ps,
                                      indptr_index=OPERATORS[op_name][1].index("kv_indptr"))
        cands.append(small)
    t2 = time.perf_counter()
    report = DynamicReport(cands, errors, workloads=cand.checked, timings={"validate": t1 - t0, "benchmark": t2 - t1},
                           dispatch=dispatch)
    if progress:
        progress("evaluate", report)
    best = report.best()
    if best is None:
        err = CleaveError(f"{op_name}: the kernel is not correct over its workloads: {cand.failure}")
        err.report = report
        raise err
    kernel = PagedKernel(op_name, spec, source, best.kernel, label=best.label, variant="solo",
                         latency_us=best.geomean_us, report=report)
    kernel.dispatch = dispatch
    return kernel
