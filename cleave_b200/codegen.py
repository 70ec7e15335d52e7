"""Plan -> kernel text. The seam the reference fills with TileLang source
(``TilelangCodeGen.gen``, python/cleave/codegen/__init__.py:24-48) is filled here with a small Python
module that defines ``main_kernel`` as a :class:`KernelSpec`: which hand-written kernel family to
call and with what parameters. The text is persisted, hashed and compared exactly like the
reference's generated source, so equal plans must - and do - give byte-equal text.
"""

from __future__ import annotations

import json
from dataclasses import dataclass, field

from .core.errors import CodegenError

FAMILIES = ("matmul", "rmsnorm_matmul", "swiglu", "attention_decode", "mla_decode",
            "gqa_paged_decode", "mla_paged_decode", "gqa_ragged_prefill", "gqa_paged_prefill",
            "matmul_matmul", "qknorm_attention", "matmul_rowsum", "lora")
FORMAT = 1


@dataclass(frozen=True)
class KernelParam:
    name: str      # buffer name: PlaceHolder_<NAME> for inputs, OutputNode[_i] for outputs
    dtype: str
    dims: tuple    # ints, or dim names for dynamic extents
    role: str      # "input" | "output" | "scalar"


@dataclass(frozen=True)
class KernelSpec:
    """One kernel of the library, fully parameterised."""

    family: str
    dtype: str                       # storage dtype: "float16" | "bfloat16"
    dims: dict = field(default_factory=dict)    # static extents (M, N, K, HQ, ...)
    split: int = 1                   # K / KV split factor the plan asked for (1 = solo)
    role: str = "main"               # "main" (fused split, one launch) - the only role emitted
    attrs: dict = field(default_factory=dict)   # eps, scale, gamma, max_ctas ...
    params: tuple = ()               # KernelParam, inputs in call order then outputs

    def to_dict(self) -> dict:
        return {"format": FORMAT, "family": self.family, "dtype": self.dtype, "dims": dict(self.dims),
                "split": self.split, "role": self.role, "attrs": dict(self.attrs),
                "params": [[p.name, p.dtype, list(p.dims), p.role] for p in self.params]}

    @classmethod
    def from_dict(cls, d: dict) -> "KernelSpec":
        if d.get("format") != FORMAT:
            raise CodegenError(f"unsupported kernel-spec format {d.get('format')!r}")
        if d["family"] not in FAMILIES:
            raise CodegenError(f"unknown kernel family {d['family']!r}")
        params = tuple(KernelParam(n, t, tuple(s), r) for n, t, s, r in d.get("params", ()))
        return cls(d["family"], d["dtype"], dict(d.get("dims", {})), int(d.get("split", 1)),
                   d.get("role", "main"), dict(d.get("attrs", {})), params)

    @property
    def inputs(self):
        return [p for p in self.params if p.role != "output"]

    @property
    def outputs(self):
        return [p for p in self.params if p.role == "output"]


def _ph(name):
    return f"PlaceHolder_{name}"


def default_params(family: str, dtype: str, dims: dict, attrs: dict) -> tuple:
    """The call signature of a family, with the reference's buffer-naming convention
    (python/cleave/codegen/split.py:7-10: inputs ``PlaceHolder_<NAME>``, outputs ``OutputNode[_i]``)."""
    P = KernelParam
    g = lambda k: dims[k]  # noqa: E731
    if family in ("matmul", "rmsnorm_matmul"):
        ps = [P(_ph("x"), dtype, (g("M"), g("K")), "input"), P(_ph("w"), dtype, (g("K"), g("N")), "input")]
        if family == "rmsnorm_matmul" and attrs.get("gamma"):
            ps.insert(1, P(_ph("gamma"), dtype, (g("K"),), "input"))
        return tuple(ps + [P("OutputNode", dtype, (g("M"), g("N")), "output")])
    if family == "swiglu":
        return (P(_ph("x"), dtype, (g("M"), g("K")), "input"), P(_ph("w0"), dtype, (g("K"), g("N")), "input"),
                P(_ph("w1"), dtype, (g("K"), g("N")), "input"), P("OutputNode", dtype, (g("M"), g("N")), "output"))
    if family == "matmul_rowsum":
        return (P(_ph("x"), dtype, (g("M"), g("K")), "input"), P(_ph("w"), dtype, (g("K"), g("N")), "input"),
                P("OutputNode", dtype, (g("M"), 1), "output"))
    if family == "lora":
        return (P(_ph("x"), dtype, (g("M"), g("K")), "input"), P(_ph("w"), dtype, (g("K"), g("N")), "input"),
                P(_ph("a"), dtype, (g("K"), g("R")), "input"), P(_ph("b"), dtype, (g("R"), g("N")), "input"),
                P("OutputNode", dtype, (g("M"), g("N")), "output"))
    if family in ("attention_decode", "matmul_matmul", "qknorm_attention"):
        return (P(_ph("q"), dtype, (g("HQ"), g("SQ"), g("D")), "input"),
                P(_ph("k"), dtype, (g("HKV"), g("SKV"), g("D")), "input"),
                P(_ph("v"), dtype, (g("HKV"), g("SKV"), g("D")), "input"),
                P("OutputNode", dtype, (g("HQ"), g("SQ"), g("D")), "output"))
    if family == "mla_decode":
        return (P(_ph("q"), dtype, (g("B"), g("H"), g("D")), "input"), P(_ph("kv"), dtype, (g("B"), g("SKV"), g("D")), "input"),
                P(_ph("q_pe"), dtype, (g("B"), g("H"), g("PE")), "input"),
                P(_ph("k_pe"), dtype, (g("B"), g("SKV"), g("PE")), "input"),
                P("OutputNode", dtype, (g("B"), g("H"), g("D")), "output"))
    if family == "gqa_paged_decode":
        hq, hkv, d, ps_ = g("num_qo_heads"), g("num_kv_heads"), g("head_dim"), g("page_size")
        out = [P(_ph("q"), dtype, ("batch", hq, d), "input"),
               P(_ph("k_cache"), dtype, ("num_pages", ps_, hkv, d), "input"),
               P(_ph("v_cache"), dtype, ("num_pages", ps_, hkv, d), "input"),
               P(_ph("kv_indptr"), "int32", ("len_indptr",), "input"),
               P(_ph("kv_indices"), "int32", ("num_kv_indices",), "input")]
        if ps_ != 1:
            out.append(P(_ph("kv_last_page_len"), "int32", ("batch",), "input"))
        out += [P("sm_scale", "float32", (), "scalar"), P("OutputNode", dtype, ("batch", hq, d), "output"),
                P("OutputNode_1", "float32", ("batch", hq), "output")]
        return tuple(out)
    if family == "mla_paged_decode":
        h, c, k = g("num_qo_heads"), g("head_dim_ckv"), g("head_dim_kpe")
        return (P(_ph("q_nope"), dtype, ("batch", h, c), "input"), P(_ph("q_pe"), dtype, ("batch", h, k), "input"),
                P(_ph("ckv_cache"), dtype, ("num_pages", 1, c), "input"),
                P(_ph("kpe_cache"), dtype, ("num_pages", 1, k), "input"),
                P(_ph("kv_indptr"), "int32", ("len_indptr",), "input"),
                P(_ph("kv_indices"), "int32", ("num_kv_indices",), "input"),
                P("sm_scale", "float32", (), "scalar"), P("OutputNode", dtype, ("batch", h, c), "output"),
                P("OutputNode_1", "float32", ("batch", h), "output"))
    if family in ("gqa_ragged_prefill", "gqa_paged_prefill"):
        hq, hkv, d = g("num_qo_heads"), g("num_kv_heads"), g("head_dim")
        out = [P(_ph("q"), dtype, ("total_q", hq, d), "input")]
        if family == "gqa_paged_prefill":
            out += [P(_ph("k_cache"), dtype, ("num_pages", 1, hkv, d), "input"),
                    P(_ph("v_cache"), dtype, ("num_pages", 1, hkv, d), "input")]
        else:
            out += [P(_ph("k"), dtype, ("total_kv", hkv, d), "input"), P(_ph("v"), dtype, ("total_kv", hkv, d), "input")]
        out += [P(_ph("qo_indptr"), "int32", ("len_indptr",), "input"), P(_ph("kv_indptr"), "int32", ("len_indptr",), "input")]
        if family == "gqa_paged_prefill":
            out.append(P(_ph("kv_indices"), "int32", ("num_kv_indices",), "input"))
        out += [P("sm_scale", "float32", (), "scalar"), P("OutputNode", dtype, ("total_q", hq, d), "output"),
                P("OutputNode_1", "float32", ("total_q", hq), "output")]
        return tuple(out)
    raise CodegenError(f"unknown kernel family {family!r}")


def make_spec(family: str, dtype: str, dims: dict, *, split: int = 1, attrs: dict | None = None) -> KernelSpec:
    attrs = dict(attrs or {})
    return KernelSpec(family, dtype, dict(dims), int(split), "main", attrs, default_params(family, dtype, dims, attrs))


_HEADER = ("# cleave_b200 kernel spec: selects and parameterises a hand-written sm_100a kernel.\n"
           "# Loaded by cleave_b200.runtime.compile._load_main_kernel_from_code; no code is generated.\n"
           "import json\n\nfrom cleave_b200.codegen import KernelSpec\n\n")


class B200CodeGen:
    """Same call shape as the reference's ``TilelangCodeGen(apply_rasterization, debug).gen(graph)``."""

    def __init__(self, apply_rasterization: int = 16, debug: bool = False):
        self.apply_rasterization, self.debug = apply_rasterization, debug

    def gen(self, plan_or_spec) -> str:
        """Module text defining ``main_kernel``. Accepts a :class:`KernelSpec`, a scheduled plan
        of the reference (anything with ``tile.flat_graph``), a tiled graph, or a
        ``[partial, combine]`` pair of those - a split pair collapses into ONE fused kernel."""
        spec = plan_or_spec if isinstance(plan_or_spec, KernelSpec) else recognise(plan_or_spec)
        body = json.dumps(spec.to_dict(), sort_keys=True, indent=1)
        return f'{_HEADER}main_kernel = KernelSpec.from_dict(json.loads(r"""\n{body}\n"""))\n'


# ----------------------------------------------------------------------------- plan recogniser
def _nodes_of(obj):
    graph = getattr(getattr(obj, "tile", None), "flat_graph", None) or getattr(obj, "flat_graph", None) or obj
    nodes = getattr(graph, "nodes", None)
    if nodes is None:
        raise CodegenError(f"cannot find a node list on {type(obj).__name__}")
    return list(nodes)


def _kind(node) -> str:
    op = getattr(node, "op", None)
    return type(op).__name__ if op is not None else type(node).__name__


def _shape(node) -> tuple:
    try:
        return tuple(int(s) for s in node.get_shape(0))
    except Exception:  # noqa: BLE001 - fakes and placeholders expose .shape
        return tuple(int(s) for s in getattr(node, "shape", ()))


def _dtype_of(node, default="float16") -> str:
    try:
        return str(node.get_dtype(0))
    except Exception:  # noqa: BLE001
        return str(getattr(node, "dtype", default))


def recognise(obj) -> KernelSpec:
    """Classify a scheduled plan by the op pattern of its flat graph and read the shapes off its
    placeholders. Patterns (op class names of python/cleave/ir/ops): ``{Matmul}`` -> matmul;
    ``{Matmul, Mul, ReduceSum, Div, RSqrt|Sqrt}`` -> rmsnorm_matmul; ``{Matmul x2, Silu, Mul}`` ->
    swiglu; ``{Matmul x2, Exp, ReduceSum, Div}`` -> attention_decode (with ``RSqrt`` -> qknorm_attention,
    without ``Exp`` -> matmul_matmul), with a third score matmul and an ``Add`` -> mla_decode;
    ``{Matmul, ReduceSum}`` -> matmul_rowsum; ``{Matmul x3, Add}`` over four placeholders -> lora. Leading ``SplitView`` nodes carry the split factor. Tile shapes and
    thread counts in the plan are hints scored for another architecture and are not used."""
    if isinstance(obj, (list, tuple)):  # [partial, combine]: the partial carries the structure
        if not obj:
            raise CodegenError("empty plan list")
        return recognise(obj[0])
    nodes = _nodes_of(obj)
    kinds = [_kind(n) for n in nodes]
    phs = [n for n, k in zip(nodes, kinds) if k.startswith("PlaceHolder")]
    count = lambda k: sum(1 for x in kinds if x == k)  # noqa: E731
    split = 1
    for n, k in zip(nodes, kinds):
        if k == "SplitView":
            split = max(split, _shape(n)[0])
    declared = getattr(obj, "split_factor", None)
    if declared:
        split = int(declared)
    dtype = _dtype_of(phs[0]) if phs else "float16"
    n_mm = count("Matmul")
    shapes = [_shape(n) for n in phs]
    if n_mm == 1 and "Exp" not in kinds:
        (m, k), (k2, n) = shapes[0][-2:], shapes[1][-2:]
        if k != k2:
            raise CodegenError(f"matmul placeholders do not chain: {shapes}")
        fam = "rmsnorm_matmul" if "ReduceSum" in kinds and ("RSqrt" in kinds or "Sqrt" in kinds) else "matmul"
        if fam == "matmul" and "ReduceSum" in kinds:
            return make_spec("matmul_rowsum", dtype, {"M": m, "N": n, "K": k}, split=split)
        attrs = {}
        if fam == "rmsnorm_matmul":
            eps = [getattr(getattr(n, "op", None), "value", None) for n, kd in zip(nodes, kinds) if kd == "Add"]
            attrs["eps"] = float(next((e for e in eps if e is not None), 0.0))
        return make_spec(fam, dtype, {"M": m, "N": n, "K": k}, split=split, attrs=attrs)
    if n_mm == 2 and "Silu" in kinds:
        (m, k), (_, n) = shapes[0][-2:], shapes[1][-2:]
        return make_spec("swiglu", dtype, {"M": m, "N": n, "K": k}, split=split)
    if n_mm == 2 and len(shapes) == 3 and all(len(sh) >= 3 for sh in shapes):
        (hq, sq, d), (hkv, skv, _) = shapes[0][-3:], shapes[1][-3:]
        dims = {"HQ": hq, "HKV": hkv, "SQ": sq, "SKV": skv, "D": d}
        if "Exp" not in kinds:
            return make_spec("matmul_matmul", dtype, dims, split=split)
        if "RSqrt" in kinds or "Sqrt" in kinds:
            eps = [getattr(getattr(n, "op", None), "value", None) for n, kd in zip(nodes, kinds) if kd == "Add"]
            return make_spec("qknorm_attention", dtype, dims, split=split,
                             attrs={"eps": float(next((e for e in eps if e is not None), 0.0))})
        return make_spec("attention_decode", dtype, dims, split=split)
    if n_mm == 3 and "Exp" not in kinds and len(shapes) == 4:
        (m, k), (_, n) = shapes[0][-2:], shapes[1][-2:]
        r = min(s_[-1] for s_ in shapes)
        return make_spec("lora", dtype, {"M": m, "N": n, "K": k, "R": r}, split=split)
    if "Exp" in kinds and n_mm == 3 and len(shapes) == 4:
        by_rank = sorted(shapes, key=lambda s: (s[-1], s[-2]))
        (b, h, pe), (_, skv, _), (_, _, d) = by_rank[0], by_rank[1], by_rank[2]
        h = min(s[-2] for s in shapes)
        skv = max(s[-2] for s in shapes)
        return make_spec("mla_decode", dtype, {"B": b, "H": h, "SKV": skv, "D": d, "PE": pe}, split=split)
    raise CodegenError(f"no kernel family matches the plan's op pattern {sorted(set(kinds))}")
