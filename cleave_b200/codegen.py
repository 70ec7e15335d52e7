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
            "matmul_matmul", "qknorm_attention", "matmul_rowsum", "lora", "split_combine", "mla_paged_prefill")
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
    role: str = "main"               # "main" (fused: one launch whatever the split), "partial" or "combine"
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

    def input_roles(self) -> list:
        """The library's name for each input, in call order (``x``, ``w``, ``q`` ...). A spec made from a
        reference plan keeps the plan's placeholder names on its parameters and lists which of them plays
        which part in ``attrs["bind"]``; otherwise the part is the parameter name without ``PlaceHolder_``."""
        bind = {v: k for k, v in (self.attrs.get("bind") or {}).items()}
        return [bind.get(p.name, p.name.replace("PlaceHolder_", "", 1)) for p in self.inputs]

    def by_role(self, args) -> dict:
        return dict(zip(self.input_roles(), args))

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
    if family == "mla_paged_prefill":
        h, c, k = g("num_qo_heads"), g("head_dim_ckv"), g("head_dim_kpe")
        return (P(_ph("q_nope"), dtype, ("total_q", h, c), "input"), P(_ph("q_pe"), dtype, ("total_q", h, k), "input"),
                P(_ph("ckv_cache"), dtype, ("num_pages", 1, c), "input"),
                P(_ph("kpe_cache"), dtype, ("num_pages", 1, k), "input"),
                P(_ph("qo_indptr"), "int32", ("len_indptr",), "input"), P(_ph("kv_indptr"), "int32", ("len_indptr",), "input"),
                P(_ph("kv_indices"), "int32", ("num_kv_indices",), "input"),
                P("sm_scale", "float32", (), "scalar"), P("OutputNode", dtype, ("total_q", h, c), "output"),
                P("OutputNode_1", "float32", ("total_q", h), "output"))
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


def make_two_stage_specs(family: str, dtype: str, dims: dict, split: int, attrs: dict | None = None):
    """``(partial, combine)`` specs of the two-stage form of a split (the reference's partial + combine kernel
    pairs, python/cleave/codegen/split.py:13-123): the partial kernel writes one result per split, the combine
    kernel sums them. Built for the split-K matmul and for split-KV decode attention with one query row."""
    P = KernelParam
    attrs = dict(attrs or {})
    split = int(split)
    ins = tuple(p for p in default_params(family, dtype, dims, attrs) if p.role != "output")
    if family == "matmul":
        m, n = dims["M"], dims["N"]
        part_out = (P("OutputNode", dtype, (split, m, n), "output"),)
        comb_in = (P("PlaceHolder_partial", dtype, (split, m, n), "input"),)
        comb_attrs = {"axes": [0], "divide": False}
        final = (P("OutputNode", dtype, (m, n), "output"),)
    elif family == "attention_decode" and dims["SQ"] == 1:
        hq, d = dims["HQ"], dims["D"]
        scale = float(attrs.get("scale", d ** -0.5))
        attrs.setdefault("scale", scale)
        attrs.setdefault("shift", -50.0 * scale)
        part_out = (P("OutputNode", dtype, (hq, split, 1, d), "output"), P("OutputNode_1", dtype, (hq, split, 1), "output"))
        comb_in = (P("PlaceHolder_o_partial", dtype, (hq, split, 1, d), "input"),
                   P("PlaceHolder_l_partial", dtype, (hq, split, 1), "input"))
        comb_attrs = {"axes": [1, 1], "divide": True, "num": 0, "den": 1}
        final = (P("OutputNode", dtype, (hq, 1, d), "output"),)
    else:
        raise CodegenError(f"no two-stage form of {family} {dims}")
    partial = KernelSpec(family, dtype, dict(dims), split, "partial", attrs, ins + part_out)
    combine = KernelSpec("split_combine", dtype, {}, split, "combine", comb_attrs, comb_in + final)
    return partial, combine


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
# A scheduled plan of the reference (python/cleave/pipeline/plans.py:16-41) carries a tiled flat graph:
# ``plan.tile.flat_graph.nodes`` in topological order, each node an instance of one of the classes of
# python/cleave/ir/ops (``PlaceHolderNode``, ``Matmul``, ``SplitView``, ``Div`` ...), with ``name``,
# ``get_shape(0)``, ``get_dtype(0)`` and ``inputs`` (edges with ``src_node``). Element-wise nodes with a scalar
# operand hold it in ``const`` (python/cleave/ir/ops/elementwise.py:90-101; ``const_on_left`` for ``c / x``).
# The recogniser reads the dataflow, not the node order: which placeholder feeds which matmul operand decides
# its role, the constants on the way to ``Exp`` give the score scale, those between the sum of squares and
# ``RSqrt`` give eps. Tile shapes and thread counts in the plan were scored for another architecture; the
# kernels pick their own (``cleave_b200.arch.snap_tile`` maps the hints onto what exists).

_VIEWS = ("SplitView", "Reshape", "View", "Transpose", "Broadcast", "Cast")


def _graph_of(obj):
    graph = getattr(getattr(obj, "tile", None), "flat_graph", None) or getattr(obj, "flat_graph", None) or obj
    nodes = getattr(graph, "nodes", None)
    if nodes is None:
        raise CodegenError(f"cannot find a node list on {type(obj).__name__}")
    return list(nodes)


def _kind(node) -> str:
    return type(node).__name__


def _shape(node) -> tuple:
    try:
        return tuple(int(s) for s in node.get_shape(0))
    except Exception:  # noqa: BLE001
        return tuple(int(s) for s in getattr(node, "shape", ()))


def _dtype_of(node, default="float16") -> str:
    try:
        return str(node.get_dtype(0))
    except Exception:  # noqa: BLE001
        return str(getattr(node, "dtype", default))


class _Flow:
    """Dataflow view of a flat graph."""

    def __init__(self, obj):
        self.nodes = _graph_of(obj)
        self.pos = {id(n): i for i, n in enumerate(self.nodes)}
        self._anc = {}

    def preds(self, n):
        return [e.src_node for e in (getattr(n, "inputs", None) or []) if getattr(e, "src_node", None) is not None]

    def of(self, *kinds):
        return [n for n in self.nodes if _kind(n) in kinds]

    def ancestors(self, n):
        key = id(n)
        if key not in self._anc:
            seen, stack = {}, list(self.preds(n))
            while stack:
                m = stack.pop()
                if id(m) not in seen:
                    seen[id(m)] = m
                    stack.extend(self.preds(m))
            self._anc[key] = seen
        return self._anc[key]

    def below(self, n, m) -> bool:
        """True when ``m`` is an ancestor of ``n``."""
        return id(m) in self.ancestors(n)

    def root(self, n):
        """The placeholder ``n`` is a plain view of, or None when it is computed."""
        while n is not None and not _kind(n).startswith("PlaceHolder"):
            ps = self.preds(n)
            if _kind(n) not in _VIEWS or len(ps) != 1:
                return None
            n = ps[0]
        return n

    def scalar_ops(self, target, stop=None):
        """The element-wise nodes with a scalar operand among the ancestors of ``target`` (and ``target``
        itself), in graph order; with ``stop`` only those computed from ``stop``."""
        cand = list(self.ancestors(target).values()) + [target]
        out = [n for n in cand if getattr(n, "const", None) is not None and (stop is None or self.below(n, stop))]
        return sorted(out, key=lambda n: self.pos[id(n)])


def _score_affine(flow, exp_node):
    """``(scale, shift)`` of the scalar operations between the score product and ``Exp``, composed into
    ``exp(scale * s + shift)``. The fused kernels use the scale only (softmax does not depend on a constant
    shift); the two-stage partial kernels reproduce the shift, which is part of what they emit."""
    a, b = 1.0, 0.0
    for n in flow.scalar_ops(exp_node):
        k, c = _kind(n), float(n.const)
        if k == "Div":
            if getattr(n, "const_on_left", False):
                raise CodegenError("a constant divided by the scores is not an attention score scale")
            a, b = a / c, b / c
        elif k == "Mul":
            a, b = a * c, b * c
        elif k == "Add":
            b += c
        elif k == "Sub" and not getattr(n, "const_on_left", False):
            b -= c
        else:
            raise CodegenError(f"unexpected scalar operation {k} before Exp")
    return a, b


def _score_scale(flow, exp_node) -> float:
    return _score_affine(flow, exp_node)[0]


def _rms_eps(flow, rsqrt_node, k_extent) -> float:
    """eps of ``rsqrt(mean(x^2) + eps)``: the scalar operations between the sum of squares and ``RSqrt`` are
    composed into ``a * sum + b``; the form is an RMS norm over ``k_extent`` values when ``a * k_extent = 1``,
    and then eps = ``b``."""
    sums = [n for n in flow.ancestors(rsqrt_node).values() if _kind(n) == "ReduceSum"]
    if len(sums) != 1:
        raise CodegenError("RSqrt without exactly one sum of squares below it")
    a, b = 1.0, 0.0
    for n in flow.scalar_ops(rsqrt_node, stop=sums[0]):
        k, c = _kind(n), float(n.const)
        if k == "Div" and not getattr(n, "const_on_left", False):
            a, b = a / c, b / c
        elif k == "Mul":
            a, b = a * c, b * c
        elif k == "Add":
            b += c
        elif k == "Sub" and not getattr(n, "const_on_left", False):
            b -= c
        else:
            raise CodegenError(f"unexpected scalar operation {k} inside an RMS norm")
    if abs(a * k_extent - 1.0) > 1e-3:
        raise CodegenError(f"the normalisation divides the sum of squares by {1.0 / a:g}, not by the row length {k_extent}")
    return b


def _split_factor(flow) -> int:
    s = 1
    for n in flow.of("SplitView"):
        src = flow.preds(n)[0] if flow.preds(n) else None
        shp, axis = _shape(n), getattr(n, "axis", None)
        if src is not None and axis is not None and len(shp) == len(_shape(src)) + 1:
            s = max(s, shp[int(axis)])      # the split axis is inserted in front of the axis it cuts
        elif shp:
            s = max(s, shp[0])
    return s


class _Axes:
    """Which tensor axes a graph identifies with one another. Every placeholder axis gets a label; a matmul
    merges the labels of the two axes it contracts, an element-wise node those of equal extents it lines up.
    The resulting classes do not depend on how the search re-associated a product chain or which operands
    it transposed, so the part an input plays can be read off them: ``x @ w`` contracts the LAST axis of x
    with the FIRST axis of w however the plan writes it."""

    def __init__(self, flow: _Flow):
        self.flow, self.parent, self.labels, self.contractions = flow, {}, {}, []
        for n in flow.nodes:
            self.labels[id(n)] = self._visit(n)

    def find(self, a):
        while self.parent.setdefault(a, a) != a:
            self.parent[a] = self.parent[self.parent[a]]
            a = self.parent[a]
        return a

    def union(self, a, b):
        ra, rb = self.find(a), self.find(b)
        if ra != rb:
            self.parent[max(ra, rb, key=str)] = min(ra, rb, key=str)

    def _visit(self, n):
        k, shp, ps = _kind(n), _shape(n), self.flow.preds(n)
        if k.startswith("PlaceHolder"):
            return [(n.name, i) for i in range(len(shp))]
        ins = [self.labels[id(p)] for p in ps]
        if k == "Matmul":
            (la, lb) = ins
            if len(la) == 1:      # a vector operand (a reduced matrix) is a single row or column
                ar, ac = (n.name, "unit_a"), la[0]
            else:
                ar, ac = (la[-1], la[-2]) if getattr(n, "transpose_A", False) else (la[-2], la[-1])
            if len(lb) == 1:
                br, bc = lb[0], (n.name, "unit_b")
            else:
                br, bc = (lb[-1], lb[-2]) if getattr(n, "transpose_B", False) else (lb[-2], lb[-1])
            self.union(ac, br)
            self.contractions.append((n, ac))
            return [(n.name, "b", i) for i in range(len(shp) - 2)] + [ar, bc]
        if k == "SplitView":
            axis = int(getattr(n, "axis", 0))
            return ins[0][:axis] + [(n.name, "split")] + ins[0][axis:]
        if k in ("ReduceSum", "ReduceMax", "ReduceMin"):
            axis = int(getattr(n, "axis", len(ins[0]) - 1))
            if len(shp) == len(ins[0]):          # keepdims
                return ins[0][:axis] + [(n.name, "unit")] + ins[0][axis + 1:]
            return ins[0][:axis] + ins[0][axis + 1:]
        if len(ins) == 2 and len(ins[0]) == len(ins[1]):
            sa, sb = _shape(ps[0]), _shape(ps[1])
            for i, (x, y) in enumerate(zip(ins[0], ins[1])):
                if sa[i] == sb[i] and sa[i] != 1:
                    self.union(x, y)
            return list(ins[0] if sa >= sb else ins[1])
        if ins:
            best = max(ins, key=len)
            return list(best) if len(best) == len(shp) or not shp else list(best)[:len(shp)]
        return [(n.name, i) for i in range(len(shp))]

    def cls(self, node, axis):
        labs = self.labels[id(node)]
        return self.find(labs[axis])

    def contracted(self, mm):
        return next(self.find(c) for m, c in self.contractions if m is mm)


def _leaves(flow, node):
    """The placeholders ``node`` is computed from."""
    if _kind(node).startswith("PlaceHolder"):
        return [node]
    seen = [p for p in flow.ancestors(node).values() if _kind(p).startswith("PlaceHolder")]
    return sorted(seen, key=lambda n: flow.pos[id(n)])


def _axis_in(axes, ph, cls):
    """Position (counted from the end: -1 last, -2 second to last) of the axis of ``ph`` that lies in ``cls``."""
    rank = len(_shape(ph))
    for i in range(rank):
        if axes.cls(ph, i) == cls:
            return i - rank
    return None


def _plan_params(flow, dtype, roles: dict) -> tuple:
    """Inputs = the placeholders in graph order under their own names (the order and the names the
    reference's generated kernels use, python/cleave/runtime/reference.py:63-75), and the graph's output nodes
    with their physical shapes."""
    P = KernelParam
    ins = [P(n.name, _dtype_of(n, dtype), _shape(n), "input") for n in flow.nodes if _kind(n).startswith("PlaceHolder")]
    missing = set(roles.values()) - {p.name for p in ins}
    if missing:
        raise CodegenError(f"placeholders {sorted(missing)} are not in the graph")
    outs = [P(n.name, _dtype_of(n, dtype), _shape(n), "output") for n in flow.of("OutputNode")]
    return tuple(ins), tuple(outs)


def recognise(obj) -> KernelSpec:
    """The kernel a scheduled plan asks for. ``obj`` is a reference ``Plan``, its ``TileDict`` (anything with
    ``flat_graph``), a tiled graph, or a ``[partial, combine]`` pair, which becomes ONE fused kernel with the
    pair's split factor. A lone graph with ``SplitView`` nodes is a split partial (``role = "partial"``: it
    writes the per-split partial results the reference's two-stage form passes on), a lone graph that only
    sums placeholders along a split axis is its combine (family ``split_combine``).

    Families by op pattern: one ``Matmul`` -> matmul, with a sum of squares and ``RSqrt`` -> rmsnorm_matmul,
    with a ``ReduceSum`` over the product's columns -> matmul_rowsum; two with ``Silu`` -> swiglu; two around
    ``Exp`` -> attention_decode (``RSqrt`` below ``Exp`` -> qknorm_attention), two without -> matmul_matmul;
    three around ``Exp`` -> mla_decode; three without -> lora. The search also emits re-associated and
    transposed forms of a product chain (``q (k^T v)``, ``x @ rowsum(w)``, ``x (a b)``): they compute the same
    operator and give the same kernel."""
    fused = False
    if isinstance(obj, (list, tuple)):
        if not obj:
            raise CodegenError("empty plan list")
        obj, fused = obj[0], True
    flow = _Flow(obj)
    phs = [n for n in flow.nodes if _kind(n).startswith("PlaceHolder")]
    if not phs:
        raise CodegenError("the plan has no placeholders")
    dtype = _dtype_of(phs[0])
    mms, exps = flow.of("Matmul"), flow.of("Exp")
    split = _split_factor(flow)
    declared = getattr(obj, "split_factor", None)
    if declared:
        split = int(declared)
    role = "main" if fused or split == 1 else "partial"
    if not mms:
        return _recognise_combine(flow, dtype, obj)
    axes = _Axes(flow)
    name = lambda n: n.name  # noqa: E731

    def finish(family, dims, attrs, roles):
        attrs = dict(attrs)
        ins, outs = _plan_params(flow, dtype, roles)
        default = default_params(family, dtype, dims, attrs)
        if all(_ph(r) == roles[r] for r in roles):       # already under the library's own names
            params = default if role == "main" else tuple(ins) + tuple(outs)
        else:
            attrs["bind"] = {r: roles[r] for r in sorted(roles)}
            final = [p for p in default if p.role == "output"]
            params = tuple(ins) + (tuple(final) if role == "main" else tuple(outs))
        return KernelSpec(family, dtype, dict(dims), int(split), role, attrs, params)

    def two_d(ph, what):
        shp = _shape(ph)
        if len(shp) < 2:
            raise CodegenError(f"{what} {name(ph)} must be a matrix, got shape {shp}")
        return shp[-2], shp[-1]

    def left_right(mm, cands, what):
        """Of two inputs joined by the contraction of ``mm``: (the one contracted on its last axis, the one
        contracted on its second-to-last axis) - ``x`` and ``w`` of ``x @ w`` in whatever form it was written."""
        c = axes.contracted(mm)
        pos = {id(p): _axis_in(axes, p, c) for p in cands}
        left = [p for p in cands if pos[id(p)] == -1]
        right = [p for p in cands if pos[id(p)] == -2]
        if len(left) != 1 or len(right) != 1:
            raise CodegenError(f"{what}: the inputs are not laid out as (rows, contraction) @ (contraction, columns)")
        return left[0], right[0]

    if len(mms) == 1 and not exps:
        mm = mms[0]
        rs = flow.of("RSqrt", "Sqrt")
        sums = flow.of("ReduceSum")
        if rs:
            stat = rs[0]
            stat_in = _leaves(flow, stat)
            if len(stat_in) != 1:
                raise CodegenError("the norm statistics must come from one input")
            x = stat_in[0]
            rest = [p for p in phs if p is not x]
            w = next((p for p in rest if _axis_in(axes, p, axes.contracted(mm)) == -2), None)
            if w is None or _axis_in(axes, x, axes.contracted(mm)) != -1:
                raise CodegenError("rms_norm(x) @ w: x must be (M, K) and w (K, N)")
            (m, k), (_, n) = two_d(x, "x"), two_d(w, "w")
            roles = {"x": name(x), "w": name(w)}
            attrs = {"eps": _rms_eps(flow, stat, k)}
            others = [p for p in rest if p is not w]
            if others:
                if len(others) > 1 or _shape(others[0])[-1] != k:
                    raise CodegenError("unexpected extra inputs beside x, w and the norm weight")
                attrs["gamma"] = True
                roles["gamma"] = name(others[0])
            return finish("rmsnorm_matmul", {"M": m, "N": n, "K": k}, attrs, roles)
        if len(phs) != 2:
            raise CodegenError(f"one product over {len(phs)} inputs")
        x, w = left_right(mm, phs, "x @ w")
        (m, k), (_, n) = two_d(x, "x"), two_d(w, "w")
        roles = {"x": name(x), "w": name(w)}
        if sums and role == "main":
            # rowsum(x @ w) sums over w's columns, before the product (x @ rowsum(w)) or after it
            s_ = sums[0]
            src = flow.preds(s_)[0]
            dropped = axes.find(axes.labels[id(src)][int(getattr(s_, "axis", len(_shape(src)) - 1))])
            if dropped != axes.cls(w, len(_shape(w)) - 1) or len(sums) > 1:
                raise CodegenError("a product followed by a sum that is not over the product's columns")
            return finish("matmul_rowsum", {"M": m, "N": n, "K": k}, {}, roles)
        return finish("matmul", {"M": m, "N": n, "K": k}, {}, roles)

    if len(mms) == 2 and flow.of("Silu") and not exps:
        silu = flow.of("Silu")[0]
        gate = next((mm for mm in mms if flow.below(silu, mm)), None)
        up = next((mm for mm in mms if mm is not gate), None)
        if gate is None or up is None or len(phs) != 3:
            raise CodegenError("silu(x @ w0) * (x @ w1): Silu must be applied to one of two products of three inputs")
        gl, ul = _leaves(flow, gate), _leaves(flow, up)
        shared = [p for p in gl if p in ul]
        if len(shared) != 1 or len(gl) != 2 or len(ul) != 2:
            raise CodegenError("swiglu: both products must read one shared input and one weight each")
        x, w0 = left_right(gate, gl, "x @ w0")
        x2, w1 = left_right(up, ul, "x @ w1")
        if x is not shared[0] or x2 is not x:
            raise CodegenError("swiglu: the shared input must be the left operand of both products")
        (m, k), (_, n) = two_d(x, "x"), two_d(w0, "w0")
        return finish("swiglu", {"M": m, "N": n, "K": k}, {}, {"x": name(x), "w0": name(w0), "w1": name(w1)})

    if len(mms) == 2 and len(exps) == 1 and len(phs) == 3:
        e = exps[0]
        score = next((mm for mm in mms if flow.below(e, mm)), None)
        value = next((mm for mm in mms if flow.below(mm, e)), None)
        if score is None or value is None or score is value:
            raise CodegenError("attention: Exp must sit between the score product and the value product")
        qk = _leaves(flow, score)
        v = next((p for p in phs if p not in qk), None)
        if v is None or len(qk) != 2:
            raise CodegenError("attention: q, k and v must be three inputs")
        # k shares its sequence axis with v: the value product contracts the score columns with v's rows
        c = axes.contracted(value)
        k = next((p for p in qk if _axis_in(axes, p, c) is not None), None)
        q = next((p for p in qk if p is not k), None)
        if k is None or q is None or _axis_in(axes, v, c) != -2 or _axis_in(axes, k, c) != -2:
            raise CodegenError("attention: k and v must be (kv heads, kv length, d)")
        (hq, sq, d), (hkv, skv, _) = _shape(q)[-3:], _shape(k)[-3:]
        dims = {"HQ": hq, "HKV": hkv, "SQ": sq, "SKV": skv, "D": d}
        scale, shift = _score_affine(flow, e)
        attrs = {"scale": scale}
        if role == "partial":
            attrs["shift"] = shift
        roles = {"q": name(q), "k": name(k), "v": name(v)}
        rs = [r for r in flow.of("RSqrt", "Sqrt") if flow.below(e, r)]
        if rs:
            attrs["eps"] = _rms_eps(flow, rs[0], d)
            return finish("qknorm_attention", dims, attrs, roles)
        return finish("attention_decode", dims, attrs, roles)

    if len(mms) == 2 and not exps and len(phs) == 3:
        # (q k^T) v in either association: q and k are contracted on their last axes, k and v on their rows
        pairs = {}
        for mm in mms:
            c = axes.contracted(mm)
            pairs[id(mm)] = [(p, _axis_in(axes, p, c)) for p in phs if _axis_in(axes, p, c) is not None]
        d_pair = next((pr for pr in pairs.values() if len(pr) == 2 and all(a == -1 for _, a in pr)), None)
        s_pair = next((pr for pr in pairs.values() if len(pr) == 2 and all(a == -2 for _, a in pr)), None)
        if d_pair is None or s_pair is None:
            raise CodegenError("two products that are not (q k^T) v")
        k = next((p for p, _ in d_pair if any(p is p2 for p2, _ in s_pair)), None)
        q = next((p for p, _ in d_pair if p is not k), None)
        v = next((p for p, _ in s_pair if p is not k), None)
        if k is None or q is None or v is None:
            raise CodegenError("(q k^T) v: k must take part in both products")
        (hq, sq, d), (hkv, skv, _) = _shape(q)[-3:], _shape(k)[-3:]
        return finish("matmul_matmul", {"HQ": hq, "HKV": hkv, "SQ": sq, "SKV": skv, "D": d}, {},
                      {"q": name(q), "k": name(k), "v": name(v)})

    if len(mms) == 3 and len(exps) == 1 and len(phs) == 4:
        e = exps[0]
        scores = [mm for mm in mms if flow.below(e, mm)]
        value = next((mm for mm in mms if flow.below(mm, e)), None)
        if len(scores) != 2 or value is None:
            raise CodegenError("MLA decode: two score products below Exp and one value product above it")
        cv = axes.contracted(value)
        kv = next((p for p in phs if flow.below(value, p) and not flow.below(e, p)), None)
        if kv is None:      # the latent cache feeds a score product too, so it IS below Exp: take the value operand
            kv = next((p for p in _leaves(flow, value) if _axis_in(axes, p, cv) == -2 and
                       any(p in _leaves(flow, mm) for mm in scores) and len(_shape(p)) >= 2 and
                       _shape(p)[-1] == _shape(flow.of("OutputNode")[0])[-1]), None)
        main = next((mm for mm in scores if kv in _leaves(flow, mm)), None)
        rope = next((mm for mm in scores if mm is not main), None)
        if kv is None or main is None or rope is None:
            raise CodegenError("MLA decode: the latent cache must feed one score product and the value product")
        q = next((p for p in _leaves(flow, main) if p is not kv), None)
        rl = _leaves(flow, rope)
        k_pe = next((p for p in rl if _axis_in(axes, p, cv) is not None), None)   # shares the kv-length axis
        q_pe = next((p for p in rl if p is not k_pe), None)
        if q is None or k_pe is None or q_pe is None:
            raise CodegenError("MLA decode: q, q_pe and k_pe must be inputs")
        b_, h, d = _shape(q)[-3:]
        dims = {"B": b_, "H": h, "SKV": _shape(kv)[-2], "D": d, "PE": _shape(q_pe)[-1]}
        return finish("mla_decode", dims, {"scale": _score_scale(flow, e)},
                      {"q": name(q), "kv": name(kv), "q_pe": name(q_pe), "k_pe": name(k_pe)})

    if len(mms) == 3 and not exps and len(phs) == 4:
        # x @ w + (x @ a) @ b in any association: x is contracted (last axis) with the rows of both w and a,
        # a's columns with b's rows; w and b end in the output's columns
        cls_last = {id(p): axes.cls(p, len(_shape(p)) - 1) for p in phs}
        cls_first = {id(p): axes.cls(p, len(_shape(p)) - 2) for p in phs}
        x = next((p for p in phs if sum(1 for o in phs if o is not p and cls_first[id(o)] == cls_last[id(p)]) == 2), None)
        if x is None:
            raise CodegenError("x @ w + (x @ a) @ b: no input is contracted with two others")
        wa = [o for o in phs if o is not x and cls_first[id(o)] == cls_last[id(x)]]
        b = next((p for p in phs if p is not x and p not in wa), None)
        a = next((p for p in wa if cls_last[id(p)] == cls_first[id(b)]), None) if b is not None else None
        w = next((p for p in wa if p is not a), None)
        if a is None or w is None or cls_last[id(w)] != cls_last[id(b)]:
            raise CodegenError("x @ w + (x @ a) @ b: the low-rank pair does not line up with w")
        (m, k), (_, n), (_, r) = two_d(x, "x"), two_d(w, "w"), two_d(a, "a")
        return finish("lora", {"M": m, "N": n, "K": k, "R": r}, {},
                      {"x": name(x), "w": name(w), "a": name(a), "b": name(b)})

    kinds = sorted({_kind(n) for n in flow.nodes})
    raise CodegenError(f"no kernel family matches the plan's op pattern {kinds}")


def _recognise_combine(flow, dtype, obj) -> KernelSpec:
    """The combine stage of a split pair: every placeholder carries a split axis that a ``ReduceSum`` removes;
    an optional ``Div`` divides the first sum by the second, row by row (the split softmax denominator)."""
    phs = [n for n in flow.nodes if _kind(n).startswith("PlaceHolder")]
    sums = flow.of("ReduceSum")
    if not sums or len(sums) != len(phs) or any(flow.root(flow.preds(s)[0]) is None for s in sums):
        kinds = sorted({_kind(n) for n in flow.nodes})
        raise CodegenError(f"no kernel family matches the plan's op pattern {kinds}")
    extra = [n for n in flow.nodes if _kind(n) not in ("ReduceSum", "OutputNode", "Div") and not _kind(n).startswith("PlaceHolder")]
    if extra or len(flow.of("Div")) > 1 or len(sums) > 2:
        raise CodegenError("a combine stage with operations other than sums and one division")
    axis = int(getattr(sums[0], "axis", 0))
    split = _shape(flow.preds(sums[0])[0])[axis]
    declared = getattr(obj, "split_factor", None)
    axis_of = {id(flow.root(flow.preds(s)[0])): int(getattr(s, "axis", 0)) for s in sums}
    attrs = {"axes": [axis_of[id(p)] for p in phs], "divide": bool(flow.of("Div"))}
    if attrs["divide"]:      # which input is divided by which
        num, den = (flow.root(flow.preds(x)[0]) for x in flow.preds(flow.of("Div")[0]))
        order = [id(p) for p in phs]
        attrs["num"], attrs["den"] = order.index(id(num)), order.index(id(den))
    ins, outs = _plan_params(flow, dtype, {})
    return KernelSpec("split_combine", dtype, {}, int(declared or split), "combine", attrs, tuple(ins) + tuple(outs))
