"""``@jit`` / ``trace``: run an annotated function on proxies and match it to a kernel family
(the call surface of python/cleave/frontend/jit.py and trace.py)."""

from __future__ import annotations

import inspect
from dataclasses import dataclass, field

from . import lang as cl
from .core.errors import SpecError


def _dtype_name(dtype) -> str:
    dt = dtype.name if isinstance(dtype, cl.DType) else (dtype or "float16")
    return {"f16": "float16", "bf16": "bfloat16"}.get(dt, dt)


class _DimsBuilder:
    """``program.dims`` before the program is closed: calling it names extents and returns their values
    (``M, K = p.dims(M=16, K=4096)``, python/cleave/frontend/program.py); afterwards the attribute is the
    plain dict of the matched family's extents."""

    def __init__(self):
        self.named = {}

    def __call__(self, **extents):
        self.named.update({k: int(v) for k, v in extents.items()})
        vals = tuple(int(v) for v in extents.values())
        return vals[0] if len(vals) == 1 else vals

    def __bool__(self):
        return False


@dataclass
class Program:
    """What ``compile`` needs to know about an operator: its family, extents and signature.

    ``trace`` fills every field. ``Program(name, dtype=...)`` alone starts the imperative builder of the
    reference (python/cleave/frontend/program.py; demo/lora.py): ``dims`` names extents, ``input`` declares
    tensors, ``output`` closes the program and matches its expression to a kernel family."""

    name: str
    family: str = ""
    dtype: str = "float16"
    dims: dict = field(default_factory=_DimsBuilder)  # the extents; a callable that names them while building
    attrs: dict = field(default_factory=dict)
    input_names: list = field(default_factory=list)
    input_shapes: list = field(default_factory=list)
    output_shapes: list = field(default_factory=list)
    split: tuple = ()
    bind: dict = field(default_factory=dict)  # kernel placeholder name -> Program input name

    def __post_init__(self):
        self.dtype = _dtype_name(self.dtype)

    # ---- imperative builder
    def input(self, name: str, shape):  # noqa: A003
        if self.family:
            raise SpecError(f"{self.name}: the program is closed; declare inputs before output()")
        shape = tuple(int(d) for d in shape)
        self.input_names.append(name)
        self.input_shapes.append(shape)
        return cl.Tensor(("in", name), shape)

    def output(self, value, name: str = "y"):
        if not isinstance(value, cl.Tensor):
            raise SpecError(f"{self.name}: output() takes a traced tensor")
        shapes = dict(zip(self.input_names, self.input_shapes))
        self.family, self.dims, self.attrs, bind = _match(value, shapes)
        self.output_shapes = [tuple(value.shape)]
        self.bind = {f"PlaceHolder_{k}": v for k, v in bind.items()}
        return value

    def fingerprint(self) -> dict:
        return {"family": self.family, "dtype": self.dtype, "dims": self.dims, "attrs": self.attrs,
                "inputs": self.input_names, "split": list(self.split)}


class JitFunction:
    def __init__(self, fn, dtype=None, split=None):
        self.fn, self.dtype, self.split = fn, dtype, split
        self.__name__ = getattr(fn, "__name__", "kernel")
        self.__doc__ = fn.__doc__

    def compile(self, shapes=None, dtype=None, **kw):
        from .pipeline.compile import compile as _compile

        return _compile(self, shapes=shapes, dtype=dtype or self.dtype, **kw)

    def __call__(self, *args):
        raise TypeError(f"{self.__name__}: call .compile(shapes=...) and run the returned kernel; "
                        "there is no eager CPU path")


def jit(fn=None, *, dtype=None, split=None):
    if fn is None:
        return lambda f: JitFunction(f, dtype, split)
    return JitFunction(fn, dtype, split)


def _const(e):
    return e[1] if isinstance(e, tuple) and e[0] == "const" else None


def _scaled(e):
    """``(inner, scale)`` for ``inner / c``, ``inner * c`` or ``c * inner``; else ``(e, None)``."""
    if e[0] == "div" and _const(e[2]) is not None:
        return e[1], 1.0 / _const(e[2])
    if e[0] == "mul":
        if _const(e[2]) is not None:
            return e[1], _const(e[2])
        if _const(e[1]) is not None:
            return e[2], _const(e[1])
    return e, None


def _is_in(e):
    return isinstance(e, tuple) and e[0] == "in"


def _as_rmsnorm(e):
    """``(input expr, eps)`` when ``e`` is ``x * rsqrt(mean(x * x) + eps)`` (either factor order, eps
    optional) or ``rms_norm(x, eps)``; else None."""
    if e[0] == "rms_norm":
        return e[1], e[2]
    if e[0] != "mul":
        return None
    for x, f in ((e[1], e[2]), (e[2], e[1])):
        if not (isinstance(f, tuple) and f[0] == "rsqrt"):
            continue
        ms, eps = f[1], 0.0
        if ms[0] == "add":
            if _const(ms[2]) is not None:
                ms, eps = ms[1], _const(ms[2])
            elif _const(ms[1]) is not None:
                ms, eps = ms[2], _const(ms[1])
        if ms[0] == "mean" and ms[1] == ("mul", x, x):
            return x, float(eps)
    return None


def _match(out, shapes):
    """``(family, dims, attrs, {placeholder: input name})`` for the traced expression ``out``."""
    e = out.expr
    if e[0] == "sum" and e[1][0] == "matmul" and _is_in(e[1][1]) and _is_in(e[1][2]):
        x, w = e[1][1][1], e[1][2][1]
        if len(shapes[x]) == 2 and len(shapes[w]) == 2 and len(out.shape) == 2:
            (m, k), (_, n) = shapes[x], shapes[w]
            return "matmul_rowsum", {"M": m, "N": n, "K": k}, {}, {"x": x, "w": w}
    if e[0] == "add":
        for base, low in ((e[1], e[2]), (e[2], e[1])):
            if (base[0] == "matmul" and _is_in(base[1]) and _is_in(base[2]) and low[0] == "matmul" and _is_in(low[2])
                    and low[1][0] == "matmul" and low[1][1] == base[1] and _is_in(low[1][2])):
                x, w, a, b = base[1][1], base[2][1], low[1][2][1], low[2][1]
                (m, k), (_, n), (_, r) = shapes[x], shapes[w], shapes[a]
                return "lora", {"M": m, "N": n, "K": k, "R": r}, {}, {"x": x, "w": w, "a": a, "b": b}
    if e[0] == "matmul":
        a, b = e[1], e[2]
        if a[0] == "matmul" and _is_in(a[1]) and a[2][0] == "T" and _is_in(a[2][1]) and _is_in(b) and len(out.shape) == 3:
            q, k, v = a[1][1], a[2][1][1], b[1]
            (hq, sq, d), (hkv, skv, _) = shapes[q], shapes[k]
            return ("matmul_matmul", {"HQ": hq, "HKV": hkv, "SQ": sq, "SKV": skv, "D": d}, {}, {"q": q, "k": k, "v": v})
        if a[0] == "softmax" and _is_in(b):
            inner, scale = _scaled(a[1])
            if inner[0] == "matmul" and inner[2][0] == "T":
                nq, nk = _as_rmsnorm(inner[1]), _as_rmsnorm(inner[2][1])
                if nq and nk and _is_in(nq[0]) and _is_in(nk[0]) and nq[1] == nk[1]:
                    q, k, v = nq[0][1], nk[0][1], b[1]
                    (hq, sq, d), (hkv, skv, _) = shapes[q], shapes[k]
                    attrs = {"eps": nq[1]}
                    if scale is not None:
                        attrs["scale"] = scale
                    return ("qknorm_attention", {"HQ": hq, "HKV": hkv, "SQ": sq, "SKV": skv, "D": d}, attrs,
                            {"q": q, "k": k, "v": v})
        if _is_in(a) and _is_in(b):
            (m, k), (_, n) = shapes[a[1]], shapes[b[1]]
            return "matmul", {"M": m, "N": n, "K": k}, {}, {"x": a[1], "w": b[1]}
        if a[0] == "rms_norm" and _is_in(a[1]) and _is_in(b):
            (m, k), (_, n) = shapes[a[1][1]], shapes[b[1]]
            return "rmsnorm_matmul", {"M": m, "N": n, "K": k}, {"eps": a[2]}, {"x": a[1][1], "w": b[1]}
        if a[0] == "mul" and _is_in(b):
            norm, g = (a[1], a[2]) if a[1][0] == "rms_norm" else (a[2], a[1])
            if norm[0] == "rms_norm" and _is_in(norm[1]) and _is_in(g):
                (m, k), (_, n) = shapes[norm[1][1]], shapes[b[1]]
                return ("rmsnorm_matmul", {"M": m, "N": n, "K": k}, {"eps": norm[2], "gamma": True},
                        {"x": norm[1][1], "gamma": g[1], "w": b[1]})
        if a[0] == "softmax" and _is_in(b):
            inner, scale = _scaled(a[1])
            if inner[0] == "matmul" and _is_in(inner[1]) and inner[2][0] == "T" and _is_in(inner[2][1]):
                q, k, v = inner[1][1], inner[2][1][1], b[1]
                (hq, sq, d), (hkv, skv, _) = shapes[q], shapes[k]
                return ("attention_decode", {"HQ": hq, "HKV": hkv, "SQ": sq, "SKV": skv, "D": d},
                        {} if scale is None else {"scale": scale}, {"q": q, "k": k, "v": v})
            if inner[0] == "add" and scale is not None:
                t1, t2 = inner[1], inner[2]
                ok = all(t[0] == "matmul" and _is_in(t[1]) and t[2][0] == "T" and _is_in(t[2][1]) for t in (t1, t2))
                if ok:
                    main, rope = (t1, t2) if t1[2][1][1] == b[1] else (t2, t1)
                    q, kv, qpe, kpe = main[1][1], main[2][1][1], rope[1][1], rope[2][1][1]
                    if kv == b[1]:
                        (bb, h, d), (_, skv, _), (_, _, pe) = shapes[q], shapes[kv], shapes[qpe]
                        return ("mla_decode", {"B": bb, "H": h, "SKV": skv, "D": d, "PE": pe}, {"scale": scale},
                                {"q": q, "kv": kv, "q_pe": qpe, "k_pe": kpe})
    if e[0] == "mul":
        gate, up = (e[1], e[2]) if e[1][0] == "silu" else (e[2], e[1])
        if gate[0] == "silu" and gate[1][0] == "matmul" and up[0] == "matmul":
            g, u = gate[1], up
            if all(_is_in(t) for t in (g[1], g[2], u[1], u[2])) and g[1] == u[1]:
                (m, k), (_, n) = shapes[g[1][1]], shapes[g[2][1]]
                return "swiglu", {"M": m, "N": n, "K": k}, {}, {"x": g[1][1], "w0": g[2][1], "w1": u[2][1]}
    raise SpecError("the traced function is none of the operators this library implements "
                    "(matmul, rms_norm(x) @ w, silu(x @ w0) * (x @ w1), softmax(q k^T c) v with or without RMS-normalised q and k, "
                    "MLA decode, (q k^T) v, rowsum(x @ w), x @ w + (x @ a) @ b)")


def trace(fn, shapes=None, dtype=None, *, split=None, name=None) -> Program:
    if isinstance(fn, JitFunction):
        dtype = dtype or fn.dtype
        split = fn.split if split is None else split
        name = name or fn.__name__
        fn = fn.fn
    shapes = dict(shapes or {})
    dt = _dtype_name(dtype)
    args, in_shapes, names = [], {}, []
    for p in inspect.signature(fn, eval_str=True).parameters.values():
        spec = p.annotation
        if not isinstance(spec, cl.TensorSpec):
            raise SpecError(f"{fn.__name__}: annotate {p.name!r} with cl.Tensor[...]")
        shape = []
        for d in spec.dims:
            if isinstance(d, int):
                shape.append(d)
            elif d in shapes:
                shape.append(int(shapes[d]))
            else:
                raise SpecError(f"{fn.__name__}: dim {d!r} of {p.name!r} unbound; pass shapes={{{d!r}: ...}}")
        in_shapes[p.name] = tuple(shape)
        names.append(p.name)
        args.append(cl.Tensor(("in", p.name), shape))
    out = fn(*args)
    if not isinstance(out, cl.Tensor):
        raise SpecError(f"{fn.__name__} must return a cl.Tensor")
    family, dims, attrs, bind = _match(out, in_shapes)
    splits = ()
    if split is not None and split is not False:  # split=False asks for the unsplit plan only
        splits = tuple(split.factors) if isinstance(split, cl.Split) else tuple(int(s) for s in split)
    return Program(name or fn.__name__, family, dt, dims, attrs, names, [in_shapes[n] for n in names],
                   [tuple(out.shape)], splits, {f"PlaceHolder_{k}": v for k, v in bind.items()})
