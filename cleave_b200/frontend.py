"""``@jit`` / ``trace``: run an annotated function on proxies and match it to a kernel family
(the call surface of python/cleave/frontend/jit.py and trace.py)."""

from __future__ import annotations

import inspect
from dataclasses import dataclass, field

from . import lang as cl
from .core.errors import SpecError


@dataclass
class Program:
    """What ``compile`` needs to know about an operator: its family, extents and signature."""

    name: str
    family: str
    dtype: str
    dims: dict
    attrs: dict
    input_names: list
    input_shapes: list
    output_shapes: list
    split: tuple = ()
    bind: dict = field(default_factory=dict)  # kernel placeholder name -> Program input name

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


def _match(out, shapes):
    """``(family, dims, attrs, {placeholder: input name})`` for the traced expression ``out``."""
    e = out.expr
    if e[0] == "matmul":
        a, b = e[1], e[2]
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
                    "(matmul, rms_norm(x) @ w, silu(x @ w0) * (x @ w1), softmax(q k^T c) v, MLA decode)")


def trace(fn, shapes=None, dtype=None, *, split=None, name=None) -> Program:
    if isinstance(fn, JitFunction):
        dtype = dtype or fn.dtype
        split = fn.split if split is None else split
        name = name or fn.__name__
        fn = fn.fn
    shapes = dict(shapes or {})
    dt = dtype.name if isinstance(dtype, cl.DType) else (dtype or "float16")
    dt = {"f16": "float16", "bf16": "bfloat16"}.get(dt, dt)
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
    if split is not None:
        splits = tuple(split.factors) if isinstance(split, cl.Split) else tuple(int(s) for s in split)
    return Program(name or fn.__name__, family, dt, dims, attrs, names, [in_shapes[n] for n in names],
                   [tuple(out.shape)], splits, {f"PlaceHolder_{k}": v for k, v in bind.items()})
