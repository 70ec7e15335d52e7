"""``import cleave_b200.lang as cl``: the slice of the reference's ``cleave.lang`` that its demo
operators use (python/cleave/lang.py, python/cleave/frontend/composites.py): tensor annotations, dtypes,
``rms_norm`` / ``silu`` / ``softmax`` and a split request. A traced function is matched against the
operator families the kernel library implements; anything else is refused - the general frontend,
IR and superoptimizer of the reference are not part of this package.
"""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class DType:
    name: str


f16, bf16, f32, i32 = DType("float16"), DType("bfloat16"), DType("float32"), DType("int32")


@dataclass(frozen=True)
class Split:
    dim: str
    factors: tuple = (4, 8, 16)

    def __init__(self, dim, factors=(4, 8, 16)):
        object.__setattr__(self, "dim", dim)
        object.__setattr__(self, "factors", tuple(int(f) for f in (factors if isinstance(factors, (tuple, list)) else (factors,))))


@dataclass(frozen=True)
class TensorSpec:
    dims: tuple
    dtype: DType | None = None


class Tensor:
    """``cl.Tensor["M", "K"]`` as an annotation; a traced value inside a ``@jit`` function."""

    def __class_getitem__(cls, dims):
        return TensorSpec(tuple(dims) if isinstance(dims, tuple) else (dims,))

    def __init__(self, expr, shape):
        self.expr, self.shape = expr, tuple(shape)

    @property
    def mT(self):
        return Tensor(("T", self.expr), self.shape[:-2] + (self.shape[-1], self.shape[-2]))

    def __matmul__(self, other):
        if self.shape[-1] != other.shape[-2]:
            raise ValueError(f"matmul: inner extents differ, {self.shape} @ {other.shape}")
        lead = self.shape[:-2] if len(self.shape) >= len(other.shape) else other.shape[:-2]
        lead = tuple(max(a, b) for a, b in zip(self.shape[:-2], other.shape[:-2])) if len(self.shape) == len(other.shape) else lead
        return Tensor(("matmul", self.expr, other.expr), lead + (self.shape[-2], other.shape[-1]))

    def _bin(self, kind, other, swap=False):
        o = other.expr if isinstance(other, Tensor) else ("const", float(other))
        a, b = (o, self.expr) if swap else (self.expr, o)
        return Tensor((kind, a, b), self.shape)

    def __mul__(self, other):
        return self._bin("mul", other)

    def __rmul__(self, other):
        return self._bin("mul", other, swap=True)

    def __truediv__(self, other):
        return self._bin("div", other)

    def __add__(self, other):
        return self._bin("add", other)

    def __radd__(self, other):
        return self._bin("add", other, swap=True)

    def _last_axis(self, dim, what):
        if dim not in (-1, len(self.shape) - 1):
            raise ValueError(f"{what} is taken along the last axis")

    def sum(self, dim: int = -1, keepdim: bool = False):  # noqa: A003
        self._last_axis(dim, "sum")
        return Tensor(("sum", self.expr), self.shape[:-1] + ((1,) if keepdim else ()))

    def mean(self, dim: int = -1, keepdim: bool = False):
        """``sum / extent`` as the reference defines it (python/cleave/frontend/tensor.py:273-274)."""
        self._last_axis(dim, "mean")
        return Tensor(("mean", self.expr), self.shape[:-1] + ((1,) if keepdim else ()))

    def rsqrt(self):
        return Tensor(("rsqrt", self.expr), self.shape)


def rms_norm(x, dim: int = -1, eps: float = 0.0):
    """``x * rsqrt(mean(x*x) + eps)`` along the last axis, without weight."""
    if dim not in (-1, len(x.shape) - 1):
        raise ValueError("rms_norm is taken along the last axis")
    return Tensor(("rms_norm", x.expr, float(eps)), x.shape)


def rsqrt(x):
    return x.rsqrt()


def sum(x, dim: int = -1, keepdim: bool = False):  # noqa: A001
    return x.sum(dim, keepdim)


def mean(x, dim: int = -1, keepdim: bool = False):
    return x.mean(dim, keepdim)


def silu(x):
    return Tensor(("silu", x.expr), x.shape)


def softmax(x, dim: int = -1, shift=None):
    """Softmax along the last axis. A constant ``shift`` (the demos' stand-in for the row max)
    does not change the result and is dropped: the kernels use the exact running maximum."""
    if dim not in (-1, len(x.shape) - 1):
        raise ValueError("softmax is taken along the last axis")
    return Tensor(("softmax", x.expr), x.shape)


def matmul(a, b):
    return a @ b
