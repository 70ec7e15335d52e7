"""cleave_b200: hand-written sm_100a kernels behind Cleave's scheduled plans.

The public surface mirrors the reference's (python/cleave/__init__.py): ``jit``, ``trace``, ``compile``,
``load``, ``Kernel``, ``Report``, the error family - with the code generator and runtime replaced by a
library of CUDA kernels reached through a C ABI.
"""

from importlib import import_module

from . import _lib  # noqa: F401
from ._lib import Cb200Error  # noqa: F401

_LAZY = {
    "B200CodeGen": ".codegen", "KernelSpec": ".codegen",
    "jit": ".frontend", "trace": ".frontend", "JitFunction": ".frontend", "Program": ".frontend",
    "compile": ".pipeline", "build": ".pipeline", "load": ".pipeline", "list_presets": ".pipeline",
    "EvalConfig": ".pipeline", "Plan": ".pipeline", "PlanSet": ".pipeline", "Report": ".pipeline",
    "Kernel": ".pipeline", "BuiltKernel": ".pipeline",
    "CleaveError": ".core.errors",
}
_SUBMODULES = {"ops", "lang", "codegen", "runtime", "pipeline", "frontend", "core", "workloads", "sharding",
               "microbench", "arch"}

__all__ = sorted(["Cb200Error", *_LAZY, *_SUBMODULES])


def __getattr__(name):
    if name in _SUBMODULES:
        return import_module(f".{name}", __name__)
    if name in _LAZY:
        return getattr(import_module(_LAZY[name], __name__), name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def __dir__():
    return __all__
