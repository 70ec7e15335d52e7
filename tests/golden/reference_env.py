"""A runnable copy of the reference's plan producer, for tests and fixture generators.

The reference's search and scheduling code (frontend -> IR -> C++ superoptimizer -> tile scheduler) is
CPU-side and out of scope for this library, but its OUTPUT - scheduled plans - is the input of the seam
this library fills (``TilelangCodeGen.gen``, python/cleave/codegen/__init__.py:24-48). This module makes
that producer importable where a reference checkout is available, so that real plans can be fed to
``cleave_b200.codegen``:

* a writable copy of ``python/cleave`` (the checkout itself may be read-only),
* the C++ superoptimizer compiled from ``src/superoptimizer/*.cc`` with plain ``g++`` calls and linked
  with its Cython binding into ``cleave/superoptimizer/core*.so``,
* stub ``graphviz`` and ``black`` modules (absent here; only used for drawing and for formatting text),
* the three ``tvm`` aliases the reference's pinned TileLang fork provides and upstream TileLang lacks
  (``tvm.tirx``, ``tvm.s_tir.Schedule``, ``tvm.s_tir.schedule.SBlockRV``).

Everything is written under one cache directory (``CLEAVE_B200_REF_ENV``, default a folder in the
system temp directory) and reused; nothing of the reference is copied into this repository.
"""

from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys
import sysconfig
import tempfile
import types
from concurrent.futures import ThreadPoolExecutor

REFERENCE_ROOT = os.environ.get("CLEAVE_REFERENCE_ROOT", "/root/reference")
ENV_DIR = os.environ.get("CLEAVE_B200_REF_ENV", os.path.join(tempfile.gettempdir(), "cleave_b200_ref_env"))


def available() -> bool:
    return os.path.isdir(os.path.join(REFERENCE_ROOT, "python", "cleave")) and \
        os.path.isdir(os.path.join(REFERENCE_ROOT, "src", "superoptimizer"))


def _site(*parts):
    import z3  # the pip package ships headers and libz3.so

    return os.path.join(os.path.dirname(os.path.abspath(z3.__file__)), *parts)


def _json_include():
    """nlohmann/json.hpp: the reference's 3rdparty/json submodule is empty; another installed package
    carries the header."""
    for base in sys.path:
        for cand in glob.glob(os.path.join(base, "**", "nlohmann", "json.hpp"), recursive=True):
            return os.path.dirname(os.path.dirname(cand))
    raise RuntimeError("nlohmann/json.hpp not found in site-packages")


def build(verbose: bool = False) -> str:
    """Builds (once) and returns the directory to put on ``sys.path``."""
    pkg_root = os.path.join(ENV_DIR, "python")
    ext_suffix = sysconfig.get_config_var("EXT_SUFFIX")
    so = os.path.join(pkg_root, "cleave", "superoptimizer", "core" + ext_suffix)
    if os.path.exists(so):
        return pkg_root
    os.makedirs(ENV_DIR, exist_ok=True)
    if not os.path.isdir(os.path.join(pkg_root, "cleave")):
        shutil.copytree(os.path.join(REFERENCE_ROOT, "python", "cleave"), os.path.join(pkg_root, "cleave"))
    gxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    inc = ["-I" + os.path.join(REFERENCE_ROOT, "include"), "-I" + _json_include(), "-I" + _site("include")]
    obj_dir = os.path.join(ENV_DIR, "obj")
    os.makedirs(obj_dir, exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(REFERENCE_ROOT, "src", "superoptimizer", "**", "*.cc"), recursive=True))

    def cc(src):
        rel = os.path.relpath(src, os.path.join(REFERENCE_ROOT, "src", "superoptimizer"))
        obj = os.path.join(obj_dir, rel.replace(os.sep, "_") + ".o")
        if not os.path.exists(obj):
            subprocess.check_call([gxx, "-std=c++17", "-O2", "-fPIC", "-fopenmp", "-w", *inc, "-c", src, "-o", obj],
                                  stdout=None if verbose else subprocess.DEVNULL)
        return obj

    with ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
        objs = list(ex.map(cc, srcs))
    cy_dir = os.path.join(ENV_DIR, "cython")
    os.makedirs(cy_dir, exist_ok=True)
    pyx = os.path.join(pkg_root, "cleave", "superoptimizer", "_cython", "core.pyx")
    cpp = os.path.join(cy_dir, "core.cpp")
    subprocess.check_call([sys.executable, "-m", "cython", "--cplus", "-3", pyx, "-o", cpp])
    py_inc = sysconfig.get_paths()["include"]
    z3_lib = _site("lib")
    subprocess.check_call([gxx, "-std=c++17", "-O2", "-fPIC", "-fopenmp", "-w", "-shared", *inc, "-I" + py_inc, cpp, *objs,
                           "-L" + z3_lib, "-lz3", "-Wl,-rpath," + z3_lib, "-o", so])
    return pkg_root


def _stub_modules():
    if "graphviz" not in sys.modules:
        try:
            import graphviz  # noqa: F401
        except ImportError:
            g = types.ModuleType("graphviz")

            class Digraph:  # drawing is never needed to produce a plan
                def __init__(self, *a, **k):
                    pass

                def __getattr__(self, name):
                    return lambda *a, **k: None

            g.Digraph = Digraph
            sys.modules["graphviz"] = g
    if "black" not in sys.modules:
        try:
            import black  # noqa: F401
        except ImportError:
            b = types.ModuleType("black")
            b.format_str = lambda src, mode=None, **k: src
            b.Mode = b.FileMode = lambda *a, **k: None
            sys.modules["black"] = b


def activate():
    """Builds the environment if needed, then makes ``import cleave`` resolve to it. Returns the package."""
    if not available():
        raise RuntimeError(f"no reference checkout at {REFERENCE_ROOT}")
    os.environ.setdefault("CUDA_VISIBLE_DEVICES", "")        # offline target of python/cleave/core/target.py:21-28
    os.environ.setdefault("CLEAVE_CACHE_ROOT", os.path.join(ENV_DIR, "cache"))
    pkg_root = build()
    _stub_modules()
    import tilelang  # noqa: F401  (must come first: it puts its bundled tvm on the path)
    import tvm

    if not hasattr(tvm, "tirx"):
        tvm.tirx = tvm.tir
        sys.modules.setdefault("tvm.tirx", tvm.tir)
    if not hasattr(tvm, "s_tir"):
        s_tir = types.ModuleType("tvm.s_tir")
        s_tir.Schedule = tvm.tir.Schedule
        sched = types.ModuleType("tvm.s_tir.schedule")
        sched.SBlockRV = tvm.tir.schedule.BlockRV
        s_tir.schedule = sched
        tvm.s_tir = s_tir
        sys.modules["tvm.s_tir"] = s_tir
        sys.modules["tvm.s_tir.schedule"] = sched
    if pkg_root not in sys.path:
        sys.path.insert(0, pkg_root)
    import cleave

    return cleave


if __name__ == "__main__":
    print(build(verbose=True))
