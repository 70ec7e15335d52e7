"""Scratch ownership helpers with the reference's names (python/cleave/runtime/autotune.py:169-263).

The reference's split-KV pairs expose their fp32 partial buffers as kernel parameters
(``Partial_<name>_{split,combine}``) and ``with_scratch`` hides them from the caller. The kernels of
this library fuse the combine and take their workspace through the C ABI, so a compiled kernel
has no partial parameters: ``with_scratch`` returns it unchanged and the workspace is owned, once
per (device, stream), by :func:`cleave_b200.ops.workspace`.
"""

from __future__ import annotations

_PARTIAL_PREFIX = "Partial_"


def _scratch_params(kernel):
    prim_func = kernel.adapter.prim_func
    return [(i, prim_func.buffer_map.get(p).name, prim_func.buffer_map.get(p).dtype)
            for i, p in enumerate(prim_func.params)
            if prim_func.buffer_map.get(p) is not None and prim_func.buffer_map.get(p).name.startswith(_PARTIAL_PREFIX)]


def with_scratch(kernel):
    """``kernel`` callable as ``(*inputs, *outputs)``; partial buffers, if it had any, would be
    owned here. Kernels of this library have none."""
    assert not _scratch_params(kernel), "fused kernels expose no partial buffers"
    return kernel


def param_index(kernel, buffer_name: str) -> int:
    """Position of ``buffer_name`` among the caller's tensor arguments."""
    inner = getattr(kernel, "kernel", kernel)
    prim_func = inner.adapter.prim_func
    for position, param in enumerate(prim_func.params):
        buffer = prim_func.buffer_map.get(param)
        if buffer is not None and buffer.name == buffer_name:
            return position
    raise KeyError(f"{buffer_name!r} is not a parameter of this kernel")
