"""Scratch ownership for compiled kernels, under the reference's names
(python/cleave/runtime/autotune.py:169-263).

The reference's split pairs expose their fp32 partial buffers as kernel parameters (``Partial_<name>_{split,
combine}``); ``with_scratch`` allocates them once per shape and hides them from the caller, so that a second call
allocates nothing (tests/graph/handwritten/test_splitkv_decode.py:85-111). The kernels of this library take their
split scratch as one workspace through the C ABI instead. ``with_scratch`` keeps the same promise in that form:
the wrapper it returns makes its first launch allocate the workspace, holds on to it (and so pins it for the
lifetime of the wrapper), and every later call on the same device and stream allocates nothing.
"""

from __future__ import annotations

_PARTIAL_PREFIX = "Partial_"


def _scratch_params(kernel):
    """``(position, buffer name, dtype)`` of the parameters that are partial buffers; kernels of this library
    have none (their scratch is the workspace)."""
    prim_func = kernel.adapter.prim_func
    found = []
    for position, param in enumerate(prim_func.params):
        buffer = prim_func.buffer_map.get(param)
        if buffer is not None and buffer.name.startswith(_PARTIAL_PREFIX):
            found.append((position, buffer.name, buffer.dtype))
    return found


class ScratchOwner:
    """``kernel`` with its workspace held by this object: callable as ``(*inputs, *outputs)``."""

    def __init__(self, kernel):
        if _scratch_params(kernel):
            raise ValueError("this kernel exposes partial buffers as parameters; the library's kernels take a workspace")
        self.kernel, self.adapter = kernel, kernel.adapter
        self._held: dict = {}

    def get_kernel_source(self) -> str:
        return self.kernel.get_kernel_source()

    @property
    def workspaces(self) -> list:
        """The workspace tensors this wrapper holds (one per kernel family, device and stream it has run on)."""
        return list(self._held.values())

    @property
    def scratch_bytes(self) -> int:
        return sum(t.numel() for t in self._held.values())

    def __call__(self, *args):
        from .. import ops

        before = dict(ops._workspaces)
        result = self.kernel(*args)
        for key, tensor in ops._workspaces.items():
            if key not in before or before[key] is not tensor or key in self._held:
                self._held[key] = tensor          # new, regrown, or already ours: keep the reference
        if not self._held:                        # the launch reused a workspace another kernel made: share it
            self._held.update({k: t for k, t in ops._workspaces.items() if k[2] == ops._stream()})
        return result


def with_scratch(kernel):
    """``kernel`` wrapped so that its split scratch is owned in one place and allocated once."""
    return kernel if isinstance(kernel, ScratchOwner) else ScratchOwner(kernel)


def param_index(kernel, buffer_name: str) -> int:
    """Position of ``buffer_name`` among the caller's tensor arguments."""
    inner = getattr(kernel, "kernel", kernel)
    prim_func = inner.adapter.prim_func
    for position, param in enumerate(prim_func.params):
        buffer = prim_func.buffer_map.get(param)
        if buffer is not None and buffer.name == buffer_name:
            return position
    raise KeyError(f"{buffer_name!r} is not a parameter of this kernel")
