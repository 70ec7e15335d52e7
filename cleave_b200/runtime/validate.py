"""The validate and bench stages of one candidate.

Contract shared with the reference (python/cleave/runtime/validate.py): a candidate is checked against a
reference that the parent process published once as ``<dir>/reference.pt`` = ``{"inputs_by_name",
"reference"}``; the check raises, and whatever escapes carries ``_cleave_stage`` in {"compile", "validate",
"bench"} so that the farm can type the failure; timing follows ``cleave_b200.runtime.timer``. The default
tolerance here is the 2e-2 / 2e-2 this library's 16-bit outputs are held to against fp32 (the reference's own
default, 0.5 / 0.5 at python/cleave/runtime/validate.py:27, is looser).
"""

from __future__ import annotations

import contextlib
import os
from dataclasses import dataclass
from pathlib import Path

from .reference import order_inputs_for_kernel, reconcile_output_layout
from .timer import mean_launch_ms


@dataclass(frozen=True)
class Tolerance:
    rtol: float
    atol: float
    equal_nan: bool = False


DEFAULT_TOLERANCE = Tolerance(rtol=2e-2, atol=2e-2)
PAGED_TOLERANCE = Tolerance(rtol=1e-2, atol=1e-2)  # python/cleave/dynamic/registry.py:29


@dataclass(frozen=True)
class BenchOptions:
    warmup: int = 16
    iters: int = 1000


_BENCHMARK_GRAPH_BATCH = 100
_REFERENCE_FILE_NAME = "reference.pt"


@contextlib.contextmanager
def _stage(name):
    """Whatever escapes the block is labelled with the stage it came from, unless an inner block
    already labelled it."""
    try:
        yield
    except BaseException as exc:
        if getattr(exc, "_cleave_stage", None) is None:
            with contextlib.suppress(Exception):  # a few builtin exception types take no attributes
                exc._cleave_stage = name
        raise


class ReferenceStore:
    """The published reference of one build: a single file in a directory the workers can read."""

    def __init__(self, directory):
        self.path = Path(directory) / _REFERENCE_FILE_NAME

    def publish(self, inputs_by_name: dict, reference: list) -> int:
        """Writes the payload so that a reader never sees half a file; returns the bytes of all tensors."""
        import torch

        self.path.parent.mkdir(parents=True, exist_ok=True)
        scratch = self.path.with_name(f"{self.path.name}.tmp.{os.getpid()}")
        torch.save({"inputs_by_name": dict(inputs_by_name), "reference": list(reference)}, scratch)
        os.replace(scratch, self.path)
        tensors = [*inputs_by_name.values(), *reference]
        return sum(t.numel() * t.element_size() for t in tensors if hasattr(t, "numel"))

    def read(self, device="cuda"):
        import torch

        blob = torch.load(self.path, map_location=device, weights_only=True)
        return dict(blob["inputs_by_name"]), list(blob["reference"])


def publish_reference(reference_cache_dir, spec, device="cuda"):
    """Build inputs and reference for ``spec`` once, in the parent, and persist them for the workers.
    Returns ``(out_idx, io_bytes)``."""
    from .compile import build_inputs_and_reference

    inputs_by_name, reference, out_idx = build_inputs_and_reference(spec, device=device)
    return out_idx, ReferenceStore(reference_cache_dir).publish(inputs_by_name, reference)


def _load_reference(reference_cache_dir, device="cuda"):
    return ReferenceStore(reference_cache_dir).read(device)


def benchmark_compiled_kernel(kernel, input_tensors, *, warmup_iters=0, profile_iters=1):
    """Mean milliseconds per launch (CUDA events around CUDA-graph replays)."""
    return mean_launch_ms(kernel, input_tensors, warmup=warmup_iters, iters=profile_iters,
                          batch=_BENCHMARK_GRAPH_BATCH)


def _validate_kernel_outputs(kernel, inputs, reference, *, tolerance: Tolerance = DEFAULT_TOLERANCE):
    """Launch once and compare every output with its reference in fp32; raises ``AssertionError`` naming
    the output that is off."""
    import torch

    produced = kernel(*inputs)
    produced = list(produced) if isinstance(produced, (list, tuple)) else [produced]
    if len(produced) != len(reference):
        raise AssertionError(f"Kernel returned {len(produced)} outputs but the reference has {len(reference)}.")
    for i, (got, want) in enumerate(zip(produced, reference)):
        want = reconcile_output_layout(want, got.shape)   # the kernel may keep unit axes the reference drops
        try:
            torch.testing.assert_close(got.float(), want.float(), rtol=tolerance.rtol, atol=tolerance.atol,
                                       equal_nan=tolerance.equal_nan)
        except AssertionError as exc:
            raise AssertionError(f"output {i}: {exc}") from None
    if produced and produced[0].is_cuda:
        torch.cuda.synchronize()  # a fault in the launch surfaces here, inside the validate stage


def _check_kernel(kernel, *, spec=None, reference_cache_dir=None, tolerance: Tolerance = DEFAULT_TOLERANCE,
                  benchmark: BenchOptions | None = None):
    """Validate, then (with ``benchmark``) time: mean milliseconds per launch, or None."""
    with _stage("validate"):
        if reference_cache_dir is None:
            from .compile import build_inputs_and_reference

            inputs_by_name, reference, _ = build_inputs_and_reference(spec)
        else:
            inputs_by_name, reference = _load_reference(reference_cache_dir)
        inputs = order_inputs_for_kernel(inputs_by_name, kernel)
        _validate_kernel_outputs(kernel, inputs, reference, tolerance=tolerance)
    if benchmark is None:
        return None
    with _stage("bench"):
        return benchmark_compiled_kernel(kernel, inputs, warmup_iters=benchmark.warmup,
                                         profile_iters=benchmark.iters)
