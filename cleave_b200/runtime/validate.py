"""Tolerances, the on-disk reference a worker validates against, and the check itself
(mirrors python/cleave/runtime/validate.py of the reference)."""

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


# The reference's loose default is 0.5 / 0.5 (python/cleave/runtime/validate.py:27); every kernel
# of this library is held to the tighter bound its 16-bit outputs allow against fp32.
DEFAULT_TOLERANCE = Tolerance(rtol=2e-2, atol=2e-2)
PAGED_TOLERANCE = Tolerance(rtol=1e-2, atol=1e-2)  # python/cleave/dynamic/registry.py:29


@dataclass(frozen=True)
class BenchOptions:
    warmup: int = 16
    iters: int = 1000


@contextlib.contextmanager
def _stage(name):
    """Tag an escaping exception with the pipeline stage it came from."""
    try:
        yield
    except BaseException as exc:
        if getattr(exc, "_cleave_stage", None) is None:
            try:
                exc._cleave_stage = name
            except Exception:  # noqa: BLE001 - some builtins reject attributes
                pass
        raise


_BENCHMARK_GRAPH_BATCH = 100
_REFERENCE_FILE_NAME = "reference.pt"


def benchmark_compiled_kernel(kernel, input_tensors, *, warmup_iters=0, profile_iters=1):
    """Mean milliseconds per launch, CUDA events around CUDA-graph replays."""
    return mean_launch_ms(kernel, input_tensors, warmup=warmup_iters, iters=profile_iters,
                          batch=_BENCHMARK_GRAPH_BATCH)


def _reference_cache_file(reference_cache_dir):
    return Path(reference_cache_dir) / _REFERENCE_FILE_NAME


def publish_reference(reference_cache_dir, spec, device="cuda"):
    """Build (inputs, reference) once in the parent and persist them for the workers.
    Returns ``(out_idx, io_bytes)``."""
    import torch

    from .compile import build_inputs_and_reference

    inputs_by_name, reference, out_idx = build_inputs_and_reference(spec, device=device)
    path = _reference_cache_file(reference_cache_dir)
    tmp = path.with_name(f"{path.name}.tmp.{os.getpid()}")
    os.makedirs(reference_cache_dir, exist_ok=True)
    torch.save({"inputs_by_name": inputs_by_name, "reference": list(reference)}, tmp)
    os.replace(tmp, path)
    io_bytes = sum(t.element_size() * t.nelement() for t in list(inputs_by_name.values()) + list(reference)
                   if hasattr(t, "nelement"))
    return out_idx, io_bytes


def _load_reference(reference_cache_dir, device="cuda"):
    import torch

    payload = torch.load(_reference_cache_file(reference_cache_dir), map_location=device, weights_only=True)
    return dict(payload["inputs_by_name"]), list(payload["reference"])


def _as_list(x):
    return list(x) if isinstance(x, (tuple, list)) else [x]


def _validate_kernel_outputs(kernel, inputs, reference, *, tolerance: Tolerance = DEFAULT_TOLERANCE):
    """Run ``kernel(*inputs)`` and assert it matches ``reference`` within ``tolerance``."""
    import torch

    actual = _as_list(kernel(*inputs))
    assert len(actual) == len(reference), (
        f"Kernel returned {len(actual)} outputs but the reference has {len(reference)}.")
    reference = [reconcile_output_layout(r, a.shape) for r, a in zip(reference, actual)]
    actual = [a.float() for a in actual]
    reference = [r.float() for r in reference]
    torch.testing.assert_close(actual, reference, rtol=tolerance.rtol, atol=tolerance.atol,
                               equal_nan=tolerance.equal_nan)
    if actual and actual[0].is_cuda:
        torch.cuda.synchronize()


def _check_kernel(kernel, *, spec=None, reference_cache_dir=None, tolerance: Tolerance = DEFAULT_TOLERANCE,
                  benchmark: BenchOptions | None = None):
    """Validate ``kernel`` against the reference, then optionally time it; returns mean ms or None."""
    from .compile import build_inputs_and_reference

    with _stage("validate"):
        if reference_cache_dir is not None:
            inputs_by_name, reference = _load_reference(reference_cache_dir)
        else:
            inputs_by_name, reference, _ = build_inputs_and_reference(spec)
        inputs = order_inputs_for_kernel(inputs_by_name, kernel)
        _validate_kernel_outputs(kernel, inputs, reference, tolerance=tolerance)
    if benchmark is None:
        return None
    with _stage("bench"):
        return benchmark_compiled_kernel(kernel, inputs, warmup_iters=benchmark.warmup,
                                         profile_iters=benchmark.iters)
