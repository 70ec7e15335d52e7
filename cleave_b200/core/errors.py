"""The error family of the pipeline. The class names and their places in the hierarchy are the reference's
(python/cleave/core/errors.py), so that callers keep their ``except`` clauses; each class says here which stage
raises it, and ``for_stage`` is how the candidate farm types a failure by the stage it escaped from."""


class CleaveError(Exception):
    """Root of everything this package raises on purpose."""


class SpecError(CleaveError, ValueError):
    """The front door: a traced function that is none of the operators built here, an unbound dimension,
    an annotation that is not a tensor spec."""


class CodegenError(CleaveError):
    """Plan -> kernel text: the plan's op pattern has no kernel, or its layout is one the kernels do not read."""


class CompileError(CleaveError):
    """Kernel text -> bound kernel: the text does not define a kernel spec, the library is missing, or the
    stage has no kernel."""


class SmemExceeded(CompileError):
    """A plan that needs more shared memory than an SM has (kept for callers that catch it; the hand-written
    kernels size their own shared memory and refuse shapes with a status code instead)."""


class ValidationError(CleaveError, AssertionError):
    """A candidate whose output differs from the reference beyond the tolerance."""


class BenchmarkError(CleaveError):
    """A candidate that validated but could not be timed."""


class CandidateTimeout(CleaveError, TimeoutError):
    """A candidate that ran past its per-candidate limit in a worker (the worker's process group is killed)."""


class WorkerCrash(CleaveError):
    """A worker process that died without reporting (a crash fails one candidate, not the build)."""


class PagingRefusal(CleaveError, AssertionError):
    """A paged operator asked for with a layout the access layer does not cover (head_dim, latent widths)."""


_BY_STAGE = {"codegen": CodegenError, "compile": CompileError, "validate": ValidationError, "bench": BenchmarkError}


def for_stage(stage):
    """The error class a failure that escaped ``stage`` ("codegen", "compile", "validate", "bench") is reported
    as; a failure before any stage was entered counts against compile."""
    return _BY_STAGE.get(stage, CompileError)


__all__ = ["CleaveError", "SpecError", "CodegenError", "CompileError", "SmemExceeded", "ValidationError",
           "BenchmarkError", "CandidateTimeout", "WorkerCrash", "PagingRefusal", "for_stage"]
