"""Typed errors, mirroring the reference's family (python/cleave/core/errors.py:1-50) so that
callers can keep their ``except`` clauses."""


class CleaveError(Exception):
    pass


class SpecError(CleaveError, ValueError):
    pass


class CodegenError(CleaveError):
    pass


class CompileError(CleaveError):
    pass


class SmemExceeded(CompileError):
    pass


class ValidationError(CleaveError, AssertionError):
    pass


class CandidateTimeout(CleaveError, TimeoutError):
    pass


class WorkerCrash(CleaveError):
    pass


class PagingRefusal(CleaveError, AssertionError):
    pass


class BenchmarkError(CleaveError):
    pass


__all__ = ["CleaveError", "SpecError", "CodegenError", "CompileError", "SmemExceeded", "ValidationError",
           "CandidateTimeout", "WorkerCrash", "PagingRefusal", "BenchmarkError"]
