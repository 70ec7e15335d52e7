"""The compile pipeline: plans, build, report, kernel (reference: python/cleave/pipeline)."""

from .build import BuiltKernel  # noqa: F401
from .compile import build, compile  # noqa: F401,A004
from .config import EvalConfig, list_presets  # noqa: F401
from .kernel import Kernel, Param, Stage, load  # noqa: F401
from .plans import Plan, PlanSet, schedule  # noqa: F401
from .report import Report, Result  # noqa: F401
