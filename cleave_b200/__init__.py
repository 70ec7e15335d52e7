"""cleave_b200: hand-written sm_100a kernels behind Cleave's scheduled plans."""

from . import _lib  # noqa: F401
from ._lib import Cb200Error  # noqa: F401

__all__ = ["Cb200Error", "ops"]


def __getattr__(name):
    if name == "ops":
        from importlib import import_module

        return import_module(".ops", __name__)
    raise AttributeError(name)
