"""Error family and settings shared by the host-side layers."""
from .errors import *  # noqa: F401,F403
