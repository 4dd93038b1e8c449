from . import lib, ops  # noqa: F401
from .lib import KernelError, launch_count

__all__ = ["KernelError", "launch_count", "lib", "ops"]
