"""Schedule front ends above the Scheduler interface."""

from .descript import descript_scheduler  # noqa: F401
