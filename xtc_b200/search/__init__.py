"""Autotuning over the CUDA kernels' parameter space (the reference's ``xtc.search``)."""

from .callback import CSVCallback, DBCallback, MemoryCallback, read_db
from .optimizers import Optimizers
from .strategies import Strategies, StrategyCudaGemm

__all__ = ["CSVCallback", "DBCallback", "Exploration", "ExplorationConfig", "MemoryCallback",
           "Optimizers", "Strategies", "StrategyCudaGemm", "read_db"]


def __getattr__(name: str):
    # the driver module is also the ``python -m xtc_b200.search.explore`` entry point: importing
    # it only on first use keeps it out of sys.modules until runpy executes it
    if name in ("Exploration", "ExplorationConfig"):
        from . import explore

        return getattr(explore, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
