"""Autotuning over the CUDA kernels' parameter space (the reference's ``xtc.search``)."""

from .callback import CSVCallback, DBCallback, MemoryCallback, read_db
from .explore import Exploration, ExplorationConfig
from .optimizers import Optimizers
from .strategies import Strategies, StrategyCudaGemm

__all__ = ["CSVCallback", "DBCallback", "Exploration", "ExplorationConfig", "MemoryCallback",
           "Optimizers", "Strategies", "StrategyCudaGemm", "read_db"]
