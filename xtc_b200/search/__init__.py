"""Autotuning over the CUDA kernels' parameter space (the reference's ``xtc.search``)."""

from .explore import Exploration, ExplorationConfig
from .strategies import Strategies, StrategyCudaGemm

__all__ = ["Exploration", "ExplorationConfig", "Strategies", "StrategyCudaGemm"]
