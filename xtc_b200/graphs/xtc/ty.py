"""``import xtc_b200.graphs.xtc.ty as T`` (the reference's ``xtc.graphs.xtc.ty``)."""

from .core import Tensor, TensorType

__all__ = ["Tensor", "TensorType"]
