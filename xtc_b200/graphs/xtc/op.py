"""``import xtc_b200.graphs.xtc.op as O`` -- the operator factory.

Same names and arguments as the reference's ``xtc.graphs.xtc.op``
(``op_factory.py:38-112``, ``builder.py:16-33``).
"""

from __future__ import annotations

from typing import Any

from .core import CONTEXT, Expr, TensorType, graph_builder as graph, make_op, make_tensor

__all__ = ["graph", "tensor", "matmul", "conv2d", "relu", "pad", "pad2d", "unpad", "reshape",
           "transpose", "inputs", "outputs", "type"]


def tensor(*args: Any, name: str | None = None, **attrs: Any) -> Expr:
    return make_tensor(*args, name=name, **attrs)


def matmul(a: Expr, b: Expr, name: str | None = None, **attrs: Any) -> Expr:
    return make_op("matmul", (a, b), name, **attrs)


def conv2d(inp: Expr, weight: Expr, name: str | None = None, **attrs: Any) -> Expr:
    return make_op("conv2d", (inp, weight), name, **attrs)


def relu(inp: Expr, name: str | None = None, **attrs: Any) -> Expr:
    return make_op("relu", (inp,), name, **attrs)


def pad(inp: Expr, name: str | None = None, **attrs: Any) -> Expr:
    return make_op("pad", (inp,), name, **attrs)


def pad2d(inp: Expr, name: str | None = None, **attrs: Any) -> Expr:
    return make_op("pad2d", (inp,), name, **attrs)


def unpad(inp: Expr, name: str | None = None, **attrs: Any) -> Expr:
    return make_op("unpad", (inp,), name, **attrs)


def reshape(inp: Expr, name: str | None = None, **attrs: Any) -> Expr:
    return make_op("reshape", (inp,), name, **attrs)


def transpose(inp: Expr, name: str | None = None, **attrs: Any) -> Expr:
    return make_op("transpose", (inp,), name, **attrs)


def outputs(*outs: Expr) -> None:
    CONTEXT.stack[-1].outputs.extend(outs)


def inputs(*inps: Expr) -> None:
    CONTEXT.stack[-1].inputs.extend(inps)


def type(*args: Any, **attrs: Any) -> TensorType:
    return TensorType(*args, **attrs)
