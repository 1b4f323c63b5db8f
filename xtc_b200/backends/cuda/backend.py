"""Backend object of the CUDA target (cf. ``backends/mlir/MlirBackend.py:19-76``
and ``MlirGraphBackend.py:31-60``)."""

from __future__ import annotations

import tempfile
from pathlib import Path
from typing import Any

from .compiler import CudaCompiler
from .scheduler import CudaSchedule, CudaScheduler


class CudaBackend:
    """``Backend(graph)``: scheduler and compiler factory for one graph.

    Extra keyword arguments other backends understand (``use_tensor_dialect``,
    ``always_vectorize``, ``no_alias``, ...) are accepted and ignored so the
    reference's search driver can instantiate it unchanged.
    """

    def __init__(self, graph: Any, **_ignored: Any) -> None:
        self._graph = graph
        self.payload_name = graph.name or "payload"
        assert graph.inputs_types is not None, (
            "graph inputs need constant shapes and dtypes (types were not forwarded)")

    @property
    def graph(self) -> Any:
        return self._graph

    def get_scheduler(self, **kwargs: Any) -> CudaScheduler:
        return CudaScheduler(self, **kwargs)

    def get_compiler(self, **kwargs: Any) -> CudaCompiler:
        return CudaCompiler(self, **kwargs)

    def np_inputs_spec(self) -> list[dict[str, Any]]:
        return [{"shape": tuple(t.shape), "dtype": str(t.dtype), "device": getattr(t, "device", None),
                 "layout": getattr(t, "layout", None)} for t in self._graph.inputs_types]

    def np_outputs_spec(self) -> list[dict[str, Any]]:
        return [{"shape": tuple(t.shape), "dtype": str(t.dtype), "device": getattr(t, "device", None)}
                for t in self._graph.outputs_types]

    def reference_impl(self, *args: Any) -> None:
        """NumPy evaluation of the graph into the trailing output arrays."""
        from ...graphs.xtc.core import Tensor

        n_in = len(self._graph.inputs)
        tensor_cls = Tensor
        outs = self._graph.forward([tensor_cls(a) for a in args[:n_in]])
        for dst, src in zip(args[n_in:], outs):
            dst[:] = src.numpy()

    def evaluate(self, schedule: CudaSchedule, compiler_args: dict = {},
                 evaluate_args: dict = {}) -> float | str:
        """Compile, validate against the NumPy graph, time; min seconds or the error text."""
        with tempfile.TemporaryDirectory() as dirname:
            libpath = Path(dirname) / f"payload_{self.payload_name}"
            compiler = self.get_compiler(dump_file=str(libpath), shared_lib=True, **compiler_args)
            module = compiler.compile(schedule)
            evaluator = module.get_evaluator(validate=True, **evaluate_args)
            results, code, error_msg = evaluator.evaluate()
        return min(results) if code == 0 else error_msg
