"""``from xtc_b200.backends.cuda import Backend`` -- the B200 execution backend.

Plug point of the reference's search driver: ``xtc.backends.<name>.Backend``
(``search/explore.py:262-268``).
"""

from .backend import CudaBackend as Backend
from .scheduler import CudaSchedule, CudaScheduler, ScheduleError
from .compiler import CudaCompiler
from .module import CudaEvaluator, CudaExecutor, CudaModule

__all__ = ["Backend", "CudaScheduler", "CudaSchedule", "ScheduleError", "CudaCompiler",
           "CudaModule", "CudaEvaluator", "CudaExecutor"]
