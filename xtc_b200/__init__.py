"""xtc_b200 -- a B200 (sm_100a) execution backend for XTC dataflow graphs.

``xtc_b200.graphs.xtc.op`` builds graphs with the reference's operator API and
``xtc_b200.backends.cuda.Backend`` runs them on hand-written CUDA kernels
through the C ABI of ``libxtc_cuda.so`` (``include/xtc_cuda.h``).
"""

__version__ = "0.1.0"
