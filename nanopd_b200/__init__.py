"""nanopd_b200 — the paged-attention hot path of nanoPD, written for NVIDIA B200 (sm_100a).

The product is the C-ABI library ``libnanopd_b200.so`` (declared in ``include/nanopd_b200.h``)
and :mod:`nanopd_b200.paged_kernels`, a ctypes binding that keeps the Python op signatures of
the reference's ``paged_kernels`` extension.  There is no CPU or PyTorch fallback: importing
``paged_kernels`` raises if the library has not been built.
"""
__version__ = "0.1.0"
