"""B200 (sm_100a) implementation of the poplin dense-contraction path.

The product is the shared library ``libpoplibs_b200.so`` (hand-written CUDA
kernels behind the C ABI declared in ``include/poplibs_b200.h``) and the C++
``poplin::`` layer on top of it.  This Python package only loads that library
through ctypes for the tests and the benchmark; it contains no arithmetic and
no fallback: if the library cannot be loaded, importing ``poplibs_b200.capi``
raises.
"""
from . import capi  # noqa: F401
from .capi import (ConvOptions, ConvParams, Context, MatmulDesc, Plan, PlbError, lib,  # noqa: F401
                   HALF, FLOAT, QUARTER)
