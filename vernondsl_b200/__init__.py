"""vernondsl_b200 -- B200 (sm_100a) execution backend for VernonDSL-style data-parallel kernels.

The product is ``libvrhi.so`` (CUDA kernels behind the C ABI of ``include/vrhi.h``); this package
is the thin Python host layer over it: handles (:mod:`rhi`), operator launches (:mod:`ops`), the
execution graph (:mod:`graph`), groups of GPUs (:mod:`group`, :mod:`partition`) and a small
Taichi-style front end for programs written like the reference's fractal.py (:mod:`lang`).
Nothing in the package computes on the CPU; without the built library it raises.
"""
from . import _lib
from ._lib import (EXACT, FAST, IMAGE, INPUT, JULIA, MANDELBROT, OUTPUT, STORAGE_BUFFER, UNIFORM, UNIFORM_CONSTANT,
                   VARYING, VrhiError, build)
from .rhi import Buffer, Device, Event, PinnedArray, Sequence, Stream

__all__ = ["Buffer", "Device", "Event", "PinnedArray", "Sequence", "Stream", "VrhiError", "build", "_lib", "INPUT", "OUTPUT",
           "UNIFORM", "UNIFORM_CONSTANT", "STORAGE_BUFFER", "IMAGE", "VARYING", "MANDELBROT", "JULIA", "EXACT", "FAST"]
