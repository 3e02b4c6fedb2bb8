"""neureka_b200: a CUDA (sm_100a) backend for Neureka's convolution / broadcast / elementwise path.

The product is the C-ABI library `libneureka_cuda.so` (include/neureka_cuda.h). This package is the
host-side mirror of the reference's plugin interface for that path -- NDConfiguration, Device,
ExecutionCall, ImplementationFor and the backend registration table -- used to drive the library
exactly the way Neureka's JVM side would.
"""
from .ndconf import NDConfiguration, Layout  # noqa: F401

__all__ = ["NDConfiguration", "Layout"]
