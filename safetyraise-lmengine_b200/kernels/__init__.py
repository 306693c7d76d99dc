"""Python face of the CUDA kernel library (ctypes over ``libsrlm_kernels.so``)."""
from .library import ops, KernelLibrary  # noqa: F401
