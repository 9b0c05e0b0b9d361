"""accel_b200: a Blackwell (sm_100a) backend for the quantized decode path of golang-design/accel.

The product is `libaccelb200.so` (CUDA kernels + a C ABI, `include/accel_b200.h`).  This package is
the host side above it: `tensor` mirrors accel's operator interface for the path, `driver` binds
the Device/Block/Executable/Fence seam, `quant` and `blockpool` bind the host-side pieces, and
`runtime` dispatches single kernels on torch-owned memory.  There is no CPU path: importing works
anywhere, running needs the built library and a B200."""
from ._lib import AccelError, DeviceLost, LIB_PATH  # noqa: F401

__all__ = ["AccelError", "DeviceLost", "LIB_PATH"]
