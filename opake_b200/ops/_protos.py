"""ctypes prototypes of the non-GEMM entry points of libopake_kernels.so (see csrc/kernels/opk_api.h)."""
from ctypes import c_double, c_float, c_int32, c_int64, c_uint64, c_void_p

PROTOTYPES: dict = {}
