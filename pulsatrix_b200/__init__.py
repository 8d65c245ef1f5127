"""pulsatrix_b200: B200 (sm_100a) kernels for pulsatrix's token-sampling path, behind a C ABI.

The product is `libpsx_b200.so` (sources in `csrc/`, header `include/psx_b200.h`).  This package
is the thin Python loader used by the tests and the benchmark: it binds the C entry points with
ctypes and hands them device pointers of torch tensors.  There is no Python or CPU
implementation of the path; when the library is missing, loading fails.
"""
from .binding import (Context, sample_rows_static, read_only_pass, RowDiag, SamplingConfig, library, library_path, uniforms_mt19937_64,  # noqa: F401
                      uniforms_portable, PsxError, ROW_OK, ROW_NON_FINITE, ROW_ALL_REMOVED, ROW_TOO_WIDE,
                      ROW_DEVICE_TIMEOUT, OK, ERR_BAD_ARGUMENT, ERR_CUDA, ERR_ROW_FAILED, ERR_UNSUPPORTED)
from .workloads import WORKLOADS, Workload  # noqa: F401

__version__ = "0.1.0"
