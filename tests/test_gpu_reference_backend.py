"""The boundary against the reference's real classes.  oracle/_ref/libpsx_refcuda.so holds the
reference's own src/cuda_backend.cu, src/top_k.cpp and friends compiled in place, plus a harness
that derives from the reference's CUDABackend and overrides top_k_rows with the call into
libpsx_b200.so -- the binding a maintainer of the reference would add.  Through it run the reference's own top_k()
and the inputs and checks of its TopKRowsMatchCPUBitExactly case
(tests/backend_primitive_equivalence_cases.hpp:345-375); the reference's unmodified kernel answers
the same questions beside it.  Skipped where the compiled reference is not present."""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest

import oracle_lib as ol
import pulsatrix_b200 as psx

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
HARNESS = ROOT / "oracle" / "_ref" / "libpsx_refcuda.so"


@pytest.fixture(scope="module")
def harness():
    if not HARNESS.exists():
        pytest.skip("the reference's CUDA backend has not been compiled here (make -C oracle refcuda)")
    lib = C.CDLL(str(HARNESS))
    lib.psxrefcuda_time_top_k_rows.restype = C.c_double
    return lib


def _top_k(lib, library, x, k, largest):
    rows, cols = x.shape
    values = np.zeros((rows, max(k, 1)), dtype=np.float32)
    indices = np.zeros((rows, max(k, 1)), dtype=np.float32)
    message = C.create_string_buffer(512)
    rc = lib.psxrefcuda_top_k(library, x.ctypes.data_as(C.c_void_p), C.c_int64(rows), C.c_int64(cols), C.c_int64(k),
                              C.c_int(int(largest)), values.ctypes.data_as(C.c_void_p), indices.ctypes.data_as(C.c_void_p),
                              message, C.c_int(512))
    return rc, values, indices, message.value.decode()


def test_the_references_equivalence_case_runs_through_the_override(harness):
    message = C.create_string_buffer(512)
    rc = harness.psxrefcuda_top_k_rows_match_cpu(str(psx.library_path()).encode(), message, C.c_int(512))
    assert rc == 0, message.value.decode()


def test_the_references_top_k_on_the_derived_backend_equals_its_own_kernel_and_the_cpu(harness):
    rng = np.random.RandomState(3)
    x = np.ascontiguousarray((np.round(rng.randn(37, 53) * 2) / 2).astype(np.float32))  # TopKTest's tie-heavy 37 x 53
    x[5, 7] = np.nan
    ours_lib = str(psx.library_path()).encode()
    for k in (1, 4, 17, 53):
        for largest in (True, False):
            rc_a, va, ia, msg = _top_k(harness, ours_lib, x, k, largest)
            rc_b, vb, ib, _ = _top_k(harness, None, x, k, largest)
            cv, ci = ol.top_k_rows("oracle", x, k, largest)
            assert rc_a == 0 and rc_b == 0, msg
            assert (ia == ci).all() and (ib == ci).all()
            assert va.view(np.uint32).tolist() == cv.view(np.uint32).tolist() == vb.view(np.uint32).tolist()
    # argument errors are the reference's own (src/top_k.cpp:14-17), whatever the backend
    rc, _, _, msg = _top_k(harness, ours_lib, x, 54, True)
    assert rc == 1 and "top_k: k must be in [1, 53]" in msg


def test_the_references_kernel_can_be_timed_beside_the_override(harness):
    ours = harness.psxrefcuda_time_top_k_rows(str(psx.library_path()).encode(), C.c_int64(64), C.c_int64(20000), C.c_int64(8), C.c_int(3))
    theirs = harness.psxrefcuda_time_top_k_rows(None, C.c_int64(64), C.c_int64(20000), C.c_int64(8), C.c_int(3))
    assert ours > 0 and theirs > 0
    print(f"top_k_rows 64 x 20000, k=8: override {ours:.1f} us per call, reference kernel {theirs:.1f} us per call")
