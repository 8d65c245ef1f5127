"""Runs the C++ test program of the host API (tests/cpp/host_api_test.cpp): the reference's own
generation, top-k, sampler and determinism tests restated against include/pulsatrix/*.hpp."""
import ctypes as C
import subprocess
from pathlib import Path

import numpy as np
import pytest

import oracle_lib as ol
from pulsatrix_b200 import build

BINARY = Path(__file__).resolve().parent / "cpp" / "host_api_test"


@pytest.fixture(scope="module")
def binary():
    build.build()
    if not BINARY.exists():
        build.build_cpp_test()
    return str(BINARY)


def test_host_only_part(binary):
    out = subprocess.run([binary, "--host-only"], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "0 failures" in out.stdout


def test_seed_stream_and_shuffle_order_equal_the_reference(binary):
    out = subprocess.run([binary, "--print-streams"], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0
    lines = dict(line.split(" ", 1) for line in out.stdout.strip().splitlines())
    ol.oracle().psxo_set_seed(C.c_uint64(5))
    assert [int(x) for x in lines["seeds"].split()] == [ol.oracle().psxo_next_seed() for _ in range(5)]
    if ol.reference_available():
        order = np.zeros(24, dtype=np.int64)
        ol.reference().psxref_shuffle_order(C.c_uint(41), C.c_int64(12), C.c_int64(2), order.ctypes.data_as(C.c_void_p))
        assert [int(x) for x in lines["shuffle"].split()] == order.tolist()


@pytest.mark.gpu
def test_all_of_it_on_the_gpu(binary):
    out = subprocess.run([binary, "--all", "40000"], capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-2000:]
    assert "0 failures" in out.stdout
