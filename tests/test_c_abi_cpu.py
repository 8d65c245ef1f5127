"""CPU-only checks of the boundary: the library builds for sm_100a, loads, exports every entry
point that include/psx_b200.h declares, refuses to compute without a GPU, and its host-side
helpers reproduce the reference's uniform streams."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

import oracle_lib as ol
import pulsatrix_b200 as psx
from pulsatrix_b200 import binding, build

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    build.build()
    return psx.library()


def test_every_declared_entry_point_is_exported(lib):
    header = (ROOT / "include" / "psx_b200.h").read_text()
    declared = re.findall(r"PSX_API[^;(]*?\b(psx_\w+)\s*\(", header)
    assert sorted(declared) == sorted(binding.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.psx_b200_version() == b"0.1.0"


def test_struct_layouts_match_the_header():
    # sizeof / offsetof as a C compiler lays out psx_sampling_config and psx_row_diag
    assert C.sizeof(binding.SamplingConfig) == 64
    assert C.sizeof(binding.RowDiag) == 24
    assert binding.SamplingConfig.top_k.offset == 40 and binding.SamplingConfig.repetition_penalty.offset == 56


def test_uniform_streams_match_the_reference(lib):
    seeds = np.array([0, 1, 2, 17, 2**63 + 5, 2**64 - 1], dtype=np.uint64)
    assert (psx.uniforms_mt19937_64(seeds) == ol.mt_uniforms(seeds)).all()

    class Rng(C.Structure):
        _fields_ = [("state", C.c_uint64)]

    want = []
    for s in seeds:
        g = Rng(int(s))
        want.append(ol.oracle().psxo_prng_uniform(C.byref(g)))
    assert psx.uniforms_portable(seeds).tolist() == want


def test_no_gpu_means_an_error_not_a_fallback(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(psx.PsxError) as err:
        psx.Context(0)
    assert err.value.status == binding.ERR_CUDA and "CUDA error" in str(err.value)


def test_shard_record_size_follows_top_k(lib):
    cfg = psx.SamplingConfig.make(do_sample=True, top_k=64)
    assert lib.psx_b200_shard_record_bytes(C.addressof(cfg)) == 48 + 8 * 128
    cfg = psx.SamplingConfig.make(do_sample=False)
    assert lib.psx_b200_shard_record_bytes(C.addressof(cfg)) == 48 + 8 * 64


def test_exchange_entry_points_check_their_arguments_before_touching_a_gpu(lib):
    assert lib.psx_b200_exchange_handle_bytes() == 64  # sizeof(cudaIpcMemHandle_t)
    cfg = binding.SamplingConfig.make(do_sample=True, top_k=64)
    out, handle = C.c_void_p(), C.create_string_buffer(64)
    # no context: nothing is allocated, nothing is written
    assert lib.psx_b200_exchange_create(None, 2, 0, 8, C.addressof(cfg), C.byref(out), handle) == binding.ERR_BAD_ARGUMENT
    assert out.value is None and handle.raw == bytes(64)
    assert lib.psx_b200_exchange_open(None, handle) == binding.ERR_BAD_ARGUMENT
    assert lib.psx_b200_exchange_sample(None, None, None, 0, 0, 0, 0, None, None, C.addressof(cfg), None) == binding.ERR_BAD_ARGUMENT
    assert lib.psx_b200_exchange_results(None, None, None) == binding.ERR_BAD_ARGUMENT
    assert lib.psx_b200_exchange_test_wait(None, 0, 0) == binding.ERR_BAD_ARGUMENT
    lib.psx_b200_exchange_destroy(None)  # a null exchange is nothing to destroy
