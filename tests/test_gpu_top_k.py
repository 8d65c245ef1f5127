"""top_k_rows on the GPU against the reference's cases: bit-exact values, indices and order
(tests/top_k_test.cpp:49-144, tests/backend_primitive_equivalence_cases.hpp:345-375)."""
import json
import math
from pathlib import Path

import numpy as np
import pytest

import gpu_harness as gh
import oracle_lib as ol
import pulsatrix_b200 as psx
from test_oracle_pins import _floats, tie_heavy_values

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


def gpu_top_k(x, k, largest=True, shift=0):
    import torch
    x = np.ascontiguousarray(x, dtype=np.float32)
    flat = torch.zeros(x.size + shift + 4, dtype=torch.float32, device="cuda")
    view = flat[shift: shift + x.size].view(*x.shape)
    view.copy_(torch.from_numpy(x))
    values, indices = gh.ctx().top_k_rows(view, k, largest)
    torch.cuda.synchronize()
    return values.cpu().numpy(), indices.cpu().numpy()


def same_bits(a, b):
    return a.shape == b.shape and bool(((a.view(np.uint32) == b.view(np.uint32)) | (np.isnan(a) & np.isnan(b))).all())


@pytest.mark.parametrize("case", json.loads((GOLDEN / "top_k_cases.json").read_text())["cases"], ids=lambda c: c["name"])
def test_known_answers(case):
    values, indices = gpu_top_k(_floats(case["row"])[None, :], case["k"], case["largest"])
    want = _floats(case["values"])
    assert ((values[0] == want) | (np.isnan(values[0]) & np.isnan(want))).all()
    assert indices[0].tolist() == case["indices"]


def test_tie_heavy_matrix_matches_the_cpu_bit_for_bit():
    rows, cols = 37, 53
    v = tie_heavy_values(rows * cols, 11)
    v[5] = np.nan
    v[cols + 9] = -np.inf
    x = v.reshape(rows, cols)
    for largest in (True, False):
        for k in (1, 4, 17, cols):
            gv, gi = gpu_top_k(x, k, largest)
            cv, ci = ol.top_k_rows("oracle", x, k, largest)
            assert (gi == ci).all() and same_bits(gv, cv)


def test_rows_spanning_blocks_match_the_cpu_bit_for_bit():
    rng = np.random.RandomState(41)
    x = ((rng.randint(0, 9, size=(300, 129)) - 4) * 0.5).astype(np.float32)
    x[0, 3] = np.nan
    x[1, 7] = np.inf
    x[2, 1] = -np.inf
    x[3, 0] = -0.0
    for largest in (True, False):
        for k in (1, 7, 129):
            for shift in (0, 1):
                gv, gi = gpu_top_k(x, k, largest, shift=shift)
                cv, ci = ol.top_k_rows("oracle", x, k, largest)
                assert (gi == ci).all() and same_bits(gv, cv)


def test_long_rows_and_large_k():
    rng = np.random.RandomState(7)
    x = (rng.randn(6, 100003) * 3).astype(np.float32)
    x[1] = np.round(x[1])          # many ties
    x[2, ::7] = np.nan
    x[3] = 1.5                     # all equal: the first k columns
    for k, largest in [(1, True), (64, True), (1000, False), (4096, True)]:
        gv, gi = gpu_top_k(x, k, largest)
        cv, ci = ol.top_k_rows("oracle", x, k, largest)
        assert (gi == ci).all() and same_bits(gv, cv)


@pytest.mark.parametrize("cols", [4097, 5000, 8192, 40000, 131072])
def test_k_beyond_the_shared_memory_sorter_up_to_whole_rows(cols):
    """k > 4096 sorts the rows whole in scratch memory; k = cols is a stable full sort (TopKTest sorts whole rows)."""
    rng = np.random.RandomState(cols)
    x = (rng.randn(3, cols) * 2).astype(np.float32)
    x[1] = np.round(x[1] * 2) / 2  # many ties: equal values keep the lower column first
    x[2, ::11] = np.nan
    x[2, 5] = np.inf
    x[2, 6] = -np.inf
    x[0, 3], x[0, 4] = -0.0, 0.0
    for k, largest in [(cols, True), (cols, False), (4097, True), ((cols + 4096) // 2, False)]:
        gv, gi = gpu_top_k(x, k, largest)
        cv, ci = ol.top_k_rows("oracle", x, k, largest)
        assert (gi == ci).all() and same_bits(gv, cv)


def test_argument_errors_use_the_reference_wording():
    import torch
    x = torch.zeros((2, 4), device="cuda")
    for k in (0, 5):
        with pytest.raises(psx.PsxError) as err:
            gh.ctx().top_k_rows(x, k)
        assert err.value.status == 1 and "top_k: k must be in [1, 4]" in str(err.value)
    values, indices = gh.ctx().top_k_rows(torch.zeros((0, 4), device="cuda"), 2)
    assert values.shape == (0, 2)
