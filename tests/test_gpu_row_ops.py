"""softmax_rows, logsumexp_rows and gather_rows of the DeviceBackend on the GPU, through the C ABI,
against the CPU restatement of the reference's CPUBackend (src/cpu_backend.cpp:292-338,459-466).
Tolerance: the reference's own CPU/GPU equivalence tolerance of 1e-4
(tests/backend_primitive_equivalence_cases.hpp:22) for the float reductions; gather is bit-exact."""
import numpy as np
import pytest

import gpu_harness as gh
import oracle_lib as ol

pytestmark = pytest.mark.gpu
TOLERANCE = 1e-4

# one warp per row, one CTA, clusters of 2..8 CTAs, the three-walk kernel; odd widths take the scalar path
SHAPES = [(7, 1), (64, 33), (300, 129), (129, 1024), (37, 1025), (5, 4096), (9, 32768), (6, 49152), (3, 151936),
          (2, 128257), (2, 262144), (1, 300001)]


def _rows(rows, cols, seed):
    rng = np.random.RandomState(seed)
    x = (rng.randn(rows, cols) * 3).astype(np.float32)
    x[0, rng.randint(cols)] = 40.0  # one dominant entry
    if cols > 2:
        x[rows - 1, :2] = -np.inf   # removed logits, as ProcessLogits leaves them
    return x


@pytest.mark.parametrize("rows,cols", SHAPES)
def test_softmax_and_logsumexp_match_the_cpu_backend(rows, cols):
    import torch
    x = _rows(rows, cols, rows * 1000 + cols)
    d = torch.from_numpy(x).cuda()
    want = ol.row_primitive("oracle", "softmax_rows", x)
    got = gh.ctx().softmax_rows(d).cpu().numpy()
    assert np.abs(got - want).max() <= TOLERANCE
    assert np.allclose(got.sum(axis=1), 1.0, atol=1e-4)
    want_lse = ol.row_primitive("oracle", "logsumexp_rows", x)
    got_lse = gh.ctx().logsumexp_rows(d).cpu().numpy()
    assert np.abs(got_lse - want_lse).max() <= TOLERANCE * max(1.0, np.abs(want_lse).max())
    # in place: out may alias in
    gh.ctx().softmax_rows(d, out=d)
    torch.cuda.synchronize()
    assert d.cpu().numpy().tobytes() == got.tobytes()
    # same input, same bits
    assert gh.ctx().logsumexp_rows(torch.from_numpy(x).cuda()).cpu().numpy().tobytes() == got_lse.tobytes()


@pytest.mark.parametrize("count,dim,n", [(1, 1, 1), (31, 7, 50), (64, 128, 1000), (500, 4096, 33), (3, 151936, 5)])
def test_gather_rows_is_bit_exact(count, dim, n):
    import torch
    rng = np.random.RandomState(count + dim)
    table = rng.randn(n, dim).astype(np.float32)
    idx = rng.randint(0, n, size=count).astype(np.float32)
    got = gh.ctx().gather_rows(torch.from_numpy(table).cuda(), torch.from_numpy(idx).cuda()).cpu().numpy()
    assert got.tobytes() == ol.row_primitive("oracle", "gather_rows", table, idx).tobytes()


def test_empty_sizes_do_nothing():
    import torch
    x = torch.zeros((0, 5), device="cuda")
    assert gh.ctx().softmax_rows(x).shape == (0, 5)
    assert gh.ctx().logsumexp_rows(x).shape == (0,)
