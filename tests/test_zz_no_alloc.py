"""psx_b200_sample_rows_static: the sampling step for callers that are not allowed to allocate
device memory (a decode loop inside a server whose memory pool already owns the GPU, or a loop that
cannot afford cudaMalloc's device-wide synchronisation).  Its scratch is a fixed array inside the
library, shared by all calls, so the test calls it twice in a row -- the second call finds the
first call's leftovers in the array -- and checks both against the regular entry point on the same
inputs: token ids equal, log-probs within the 1e-5 relative tolerance of the other GPU tests.
Collected last (the file name sorts after the others), so a failure here cannot hide theirs."""
import numpy as np
import pytest

import gpu_harness as gh
import oracle_lib as ol
import pulsatrix_b200 as psx
import workload_rows
from pulsatrix_b200.workloads import WORKLOADS

pytestmark = pytest.mark.gpu


def _run_both(logits, hist, offsets, cfg, seeds):
    import torch
    rows = logits.shape[0]
    d_logits = torch.from_numpy(logits).cuda()
    d_hist = torch.from_numpy(np.ascontiguousarray(hist).ravel()).cuda()
    d_off = torch.from_numpy(offsets).cuda()
    d_u = torch.from_numpy(psx.uniforms_mt19937_64(seeds)).cuda()
    config = gh.psx_config(cfg)
    want = gh.ctx().sample_rows(d_logits, d_hist, d_off, config, d_u)
    torch.cuda.synchronize()
    tokens = torch.full((rows,), -7, dtype=torch.int64, device="cuda")
    log_probs = torch.zeros(rows, dtype=torch.float32, device="cuda")
    status = torch.full((rows,), -7, dtype=torch.int32, device="cuda")
    psx.sample_rows_static(d_logits, d_hist, d_off, config, d_u, tokens, log_probs, status)
    torch.cuda.synchronize()
    return ((want["tokens"].cpu().numpy(), want["log_probs"].cpu().numpy(), want["status"].cpu().numpy()),
            (tokens.cpu().numpy(), log_probs.cpu().numpy(), status.cpu().numpy()))


def test_static_entry_point_matches_the_regular_one_on_two_calls_in_a_row():
    # First call: 48 rows of C2 (480 parts).  Second call: a different, smaller batch with other
    # settings, which reuses the front of the same scratch array while the rest still holds call one.
    w = WORKLOADS["c2"]
    first = workload_rows.build("c2", np.arange(48))
    want, got = _run_both(first[0], first[1], first[2], workload_rows.config_of(w), first[3])
    assert (want[2] == 0).all() and (got[2] == 0).all()
    assert got[0].tolist() == want[0].tolist()
    assert (np.abs(got[1] - want[1]) <= 1e-5 * np.abs(want[1]) + 1e-9).all()

    w3 = WORKLOADS["c3"]
    second = workload_rows.build("c3", np.arange(20))
    want, got = _run_both(second[0], second[1], second[2], workload_rows.config_of(w3), second[3])
    assert (want[2] == 0).all() and (got[2] == 0).all()
    assert got[0].tolist() == want[0].tolist()
    assert (np.abs(got[1] - want[1]) <= 1e-5 * np.abs(want[1]) + 1e-9).all()

    # ... and the first batch once more, now over the second call's leftovers.
    want, got = _run_both(first[0], first[1], first[2], workload_rows.config_of(w), first[3])
    assert got[0].tolist() == want[0].tolist() and (got[2] == 0).all()
    assert (np.abs(got[1] - want[1]) <= 1e-5 * np.abs(want[1]) + 1e-9).all()


def test_static_entry_point_refuses_what_its_scratch_cannot_hold():
    import torch
    rows, vocab = 1025, 64  # 1025 parts: one more than the built-in scratch holds
    logits = torch.zeros((rows, vocab), device="cuda")
    tokens = torch.zeros(rows, dtype=torch.int64, device="cuda")
    log_probs = torch.zeros(rows, dtype=torch.float32, device="cuda")
    status = torch.zeros(rows, dtype=torch.int32, device="cuda")
    with pytest.raises(psx.PsxError) as err:
        psx.sample_rows_static(logits, None, None, psx.SamplingConfig.make(), None, tokens, log_probs, status)
    assert err.value.status == 4 and "1025 parts" in str(err.value) and "1024" in str(err.value)
    with pytest.raises(psx.PsxError) as err:  # settings are checked like everywhere else
        psx.sample_rows_static(logits[:4], None, None, psx.SamplingConfig.make(top_p=0.0), None, tokens, log_probs,
                               status)
    assert err.value.status == 1 and "top_p" in str(err.value)
    # greedy on a small batch, no history needed
    small = torch.randn((4, 3000), device="cuda", generator=torch.Generator(device="cuda").manual_seed(3))
    psx.sample_rows_static(small, None, None, psx.SamplingConfig.make(), None, tokens[:4], log_probs[:4], status[:4])
    torch.cuda.synchronize()
    assert tokens[:4].tolist() == small.argmax(dim=1).tolist() and (status[:4] == 0).all()
