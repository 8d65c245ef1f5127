"""The vocabulary-sharded step over peer memory (psx_b200_exchange_*), as far as one GPU goes: a world
of one rank, whose only peer is itself, runs the whole chain -- row pass, records written through
the peer table, the survivor stage waiting on the arrival counters, results published and waited
for -- and must give the reference fixture's tokens.  The give-up path of the bounded waits is made
to run out with a count that nothing ever reaches; the exchange stays usable afterwards.  More
than one rank: tests/test_gpu_nccl_sharded.py."""
from pathlib import Path

import numpy as np
import pytest

import gpu_harness as gh
import pulsatrix_b200 as psx
import workload_rows
from pulsatrix_b200.workloads import WORKLOADS

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"
ROW_DEVICE_TIMEOUT = 32


def one_rank_exchange(name, ids):
    import torch
    w = WORKLOADS[name]
    logits, hist, offsets, seeds = workload_rows.build(name, ids)
    ctx = gh.ctx()
    config = gh.psx_config(workload_rows.config_of(w))
    ex = ctx.exchange(1, 0, len(ids), config)
    ex.open(ex.handle)
    tensors = (torch.from_numpy(logits).cuda(), torch.from_numpy(hist.ravel().astype(np.int64)).cuda(),
               torch.from_numpy(offsets.astype(np.int64)).cuda(), torch.from_numpy(psx.uniforms_mt19937_64(seeds)).cuda())
    return w, ctx, config, ex, tensors


def step(ex, w, config, tensors):
    import torch
    d_logits, d_hist, d_off, d_u = tensors
    out = ex.sample(d_logits, 0, w.vocab, d_hist, d_off, config, d_u)
    torch.cuda.synchronize()
    return {k: v.reshape(-1)[: d_logits.shape[0]].cpu().numpy() for k, v in out.items()}


@pytest.mark.parametrize("name,count", [("c5", 48), ("c2", 33), ("c4", 64)])
def test_one_rank_exchange_matches_the_reference_fixture(name, count):
    ids = np.arange(count)
    w, ctx, config, ex, tensors = one_rank_exchange(name, ids)
    gold = np.load(GOLDEN / f"workload_{name}.npz")
    try:
        for _ in range(3):  # the counters only grow: later steps must work like the first
            got = step(ex, w, config, tensors)
            assert (got["status"] == 0).all(), got["status"]
            assert got["tokens"].tolist() == gold["token"][ids].tolist()
            want = gold["log_prob"][ids]
            assert (np.abs(got["log_probs"] - want) <= 1e-5 * np.abs(want) + 1e-9).all()
    finally:
        ex.close()


def test_records_that_never_arrive_time_out_and_the_exchange_stays_usable():
    ids = np.arange(16)
    w, ctx, config, ex, tensors = one_rank_exchange("c5", ids)
    gold = np.load(GOLDEN / "workload_c5.npz")
    try:
        ex.test_wait(2_000_000, 1)  # 2 ms; one record more than the one rank will ever write
        got = step(ex, w, config, tensors)
        assert (got["status"] == ROW_DEVICE_TIMEOUT).all(), got["status"]
        assert (got["tokens"] == -1).all()
        ex.test_wait(0, 0)
        got = step(ex, w, config, tensors)
        assert (got["status"] == 0).all(), got["status"]
        assert got["tokens"].tolist() == gold["token"][ids].tolist()
    finally:
        ex.close()


def test_exchange_rejects_what_it_cannot_do():
    ctx = gh.ctx()
    config = gh.psx_config(workload_rows.config_of(WORKLOADS["c5"]))
    with pytest.raises(psx.binding.PsxError):
        ctx.exchange(9, 0, 8, config)  # one box: at most 8 ranks
    with pytest.raises(psx.binding.PsxError):
        ctx.exchange(2, 2, 8, config)  # the rank lies outside the world
    ex = ctx.exchange(1, 0, 8, config)
    try:
        import torch
        with pytest.raises(psx.binding.PsxError):  # not open yet
            ex.sample(torch.zeros((8, 64), device="cuda"), 0, 64, torch.zeros(8, dtype=torch.int64, device="cuda"),
                      torch.arange(9, dtype=torch.int64, device="cuda"), config, torch.zeros(8, dtype=torch.float64, device="cuda"))
    finally:
        ex.close()
