"""The vocabulary-sharded path across real GPUs: N ranks, one GPU each, every rank holds a column
shard of workload C5's rows.  Twice: with NCCL all-gathers of the per-row records and of the
results, and with no library collective at all -- records and results written straight into the
peers' memory over NVLink, counters in that memory saying when they are complete
(ShardedSampler(exchange="peer")).  Tokens must equal the reference fixture on every rank, also
when the rows do not divide evenly among the ranks.  Needs at least two GPUs; skipped otherwise
(tests/test_gpu_sharded.py and tests/test_gpu_peer_exchange.py cover one GPU)."""
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

WORKER = textwrap.dedent("""
    import os, sys
    import numpy as np, torch, torch.distributed as dist
    root = sys.argv[1]
    sys.path[:0] = [root, os.path.join(root, "tests")]
    import gpu_harness as gh, pulsatrix_b200 as psx, workload_rows
    from pulsatrix_b200.sharded import ShardedSampler, sample_rows_sharded, shard_bounds
    from pulsatrix_b200.workloads import WORKLOADS
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    w = WORKLOADS["c5"]
    ids = np.arange(0, 48)
    logits, hist, offsets, seeds = workload_rows.build("c5", ids)
    gold = np.load(os.path.join(root, "tests", "golden", "workload_c5.npz"))
    begin, cols = shard_bounds(w.vocab, world, rank)
    shard = torch.from_numpy(np.ascontiguousarray(logits[:, begin: begin + cols])).cuda()
    ctx = psx.Context(local)
    cfg = gh.psx_config(workload_rows.config_of(w))
    d_hist = torch.from_numpy(hist.ravel().astype(np.int64)).cuda()
    d_off = torch.from_numpy(offsets.astype(np.int64)).cuda()
    d_u = torch.from_numpy(psx.uniforms_mt19937_64(seeds)).cuda()
    for _ in range(3):
        out = sample_rows_sharded(ctx, shard, w.vocab, d_hist, d_off, cfg, d_u)
        torch.cuda.synchronize()
        assert (out["status"].cpu().numpy() == 0).all()
        assert out["tokens"].cpu().numpy().tolist() == gold["token"][ids].tolist()
        logp = out["log_probs"].cpu().numpy()
        assert (np.abs(logp - gold["log_prob"][ids]) <= 1e-5 * np.abs(gold["log_prob"][ids]) + 1e-9).all()
    # the same rows through peer memory; then fewer rows than divide evenly (the last ranks hold fewer, or none)
    for count in (48, 45, 5):
        sampler = ShardedSampler(ctx, count, w.vocab, cfg, torch.device("cuda", local), exchange="peer")
        o = d_off[: count + 1]
        for _ in range(4):
            sampler.step(shard[:count], d_hist, o, d_u[:count])
            torch.cuda.synchronize()
            out = sampler.flat()
            assert (out["status"].cpu().numpy() == 0).all(), (rank, count, out["status"].cpu().numpy())
            assert out["tokens"].cpu().numpy().tolist() == gold["token"][ids[:count]].tolist(), (rank, count)
            logp = out["log_probs"].cpu().numpy()
            want = gold["log_prob"][ids[:count]]
            assert (np.abs(logp - want) <= 1e-5 * np.abs(want) + 1e-9).all()
        sampler.close()
    dist.barrier()
    dist.destroy_process_group()
    print("ok", rank)
""")


def test_c5_over_nccl_ranks_matches_the_reference_fixture(tmp_path):
    import torch
    gpus = torch.cuda.device_count()
    if gpus < 2:
        pytest.skip("needs two GPUs")
    world = 8 if gpus >= 8 else 4 if gpus >= 4 else 2
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    proc = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                           "--master-addr", "127.0.0.1", "--master-port", "29677", str(script), str(ROOT)],
                          capture_output=True, text=True, timeout=600, env=env)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert proc.stdout.count("ok") == world
