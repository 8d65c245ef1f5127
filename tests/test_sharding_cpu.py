"""Host-side logic of the multi-GPU paths on CPU: the column partition, and, with two gloo
ranks, that an all-gather of per-rank records lands shard-major as the survivor stage reads it
and that the row split of the benchmark covers every row once."""
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

from pulsatrix_b200.sharded import gathered_layout, row_bounds, shard_bounds

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("vocab,world", [(262144, 8), (151936, 8), (49152, 4), (1001, 3), (7, 8), (128256, 2)])
def test_shards_tile_the_vocabulary(vocab, world):
    covered = 0
    for rank in range(world):
        begin, cols = shard_bounds(vocab, world, rank)
        assert begin == covered or cols == 0
        assert begin % 4 == 0 or cols == 0
        covered = begin + cols
    assert covered == vocab
    with pytest.raises(ValueError):
        shard_bounds(vocab, world, world)


@pytest.mark.parametrize("rows,world", [(512, 8), (48, 8), (13, 4), (3, 8), (1, 2), (64, 1)])
def test_row_blocks_tile_the_rows(rows, world):
    covered, sizes = 0, set()
    for rank in range(world):
        begin, count, per = row_bounds(rows, world, rank)
        assert begin == covered and 0 <= count <= per
        covered += count
        sizes.add(per)
    assert covered == rows and len(sizes) == 1 and sizes.pop() * world >= rows


def test_gathered_layout_is_shard_major():
    offsets, per = gathered_layout(rows=512, record_bytes=1072, world=8)
    assert per == 512 * 1072 and offsets == [s * per for s in range(8)]


WORKER = textwrap.dedent("""
    import os, sys
    import torch, torch.distributed as dist
    sys.path.insert(0, sys.argv[1])
    from pulsatrix_b200.sharded import gathered_layout, shard_bounds
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    rows, record = 6, 40
    mine = torch.full((rows * record,), rank + 1, dtype=torch.uint8)
    mine[::record] = torch.arange(rows, dtype=torch.uint8)           # first byte of each record: its row
    gathered = torch.empty(world * rows * record, dtype=torch.uint8)
    dist.all_gather_into_tensor(gathered, mine)
    offsets, per = gathered_layout(rows, record, world)
    for s in range(world):
        block = gathered[offsets[s]: offsets[s] + per].view(rows, record)
        assert (block[:, 0] == torch.arange(rows, dtype=torch.uint8)).all()
        assert (block[:, 1:] == s + 1).all()
    # row split: contiguous blocks, every row exactly once
    total = 13
    lo, hi = rank * total // world, (rank + 1) * total // world
    seen = torch.zeros(total, dtype=torch.int32); seen[lo:hi] += 1
    dist.all_reduce(seen)
    assert (seen == 1).all()
    begin, cols = shard_bounds(1000, world, rank)
    width = torch.tensor([cols]); dist.all_reduce(width)
    assert int(width) == 1000
    # the second collective: every rank's block of results (tokens | log-probs | status), all-gathered,
    # read back through the views ShardedSampler hands out
    from pulsatrix_b200.sharded import row_bounds
    rows = 7
    row_begin, count, per = row_bounds(rows, world, rank)
    block = torch.zeros(16 * per, dtype=torch.uint8)
    block[: 8 * per].view(torch.int64)[:count] = torch.arange(row_begin, row_begin + count) * 10
    block[8 * per: 12 * per].view(torch.float32)[:count] = -torch.arange(row_begin, row_begin + count).float()
    block[12 * per:].view(torch.int32)[:count] = 5
    results = torch.zeros(world * 16 * per, dtype=torch.uint8)
    dist.all_gather_into_tensor(results, block)
    by_rank = results.view(world, 16 * per)
    tokens = by_rank[:, : 8 * per].view(torch.int64).reshape(-1)[:rows]
    logp = by_rank[:, 8 * per: 12 * per].view(torch.float32).reshape(-1)[:rows]
    status = by_rank[:, 12 * per:].view(torch.int32).reshape(-1)[:rows]
    assert tokens.tolist() == [10 * r for r in range(rows)]
    assert logp.tolist() == [-float(r) for r in range(rows)] and (status == 5).all()
    dist.destroy_process_group()
    print("ok", rank)
""")


def test_two_gloo_ranks_gather_records_shard_major(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    proc = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                           "--master-addr", "127.0.0.1", "--master-port", "29671", str(script), str(ROOT)],
                          capture_output=True, text=True, timeout=240, env=env)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    assert proc.stdout.count("ok") == 2


SETUP_WORKER = textwrap.dedent("""
    import os, sys
    import torch, torch.distributed as dist
    sys.path.insert(0, sys.argv[1])
    from pulsatrix_b200.binding import PsxError
    from pulsatrix_b200.sharded import ShardedSampler
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()

    class FakeExchange:  # what Context.exchange() returns, without a GPU
        def __init__(self, rank, fail_open):
            self.handle, self.fail_open, self.opened, self.closed = bytes([rank + 1]) * 64, fail_open, None, False
        def open(self, handles):
            if self.fail_open:
                raise PsxError(2, "cannot map a peer")
            self.opened = handles
        def results(self, device):
            return {"tokens": torch.zeros((world, 1), dtype=torch.int64)}
        def close(self):
            self.closed = True

    class FakeContext:
        def __init__(self, fail_create=False, fail_open=False):
            self.fail_create, self.fail_open, self.made = fail_create, fail_open, None
        def shard_record_bytes(self, config):
            return 48 + 8 * 64
        def exchange(self, world, rank, rows, config):
            if self.fail_create:
                raise PsxError(2, "no memory for the exchange buffer")
            self.made = FakeExchange(rank, self.fail_open)
            return self.made

    cpu = torch.device("cpu")
    # every rank succeeds: each has been given all handles, in rank order
    ctx = FakeContext()
    s = ShardedSampler(ctx, 5, 1000, None, cpu, exchange="peer")
    assert s.exchange == "peer" and s.peer is ctx.made
    assert ctx.made.opened == b"".join(bytes([r + 1]) * 64 for r in range(world))
    # one rank cannot make its buffer, another cannot map a peer's: every rank falls back, none keeps a half-open exchange
    for kind in ("create", "open"):
        ctx = FakeContext(fail_create=(kind == "create" and rank == 1), fail_open=(kind == "open" and rank == 0))
        s = ShardedSampler(ctx, 5, 1000, None, cpu, exchange="peer", fall_back=True)
        assert s.exchange == "nccl" and s.peer is None and s.exchange_note
        assert ctx.made is None or ctx.made.closed
        assert s.gathered.numel() == world * 5 * (48 + 8 * 64)
        # ... or, without fall_back, every rank raises
        ctx = FakeContext(fail_create=(kind == "create" and rank == 1), fail_open=(kind == "open" and rank == 0))
        try:
            ShardedSampler(ctx, 5, 1000, None, cpu, exchange="peer")
            raise SystemExit("should have raised")
        except RuntimeError:
            pass
    dist.barrier()
    dist.destroy_process_group()
    print("ok", rank)
""")


def test_two_gloo_ranks_agree_on_the_peer_exchange_or_fall_back_together(tmp_path):
    script = tmp_path / "setup_worker.py"
    script.write_text(SETUP_WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    proc = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                           "--master-addr", "127.0.0.1", "--master-port", "29673", str(script), str(ROOT)],
                          capture_output=True, text=True, timeout=240, env=env)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    assert proc.stdout.count("ok") == 2
