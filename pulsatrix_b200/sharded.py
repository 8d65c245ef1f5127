"""Vocabulary-sharded sampling across the GPUs of one box: every rank holds a contiguous block of
columns of every row, scans it locally, and one all-gather of fixed-size per-row records brings
every shard's candidates to every rank.  The ranks then share the rows out: a rank finishes the
draw for its own block of rows only, and a second, tiny all-gather (16 bytes per row: token,
log-probability, status) gives every rank every row's result.  Both collectives are plain NCCL
all-gathers into the GPU's own memory; no kernel reads another GPU's memory.

With exchange="peer" there is no library collective in a step: the packing kernel writes each
record straight into the memory of the rank that decides the row, that rank's survivor stage waits
(row by row, bounded) for a counter in its own memory that the writers raise, and a last kernel
writes the rank's results into every rank's memory and waits (bounded) for everyone else's.  The
buffers are opened once through CUDA IPC; their handles travel through one all-gather of the process
group when the sampler is built."""
from __future__ import annotations


def shard_bounds(vocab: int, world: int, rank: int):
    """Columns [begin, begin + cols) of `rank`: contiguous, ascending, multiples of 4 columns so
    that every shard starts on a 16-byte boundary when the rows do; the last takes the rest."""
    if not (0 <= rank < world):
        raise ValueError("rank outside the world")
    per = -(-vocab // world)
    per = -(-per // 4) * 4
    begin = min(rank * per, vocab)
    end = min(begin + per, vocab)
    return begin, end - begin


def row_bounds(rows: int, world: int, rank: int):
    """Rows [begin, begin + count) whose draw `rank` finishes, and the block size every rank's
    results are padded to (the same on every rank, so that the blocks can be all-gathered)."""
    if not (0 <= rank < world):
        raise ValueError("rank outside the world")
    per = -(-rows // world)
    begin = min(rank * per, rows)
    return begin, min(per, rows - begin), per


def gathered_layout(rows: int, record_bytes: int, world: int):
    """(offset of shard s, bytes per shard) in the gathered buffer: shard-major, then row."""
    per_shard = rows * record_bytes
    return [s * per_shard for s in range(world)], per_shard


class ShardedSampler:
    """The buffers of one sharded sampling step, allocated once: this rank's records, the gathered
    records, this rank's block of results and the gathered results.

    step() returns {"tokens", "log_probs", "status"}: tensors of shape (world, rows_per_rank) that
    are views of the gathered results; row r is at [r // rows_per_rank, r % rows_per_rank] (use
    flat() for plain (rows,) copies)."""

    def __init__(self, ctx, rows, vocab, config, device, group=None, exchange="nccl", fall_back=False):
        import torch
        import torch.distributed as dist
        if exchange not in ("nccl", "peer"):
            raise ValueError('exchange is "nccl" or "peer"')
        self.ctx, self.rows, self.vocab, self.config, self.group = ctx, rows, vocab, config, group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.begin_col, self.cols = shard_bounds(vocab, self.world, self.rank)
        self.row_begin, self.row_count, self.per = row_bounds(rows, self.world, self.rank)
        self.record = ctx.shard_record_bytes(config)
        self.mine = torch.empty(rows * self.record, dtype=torch.uint8, device=device)
        self.peer = None
        self.exchange, self.exchange_note = exchange, None
        if exchange == "peer":
            # Every rank goes through the same collectives whether or not its own buffer could be made and
            # its peers' mapped; one rank's failure is every rank's (fall_back: all use the all-gathers instead).
            from .binding import PsxError
            problem = None
            try:
                self.peer = ctx.exchange(self.world, self.rank, rows, config)
                handle = self.peer.handle
            except PsxError as e:
                problem, handle = str(e), bytes(64)
            mine = torch.frombuffer(bytearray(handle), dtype=torch.uint8).to(device)
            everyone = torch.empty(self.world * mine.numel(), dtype=torch.uint8, device=device)
            dist.all_gather_into_tensor(everyone, mine, group=group)
            if problem is None:
                try:
                    self.peer.open(everyone.cpu().numpy().tobytes())
                except PsxError as e:
                    problem = str(e)
            failed = torch.tensor([0 if problem is None else 1], dtype=torch.int32, device=device)
            dist.all_reduce(failed, op=dist.ReduceOp.MAX, group=group)  # (also: every rank has mapped every buffer before anyone writes)
            if int(failed.item()) == 0:
                self.out = self.peer.results(device)
                return
            if self.peer is not None:
                self.peer.close()
                self.peer = None
            if not fall_back:
                raise RuntimeError("the peer-memory exchange could not be set up on every rank" + (f": {problem}" if problem else ""))
            self.exchange, self.exchange_note = "nccl", problem or "another rank could not set up the peer-memory exchange"
        self.gathered = torch.empty(self.world * rows * self.record, dtype=torch.uint8, device=device)
        per = self.per
        # a rank's block: tokens (int64 x per) | log-probs (float32 x per) | status (int32 x per)
        self.block = torch.zeros(16 * per, dtype=torch.uint8, device=device)
        self.results = torch.zeros(self.world * 16 * per, dtype=torch.uint8, device=device)
        self.block_out = {"tokens": self.block[: 8 * per].view(torch.int64),
                          "log_probs": self.block[8 * per: 12 * per].view(torch.float32),
                          "status": self.block[12 * per:].view(torch.int32), "diag": None}
        by_rank = self.results.view(self.world, 16 * per)
        self.out = {"tokens": by_rank[:, : 8 * per].view(torch.int64),
                    "log_probs": by_rank[:, 8 * per: 12 * per].view(torch.float32),
                    "status": by_rank[:, 12 * per:].view(torch.int32)}

    @property
    def allgather_bytes(self):
        """Bytes this rank contributes to the two exchanges of a step (all-gathers, or peer stores)."""
        return self.rows * self.record, 16 * self.per

    def step(self, shard_logits, history_ids, history_offsets, uniforms):
        import torch.distributed as dist
        if shard_logits.shape != (self.rows, self.cols):
            raise ValueError(f"rank {self.rank} should hold a {self.rows} x {self.cols} block, got {tuple(shard_logits.shape)}")
        if self.peer is not None:
            self.out = self.peer.sample(shard_logits, self.begin_col, self.vocab, history_ids, history_offsets, self.config,
                                        uniforms)
            return self.out
        self.ctx.shard_scan(shard_logits, self.begin_col, self.vocab, history_ids, history_offsets, self.config, self.mine)
        dist.all_gather_into_tensor(self.gathered, self.mine, group=self.group)
        if self.row_count > 0:
            self.ctx.shard_merge(self.gathered, self.world, self.rows, self.vocab, self.config, uniforms, out=self.block_out,
                                 row_begin=self.row_begin, row_count=self.row_count)
        dist.all_gather_into_tensor(self.results, self.block, group=self.group)
        return self.out

    def close(self):
        """Frees the peer-memory exchange (after a barrier: no rank may still be inside a step)."""
        if self.peer is not None:
            import torch
            import torch.distributed as dist
            torch.cuda.synchronize()
            dist.barrier(group=self.group)
            self.peer.close()
            self.peer = None

    def flat(self, out=None):
        """(rows,) copies of the results, in row order."""
        out = out or self.out
        return {k: v.reshape(-1)[: self.rows] for k, v in out.items()}


def sample_rows_sharded(ctx, shard_logits, vocab, history_ids, history_offsets, config, uniforms, group=None,
                        out=None):
    """One sampling step over rows whose columns are spread over the ranks of `group`, with
    buffers allocated for this one call (a loop keeps a ShardedSampler instead).  shard_logits:
    this rank's (rows, shard_cols) cuda float32 block.  Returns {"tokens", "log_probs", "status"}
    as (rows,) tensors; every rank gets the same."""
    del out
    sampler = ShardedSampler(ctx, shard_logits.shape[0], vocab, config, shard_logits.device, group)
    sampler.step(shard_logits, history_ids, history_offsets, uniforms)
    return sampler.flat()
