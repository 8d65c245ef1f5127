"""Vocabulary-sharded sampling across the GPUs of one box: every rank holds a contiguous block of
columns of every row, scans it locally, and one small all-gather of fixed-size per-row records
lets every rank finish the draw.  The only collective is that all-gather (NCCL on GPUs)."""
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


def gathered_layout(rows: int, record_bytes: int, world: int):
    """(offset of shard s, bytes per shard) in the gathered buffer: shard-major, then row."""
    per_shard = rows * record_bytes
    return [s * per_shard for s in range(world)], per_shard


def sample_rows_sharded(ctx, shard_logits, vocab, history_ids, history_offsets, config, uniforms, group=None,
                        out=None):
    """One sampling step over rows whose columns are spread over the ranks of `group`.
    shard_logits: this rank's (rows, shard_cols) cuda float32 block.  Returns the output dict of
    Context.shard_merge; every rank gets the same tokens."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    rows = shard_logits.shape[0]
    begin, cols = shard_bounds(vocab, world, rank)
    if cols != shard_logits.shape[1]:
        raise ValueError(f"rank {rank} should hold {cols} columns, got {shard_logits.shape[1]}")
    record = ctx.shard_record_bytes(config)
    mine = torch.empty(rows * record, dtype=torch.uint8, device=shard_logits.device)
    ctx.shard_scan(shard_logits, begin, vocab, history_ids, history_offsets, config, mine)
    gathered = torch.empty(world * rows * record, dtype=torch.uint8, device=shard_logits.device)
    dist.all_gather_into_tensor(gathered, mine, group=group)
    return ctx.shard_merge(gathered, world, rows, vocab, config, uniforms, out=out)
