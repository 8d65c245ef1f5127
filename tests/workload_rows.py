"""Builds rows of the five workloads with the CPU checker's generator (test infrastructure)."""
from __future__ import annotations

import numpy as np

import oracle_lib
from pulsatrix_b200.workloads import WORKLOADS, Workload

# Generator seeds: workload i, row r -> GEN_BASE[i] + r.  Sampling seeds are the row numbers.
GEN_BASE = {"c1": 1_000_000, "c2": 2_000_000, "c3": 3_000_000, "c4": 4_000_000, "c5": 5_000_000}


def config_of(w: Workload, max_new_tokens=1):
    return oracle_lib.make_config(max_new_tokens=max_new_tokens, do_sample=w.do_sample, temperature=w.temperature,
                                  top_k=w.top_k, top_p=w.top_p, min_p=w.min_p,
                                  repetition_penalty=w.repetition_penalty)


def tie_rows(w: Workload):
    """Rows of a tie workload that get their maximum copied elsewhere, and how many copies."""
    rng = np.random.RandomState(20240 + w.rows)
    n = max(1, int(round(w.rows * w.tie_row_fraction))) if w.tie_row_fraction > 0 else 0
    chosen = np.sort(rng.choice(w.rows, size=n, replace=False))
    copies = rng.randint(1, 4, size=n)
    return dict(zip(chosen.tolist(), copies.tolist()))


def build(name: str, row_ids=None):
    """(logits[n, vocab] f32, history[n, H] i64, offsets[n+1] i64, sampling seeds[n] u64) for the
    given rows of a workload (all rows when row_ids is None)."""
    w = WORKLOADS[name]
    row_ids = np.arange(w.rows) if row_ids is None else np.asarray(row_ids)
    logits, hist = oracle_lib.synth_rows(GEN_BASE[name] + row_ids, w.vocab, w.sigma, w.zeta, w.history)
    if w.tie_row_fraction > 0:
        ties = tie_rows(w)
        for i, r in enumerate(row_ids.tolist()):
            if r in ties:
                rng = np.random.RandomState(77_000 + r)
                cols = rng.choice(w.vocab, size=ties[r], replace=False)
                logits[i, cols] = logits[i].max()
    offsets = np.arange(len(row_ids) + 1, dtype=np.int64) * w.history
    seeds = row_ids.astype(np.uint64)
    return logits, hist, offsets, seeds


def logits_checksum(logits: np.ndarray) -> int:
    """Order-sensitive checksum of the bit patterns, to notice a drifting generator."""
    bits = np.ascontiguousarray(logits).view(np.uint32).astype(np.uint64).ravel()
    weights = (np.arange(bits.size, dtype=np.uint64) % np.uint64(65521)) + np.uint64(1)
    return int((bits * weights).sum(dtype=np.uint64))
