"""The five synthetic sampling workloads this library is measured and checked on.

Each is a batch of independent rows: fp32 logits drawn as N(0,1)*sigma plus a Zipf bias
-zeta*log(rank+1) laid over a seeded permutation of the vocabulary, a token history per row
for the repetition penalty, and one set of decoding settings for the batch.  Only parameters
live here; tests build the rows with the CPU checker's generator and the benchmark builds
them on the device.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class Workload:
    name: str
    rows: int
    vocab: int
    sigma: float
    zeta: float
    history: int
    repetition_penalty: float
    temperature: float
    top_k: int
    top_p: float
    do_sample: bool
    min_p: float = 0.0
    shards: int = 1          # > 1: vocabulary split into this many contiguous column shards
    tie_row_fraction: float = 0.0  # share of rows whose maximum is copied to 1-3 other columns
    note: str = ""

    @property
    def logits_bytes(self) -> int:
        """Algorithmic HBM bytes of one batch: every fp32 logit read once."""
        return 4 * self.rows * self.vocab


WORKLOADS = {
    "c1": Workload("c1", rows=1000, vocab=49152, sigma=2.0, zeta=1.2, history=64, repetition_penalty=1.1,
                   temperature=0.8, top_k=50, top_p=0.9, do_sample=True,
                   note="batch 1, 1000 independent steps; step s samples with seed s"),
    "c2": Workload("c2", rows=64, vocab=151936, sigma=3.0, zeta=1.0, history=256, repetition_penalty=1.05,
                   temperature=0.7, top_k=20, top_p=0.8, do_sample=True, note="per-row seeds 0..63"),
    "c3": Workload("c3", rows=256, vocab=128256, sigma=2.5, zeta=1.5, history=512, repetition_penalty=1.2,
                   temperature=1.0, top_k=0, top_p=0.95, do_sample=True, note="full-vocabulary nucleus"),
    "c4": Workload("c4", rows=1024, vocab=49152, sigma=4.0, zeta=0.0, history=1, repetition_penalty=1.0,
                   temperature=1.0, top_k=0, top_p=1.0, do_sample=False, tie_row_fraction=0.01,
                   note="greedy + log-prob; exact ties at the maximum in 1% of rows; 1-token dummy prompt"),
    "c5": Workload("c5", rows=512, vocab=262144, sigma=3.0, zeta=1.3, history=1024, repetition_penalty=1.1,
                   temperature=0.9, top_k=64, top_p=0.9, do_sample=True, shards=8,
                   note="vocabulary in 8 contiguous shards, one per GPU"),
}
