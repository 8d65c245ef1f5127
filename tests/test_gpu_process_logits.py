"""ProcessLogits on the GPU (psx_b200_process_logits_host) against the reference's own vectors
(tests/generation_test.cpp:66-106, tolerance 1e-5, -infinity exact) and, bit for bit, against the
CPU restatement on random rows and settings."""
import json
from pathlib import Path

import numpy as np
import pytest

import gpu_harness as gh
import oracle_lib as ol
import pulsatrix_b200 as psx
import workload_rows
from pulsatrix_b200.workloads import WORKLOADS

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"
HF = json.loads((GOLDEN / "hf_logit_processing.json").read_text())


def gpu_process(logits, tokens, num_new, cfg):
    rows = np.array(logits, dtype=np.float32, ndmin=2).copy()
    hist = np.asarray(tokens, dtype=np.int64).reshape(rows.shape[0], -1)
    offsets = np.arange(rows.shape[0] + 1, dtype=np.int64) * hist.shape[1]
    status = gh.ctx().process_logits_host(rows, hist.ravel() if hist.size else np.zeros(1, dtype=np.int64), offsets,
                                          gh.psx_config(cfg, num_new))
    return rows, status


@pytest.mark.parametrize("case", HF["cases"], ids=lambda c: c["name"])
def test_logit_processing_matches_hugging_face(case):
    cfg = ol.make_config(**case["config"])
    out, status = gpu_process(HF["logits"], HF["tokens"], case["num_new_tokens"], cfg)
    expected = np.array([-np.inf if v == "ninf" else v for v in case["expected"]], dtype=np.float32)
    inf = np.isinf(expected)
    assert (status == 0).all()
    assert (out[0][inf] == expected[inf]).all()
    assert np.abs(out[0][~inf] - expected[~inf]).max() <= 1e-5


@pytest.mark.parametrize("seed", range(4))
def test_random_rows_match_the_restatement_bit_for_bit(seed):
    rng = np.random.RandomState(900 + seed)
    for _ in range(25):
        vocab = int(rng.choice([1, 2, 17, 129, 1000, 4097, 40000]))
        logits = (rng.randn(vocab) * rng.choice([0.5, 2.0, 6.0])).astype(np.float32)
        if rng.rand() < 0.3:
            logits = (np.round(logits * 2) / 2).astype(np.float32)
        tokens = rng.randint(-2, vocab + 2, size=int(rng.choice([1, 8, 200])))
        big = vocab > 1000
        cfg = ol.make_config(do_sample=bool(rng.rand() < 0.85), temperature=float(rng.choice([0.3, 0.7, 1.0, 1.9])),
                             top_k=int(rng.choice([0, 1, 5, 50] + ([] if big else [vocab, vocab + 3]))),
                             top_p=float(rng.choice([1.0, 0.95, 0.5])), min_p=float(rng.choice([0.0, 0.0, 0.05])),
                             repetition_penalty=float(rng.choice([1.0, 1.2, 0.8])), min_new_tokens=int(rng.choice([0, 3])),
                             eos_token_ids=rng.randint(0, vocab, size=2))
        num_new = int(rng.randint(0, 5))
        rc, want = ol.process_logits("oracle", logits, tokens, num_new, cfg)
        try:
            got, status = gpu_process(logits, tokens, num_new, cfg)
        except psx.PsxError as err:  # only an honest "too wide" on a large, coarse or flat row
            assert big and err.status == 3, (vocab, str(err))
            continue
        assert rc == ol.OK
        assert (got[0] == want).all(), (vocab, np.nonzero(got[0] != want)[0][:8], got[0][got[0] != want][:4], want[got[0] != want][:4])


def test_a_batch_of_large_rows():
    w = WORKLOADS["c2"]
    logits, hist, offsets, seeds = workload_rows.build("c2", np.arange(6))
    cfg = workload_rows.config_of(w)
    rows = logits.copy()
    status = gh.ctx().process_logits_host(rows, hist.ravel(), offsets, gh.psx_config(cfg))
    assert (status == 0).all()
    for r in range(6):
        rc, want = ol.process_logits("oracle", logits[r], hist[r], 0, cfg)
        assert (rows[r] == want).all()
