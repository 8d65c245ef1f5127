"""Rows the candidate lists cannot decide -- sampling with no filter at all, a nucleus wider than
the lists, a top-k beyond what a part can bound, thousands of exact ties -- are decided from the
row itself (general_row) and must come out as the reference's: no PSX_ROW_TOO_WIDE, token ids equal
(a row whose decision lies within 1e-6 of a boundary is reported, not counted), log-probs within
1e-5 relative, survivor counts equal.  The same for ProcessLogits, bit for bit."""
import numpy as np
import pytest

import gpu_harness as gh
import oracle_lib as ol
import pulsatrix_b200 as psx

pytestmark = pytest.mark.gpu

VOCAB = 70001
SETTINGS = {
    "no filter": dict(do_sample=True, temperature=1.3, repetition_penalty=1.2),
    "no filter, no penalty": dict(do_sample=True, temperature=1.0),
    "top_p 0.99 at T=2": dict(do_sample=True, temperature=2.0, top_p=0.99, repetition_penalty=1.1),
    "top_k 1000": dict(do_sample=True, temperature=0.9, top_k=1000, top_p=0.95, repetition_penalty=1.1),
    "top_k 300 + min_p": dict(do_sample=True, temperature=1.5, top_k=300, min_p=0.001),
    "min_p alone, flat": dict(do_sample=True, temperature=3.0, min_p=0.0005, repetition_penalty=0.9),
}


def _rows(rows, vocab, seed, sigma=2.0, zeta=1.0, hlen=48):
    logits, hist = ol.synth_rows(np.arange(rows) + seed, vocab, sigma, zeta, hlen)
    return logits, hist, np.arange(rows + 1, dtype=np.int64) * hlen, np.arange(rows, dtype=np.uint64) + seed


def _check(logits, hist, offsets, seeds, cfg, **kw):
    u = psx.uniforms_mt19937_64(seeds)
    tokens, logp, status, diag = gh.sample_on_gpu(logits, hist.ravel(), offsets, cfg, u, **kw)
    want = ol.rows("oracle", logits, hist.ravel(), offsets, cfg, seeds, threads=8)
    assert (status == 0).all(), f"status {np.unique(status)} at rows {np.nonzero(status)[0][:8]}"
    near = np.minimum(want["draw_margin"], want["top_p_margin"]) < 1e-6
    differ = tokens != want["token"]
    assert not (differ & ~near).any(), (np.nonzero(differ & ~near)[0][:8], tokens[differ][:8], want["token"][differ][:8])
    same = ~differ
    assert (np.abs(logp[same] - want["log_prob"][same]) <= 1e-5 * np.abs(want["log_prob"][same]) + 1e-9).all()
    if cfg.do_sample:
        assert (diag["survivors"][same] == want["survivors"][same]).all()
    return int(differ.sum())


@pytest.mark.parametrize("name", list(SETTINGS))
def test_wide_rows_are_answered_like_the_reference(name):
    logits, hist, offsets, seeds = _rows(24, VOCAB, 31_000)
    cfg = ol.make_config(max_new_tokens=1, **SETTINGS[name])
    boundary = _check(logits, hist, offsets, seeds, cfg)
    print(f"{name}: rows within 1e-6 of a boundary that differ: {boundary}")


def test_unaligned_rows_and_eos_bans_on_the_general_path():
    logits, hist, offsets, seeds = _rows(9, 40003, 77)
    eos = [int(np.argmax(logits[r])) for r in range(4)]
    cfg = ol.make_config(max_new_tokens=4, do_sample=True, temperature=1.1, repetition_penalty=1.3, eos_token_ids=eos,
                         min_new_tokens=2)
    _check(logits, hist, offsets, seeds, cfg, pad_columns=3, shift=1)


def test_all_equal_logits_keep_every_tie():
    # every logit ties with the k-th largest, so the top-k keeps the whole vocabulary (src/generation.cpp:85)
    rows, vocab = 6, 50000
    logits = np.zeros((rows, vocab), dtype=np.float32)
    logits[3:] = np.round(np.random.RandomState(1).randn(3, vocab)).astype(np.float32)  # a handful of values: long ties
    hist = np.zeros((rows, 1), dtype=np.int64)
    offsets = np.arange(rows + 1, dtype=np.int64)
    seeds = np.arange(rows, dtype=np.uint64) + 3
    for settings in (dict(do_sample=True, top_k=50), dict(do_sample=True, top_k=50, top_p=0.7), dict(do_sample=False)):
        _check(logits, hist, offsets, seeds, ol.make_config(max_new_tokens=1, **settings))


@pytest.mark.parametrize("name", ["top_p 0.99 at T=2", "top_k 1000", "top_k 300 + min_p"])
def test_process_logits_on_wide_rows_is_bit_exact(name):
    logits, hist, offsets, _ = _rows(5, 30011, 900)
    cfg = ol.make_config(max_new_tokens=1, **SETTINGS[name])
    got = logits.copy()
    status = gh.ctx().process_logits_host(got, hist.ravel(), offsets, gh.psx_config(cfg))
    assert (status == 0).all()
    for r in range(logits.shape[0]):
        rc, want = ol.process_logits("oracle", logits[r], hist[r], 0, cfg)
        assert rc == 0
        differ = np.nonzero(got[r].view(np.uint32) != want.view(np.uint32))[0]
        assert differ.size == 0, (name, r, differ[:8], got[r][differ[:8]], want[differ[:8]])
