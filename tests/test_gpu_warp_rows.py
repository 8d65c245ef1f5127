"""The survivor stage with one warp per row (greedy, and sampling under a top-k of at most 64) and the
hand-over of the rows it leaves to the block-per-row kernel: many ties at the k-th value, ties at the
maximum, every filter at once, EOS bans, penalties on either side of one, a top-k of 64 (the longer
list), batches that do not fill the last CTA.  Everything against the CPU checker: token ids equal,
log-probs within 1e-5 relative, survivor counts equal.  (Launches of fewer than 256 rows stay with the
block-per-row kernel, so the batches here are larger.)"""
import numpy as np
import pytest

import gpu_harness as gh
import oracle_lib as ol
import pulsatrix_b200 as psx

pytestmark = pytest.mark.gpu


def _rows(rows, vocab, seed, sigma=2.5, zeta=1.0, hlen=40):
    logits, hist = ol.synth_rows(np.arange(rows) + seed, vocab, sigma, zeta, hlen)
    return logits, hist, np.arange(rows + 1, dtype=np.int64) * hlen, np.arange(rows, dtype=np.uint64) + seed


@pytest.mark.parametrize("rows", [61, 256, 261])
@pytest.mark.parametrize("settings", [
    dict(do_sample=True, temperature=0.7, top_k=20, top_p=0.8, repetition_penalty=1.05),
    dict(do_sample=True, temperature=1.3, top_k=64, top_p=0.95, min_p=0.02, repetition_penalty=1.2),
    dict(do_sample=True, temperature=0.9, top_k=33, repetition_penalty=0.8),
    dict(do_sample=True, temperature=1.0, top_k=1),
    dict(do_sample=False, repetition_penalty=1.3),
    dict(do_sample=False),
])
def test_short_lists_by_warp(rows, settings):
    logits, hist, offsets, seeds = _rows(rows, 20011, 900 + rows)
    gh.check_rows_against_oracle(logits, hist, offsets, ol.make_config(max_new_tokens=1, **settings), seeds)


def test_rows_with_more_ties_than_a_warps_list_go_to_the_block_kernel():
    # every third row: 300 logits tie at the k-th value (all stay, src/generation.cpp:85); every fifth: 90 tie at the top
    logits, hist, offsets, seeds = _rows(259, 30011, 4242)
    rng = np.random.RandomState(3)
    for r in range(259):
        order = np.argsort(-logits[r])
        if r % 3 == 0:
            level = logits[r, order[12]]
            logits[r, rng.choice(order[40:], 300, replace=False)] = level
        if r % 5 == 0:
            logits[r, rng.choice(order[1:], 90, replace=False)] = logits[r, order[0]]
    for settings in (dict(do_sample=True, temperature=0.8, top_k=20, top_p=0.9, repetition_penalty=1.1),
                     dict(do_sample=True, temperature=1.1, top_k=50, min_p=0.01),
                     dict(do_sample=False, repetition_penalty=1.1)):
        cfg = ol.make_config(max_new_tokens=1, **settings)
        (_, _, status, diag), want = gh.check_rows_against_oracle(logits, hist, offsets, cfg, seeds)
        if settings["do_sample"]:
            assert diag["survivors"].max() > 128  # the block kernel's rows are among them


def test_eos_bans_and_unaligned_rows_by_warp():
    logits, hist, offsets, seeds = _rows(263, 32003, 55)
    eos = [int(np.argmax(logits[r])) for r in range(6)]
    for sample in (True, False):
        cfg = ol.make_config(max_new_tokens=4, do_sample=sample, temperature=0.9, top_k=40, top_p=0.9, repetition_penalty=1.15,
                             eos_token_ids=eos, min_new_tokens=3)
        gh.check_rows_against_oracle(logits, hist, offsets, cfg, seeds, pad_columns=1, shift=3)
        gh.check_rows_against_oracle(logits, hist, offsets, cfg, seeds, num_new_tokens=3)


@pytest.mark.parametrize("seed", range(5000, 5012))
def test_randomised_settings_by_warp(seed):
    """Random vocabularies, scales, ties on a grid, histories with ids out of range, every filter, bans: 256
    rows or more, so the launch goes by warps (and by blocks for what the warps leave)."""
    rng = np.random.RandomState(seed)
    vocab = int(rng.choice([257, 1025, 4097, 16385, 20000, 33000]))
    rows = int(rng.choice([256, 261, 300]))
    logits = (rng.randn(rows, vocab) * float(rng.choice([0.5, 2.0, 4.0, 8.0]))).astype(np.float32)
    zeta = float(rng.choice([0.0, 0.0, 1.0, 1.5]))
    if zeta:
        logits -= (zeta * np.log(rng.permutation(vocab) + 1.0)).astype(np.float32)[None, :]
    mode = rng.rand()
    if mode < 0.25:
        logits = (np.round(logits * 2) / 2).astype(np.float32)   # many exact ties
    elif mode < 0.4:
        logits = (np.round(logits * 8) / 8).astype(np.float32)
    hlen = int(rng.choice([1, 16, 300]))
    hist = rng.randint(-2, vocab + 2, size=(rows, hlen)).astype(np.int64)
    offsets = np.arange(rows + 1, dtype=np.int64) * hlen
    seeds = rng.randint(0, 2**31, size=rows).astype(np.uint64)
    cfg = ol.make_config(max_new_tokens=1, do_sample=bool(rng.rand() < 0.8), temperature=float(rng.choice([0.3, 0.7, 1.0, 1.5])),
                         top_k=int(rng.choice([1, 3, 20, 33, 64])), top_p=float(rng.choice([1.0, 0.99, 0.9, 0.5])),
                         min_p=float(rng.choice([0.0, 0.0, 0.0, 0.05])), repetition_penalty=float(rng.choice([1.0, 1.1, 1.3, 0.9])),
                         min_new_tokens=int(rng.choice([0, 2])), eos_token_ids=rng.randint(0, vocab, size=2))
    (_, _, status, _), _ = gh.check_rows_against_oracle(logits, hist, offsets, cfg, seeds, expect_ok=False)
    assert set(np.unique(status)) <= {psx.ROW_OK, psx.ROW_ALL_REMOVED}  # (every token removed: as the reference says then)
