"""Parity of the CUDA sampling path with the reference, through the C ABI, on a real GPU.

Token ids must equal the reference's bit for bit; log-probs agree within 1e-5 relative (the
tolerance the target states for floating point); survivor counts are equal.  The five workloads
are compared with the committed fixtures that the reference itself produced
(tests/golden/make_golden.py); everything else runs the CPU restatement beside the GPU on the
same seeded inputs.
"""
import math
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


def _rel_ok(got, want, tol=1e-5):
    return np.abs(got - want) <= tol * np.abs(want) + 1e-9


# ---- the five workloads at full size against the reference's own outputs -------------------------

@pytest.mark.parametrize("name", list(WORKLOADS))
def test_workload_matches_the_reference_fixture(name):
    w = WORKLOADS[name]
    gold = np.load(GOLDEN / f"workload_{name}.npz")
    cfg = workload_rows.config_of(w)
    mismatches, boundary = [], []
    for start in range(0, w.rows, 256):
        ids = np.arange(start, min(start + 256, w.rows))
        logits, hist, offsets, seeds = workload_rows.build(name, ids)
        assert [workload_rows.logits_checksum(r) for r in logits[:2]] == gold["checksum"][ids[:2]].tolist()
        uniforms = psx.uniforms_mt19937_64(seeds)
        tokens, logp, status, diag = gh.sample_on_gpu(logits, hist.ravel(), offsets, cfg, uniforms)
        assert (status == 0).all(), f"{name}: status {np.unique(status)} rows {ids[status != 0][:8]}"
        for i in np.nonzero(tokens != gold["token"][ids])[0]:
            near = min(gold["draw_margin"][ids[i]], gold["top_p_margin"][ids[i]]) < 1e-6
            (boundary if near else mismatches).append(int(ids[i]))
        same = tokens == gold["token"][ids]
        assert _rel_ok(logp[same], gold["log_prob"][ids][same]).all()
        if w.do_sample:
            assert (diag["survivors"][same] == gold["survivors"][ids][same]).all()
            assert np.allclose(diag["draw_margin"][same], gold["draw_margin"][ids][same], rtol=1e-3, atol=1e-9)
    # A draw within 1e-6 of a bucket edge is reported, not counted; anything else must be exact.
    print(f"{name}: rows {w.rows}, mismatches {len(mismatches)}, boundary rows {boundary}")
    assert not mismatches, f"{name}: token ids differ from the reference at rows {mismatches[:16]}"


# ---- size-independent properties at full size ---------------------------------------------------------

def test_top_k_one_is_greedy_and_greedy_is_the_first_maximum():
    w = WORKLOADS["c2"]
    logits, hist, offsets, seeds = workload_rows.build("c2", np.arange(16))
    logits[3, [7, 100000, 151935]] = logits[3].max() + 1.0  # exact ties: the lowest column wins
    u = psx.uniforms_mt19937_64(seeds)
    greedy = ol.make_config(max_new_tokens=1)
    t_greedy, lp_greedy, st, _ = gh.sample_on_gpu(logits, hist.ravel(), offsets, greedy, None)
    assert (st == 0).all()
    assert t_greedy.tolist() == logits.argmax(axis=1).tolist() and t_greedy[3] == 7
    k1 = ol.make_config(max_new_tokens=1, do_sample=True, top_k=1, temperature=0.7)
    t_k1, lp_k1, st, diag = gh.sample_on_gpu(logits, hist.ravel(), offsets, k1, u)
    assert (st == 0).all()
    # top_k = 1 keeps every tie at the maximum (row 3 has three); elsewhere it is the argmax.
    keep = np.arange(16) != 3
    assert t_k1[keep].tolist() == t_greedy[keep].tolist()
    assert diag["survivors"][3] == 3 and t_k1[3] in (7, 100000, 151935)
    raw = logits.astype(np.float64)
    lse = np.log(np.exp(raw - raw.max(axis=1, keepdims=True)).sum(axis=1)) + raw.max(axis=1)
    want = raw[np.arange(16), t_greedy] - lse
    assert _rel_ok(lp_greedy, want.astype(np.float32), 2e-6).all()


def test_results_do_not_depend_on_row_alignment_or_stride():
    w = WORKLOADS["c1"]
    logits, hist, offsets, seeds = workload_rows.build("c1", np.arange(8))
    logits = logits[:, :40001]  # odd row length
    hist = hist % 40001
    cfg = workload_rows.config_of(w)
    u = psx.uniforms_mt19937_64(seeds)
    base = gh.sample_on_gpu(logits, hist.ravel(), offsets, cfg, u)
    want = ol.rows("oracle", logits, hist.ravel(), offsets, cfg, seeds)
    assert base[0].tolist() == want["token"].tolist()
    for pad, shift in [(0, 1), (3, 2), (5, 3), (7, 0), (16, 4)]:
        other = gh.sample_on_gpu(logits, hist.ravel(), offsets, cfg, u, pad_columns=pad, shift=shift)
        assert other[0].tolist() == base[0].tolist()
        assert other[1].tobytes() == base[1].tobytes()  # bit-identical log-probs: the reduction order is fixed
        assert (other[2] == 0).all()


def test_repeated_calls_are_bit_identical():
    w = WORKLOADS["c3"]
    logits, hist, offsets, seeds = workload_rows.build("c3", np.arange(12))
    cfg = workload_rows.config_of(w)
    u = psx.uniforms_mt19937_64(seeds)
    first = gh.sample_on_gpu(logits, hist.ravel(), offsets, cfg, u)
    for _ in range(3):
        again = gh.sample_on_gpu(logits, hist.ravel(), offsets, cfg, u)
        assert again[0].tolist() == first[0].tolist() and again[1].tobytes() == first[1].tobytes()


# ---- randomised differential test against the CPU restatement -----------------------------------------

@pytest.mark.parametrize("seed", range(8))
def test_random_rows_and_settings_match_the_oracle(seed):
    rng = np.random.RandomState(500 + seed)
    for _ in range(12):
        vocab = int(rng.choice([1, 2, 3, 5, 17, 64, 127, 129, 1000, 4097, 20000, 70001]))
        rows = int(rng.choice([1, 3, 16]))
        scale = float(rng.choice([0.5, 2.0, 6.0]))
        logits = (rng.randn(rows, vocab) * scale).astype(np.float32)
        if rng.rand() < 0.3:  # coarse values: ties everywhere
            logits = (np.round(logits * 2) / 2).astype(np.float32)
        hlen = int(rng.choice([1, 4, 64, 300]))
        hist = rng.randint(-2, vocab + 2, size=(rows, hlen)).astype(np.int64)
        offsets = np.arange(rows + 1, dtype=np.int64) * hlen
        seeds = rng.randint(0, 2**31, size=rows).astype(np.uint64)
        big = vocab > 1000  # rows of up to 256 float4 vectors are always handled whole
        top_k = int(rng.choice([0, 1, 2, 5, 50, 200] + ([] if big else [vocab, vocab + 3])))
        top_p = float(rng.choice([1.0, 0.95, 0.8, 0.3]))
        min_p = float(rng.choice([0.0, 0.0, 0.02, 0.3]))
        do_sample = bool(rng.rand() < 0.85)
        if big and do_sample and top_k == 0 and top_p == 1.0 and min_p == 0.0:
            top_k = 40  # unfiltered sampling of a large vocabulary has no bounded survivor set
        cfg = ol.make_config(max_new_tokens=1, do_sample=do_sample, temperature=float(rng.choice([0.3, 0.7, 1.0, 1.9])),
                             top_k=top_k, top_p=top_p, min_p=min_p,
                             repetition_penalty=float(rng.choice([1.0, 1.15, 0.85])),
                             min_new_tokens=int(rng.choice([0, 2])), eos_token_ids=rng.randint(0, vocab, size=2))
        (tokens, logp, status, diag), want = gh.check_rows_against_oracle(logits, hist, offsets, cfg, seeds,
                                                                          expect_ok=False)
        # Besides what the reference itself rejects (every token banned), the only acceptable
        # failure is an honest "too wide" on coarse data or flat tails of a large vocabulary.
        assert set(np.unique(status)) <= {psx.ROW_OK, psx.ROW_ALL_REMOVED, psx.ROW_TOO_WIDE}, np.unique(status)
        if not big:
            assert (status == want["status"]).all(), (vocab, rows, top_k, top_p, min_p, status)


def test_hugging_face_vectors_decide_the_same_survivors():
    # tests/generation_test.cpp:27-106: 12 logits, history [3, 5, 5, 9]; the surviving sets of the
    # sampled cases must be the finite entries of the stored vectors.
    import json
    hf = json.loads((GOLDEN / "hf_logit_processing.json").read_text())
    logits = np.array(hf["logits"], dtype=np.float32)[None, :]
    hist = np.array([hf["tokens"]], dtype=np.int64)
    offsets = np.array([0, 4], dtype=np.int64)
    for case in hf["cases"]:
        cfg = ol.make_config(max_new_tokens=1, **case["config"])
        alive = {i for i, v in enumerate(case["expected"]) if v != "ninf"}
        seen = set()
        seeds = np.arange(400, dtype=np.uint64)
        many = np.repeat(logits, 400, axis=0)
        hist_many = np.repeat(hist, 400, axis=0)
        off_many = np.arange(401, dtype=np.int64) * 4
        (tokens, _, status, diag), _ = gh.check_rows_against_oracle(many, hist_many, off_many, cfg, seeds,
                                                                    num_new_tokens=case["num_new_tokens"])
        seen.update(tokens.tolist())
        if cfg.do_sample:
            assert seen <= alive and (diag["survivors"] == len(alive)).all()
            if len(alive) <= 4:
                assert seen == alive
        else:
            assert seen == {int(np.argmax([-math.inf if v == "ninf" else v for v in case["expected"]]))}


# ---- error statuses (tests/generation_test.cpp:224-245) -------------------------------------------------

def test_bad_rows_and_bad_settings_are_reported_like_the_reference():
    import torch
    rows, vocab = 4, 3000
    rng = np.random.RandomState(3)
    logits = rng.randn(rows, vocab).astype(np.float32)
    logits[1, 17] = np.nan
    logits[2, 2999] = np.inf
    logits[3, 0] = -np.inf
    hist = np.zeros((rows, 1), dtype=np.int64)
    offsets = np.arange(rows + 1, dtype=np.int64)
    u = np.full(rows, 0.5)
    for cfg in (ol.make_config(), ol.make_config(do_sample=True, top_k=10)):
        tokens, _, status, _ = gh.sample_on_gpu(logits, hist.ravel(), offsets, cfg, u)
        assert status.tolist() == [psx.ROW_OK, psx.ROW_NON_FINITE, psx.ROW_NON_FINITE, psx.ROW_NON_FINITE]
        assert tokens[0] >= 0 and (tokens[1:] == -1).all()
    # every token banned: EOS covers the vocabulary and min_new_tokens holds it off
    small = np.zeros((1, 5), dtype=np.float32)
    banned = ol.make_config(min_new_tokens=1, eos_token_ids=[0, 1, 2, 3, 4])
    _, _, status, _ = gh.sample_on_gpu(small, np.zeros(1, dtype=np.int64), np.array([0, 1]), banned, np.array([0.5]))
    assert status.tolist() == [psx.ROW_ALL_REMOVED]
    # invalid settings are rejected before anything is launched, with the reference's wording
    d = torch.zeros((1, 5), device="cuda")
    out = gh.ctx().alloc_outputs(1)
    for kw, text in [(dict(temperature=0.0), "temperature"), (dict(top_p=0.0), "top_p"), (dict(top_k=-1), "top_k"),
                     (dict(min_p=2.0), "min_p"), (dict(repetition_penalty=0.0), "repetition_penalty")]:
        with pytest.raises(psx.PsxError) as err:
            gh.ctx().sample_rows(d, None, None, psx.SamplingConfig.make(**kw), None, out=out)
        assert err.value.status == 1 and text in str(err.value)
    with pytest.raises(psx.PsxError):  # the host entry reports a failed row as an error
        gh.ctx().sample_rows_host(logits, hist.ravel(), offsets, psx.SamplingConfig.make(), u)


def test_host_entry_point_gives_the_same_answers():
    w = WORKLOADS["c2"]
    logits, hist, offsets, seeds = workload_rows.build("c2", np.arange(8))
    cfg = workload_rows.config_of(w)
    u = psx.uniforms_mt19937_64(seeds)
    dev = gh.sample_on_gpu(logits, hist.ravel(), offsets, cfg, u)
    wide = np.zeros((8, w.vocab + 5), dtype=np.float32)
    wide[:, :w.vocab] = logits
    for arr, stride in [(logits, None), (wide, w.vocab + 5)]:
        tokens, logp, status, diag = gh.ctx().sample_rows_host(arr, hist.ravel(), offsets, gh.psx_config(cfg), u,
                                                               row_stride=stride, vocab=w.vocab)
        assert tokens.tolist() == dev[0].tolist() and logp.tobytes() == dev[1].tobytes() and (status == 0).all()


# ---- the rarely taken paths of the survivor stage ---------------------------------------------------

def test_long_histories_overflow_the_speculative_slots_and_still_match():
    """A part whose list is several times longer than what the survivor stage fetches before it
    knows the counts (hundreds of penalised tokens with a small top-k): the rest of the list is
    appended afterwards."""
    rng = np.random.RandomState(77)
    vocab, rows, hlen = 30000, 6, 700
    logits = (rng.randn(rows, vocab) * 3.0).astype(np.float32)
    hist = np.stack([rng.choice(vocab, size=hlen, replace=False) for _ in range(rows)]).astype(np.int64)
    offsets = np.arange(rows + 1, dtype=np.int64) * hlen
    seeds = np.arange(rows, dtype=np.uint64) + 11
    for top_k, top_p in [(5, 0.9), (1, 1.0), (40, 0.5)]:
        cfg = ol.make_config(max_new_tokens=1, do_sample=True, temperature=0.8, top_k=top_k, top_p=top_p,
                             repetition_penalty=1.3)
        (tokens, logp, status, diag), want = gh.check_rows_against_oracle(logits, hist, offsets, cfg, seeds)
        assert (status == 0).all()
        assert (diag["survivors"] == want["survivors"]).all()


def test_hundreds_of_ties_at_the_kth_value_take_the_sorted_path():
    """HF semantics keep every tie at the k-th value (src/generation.cpp:85): 150 distinct large
    logits and 400 logits equal to the 150th leave 549 survivors, more than the
    one-entry-per-thread path holds."""
    rng = np.random.RandomState(78)
    vocab, rows = 20000, 4
    logits = (rng.randn(rows, vocab) - 6.0).astype(np.float32)
    for r in range(rows):
        cols = rng.choice(vocab, size=549, replace=False)
        logits[r, cols[:149]] = np.linspace(5.0, 9.0, 149).astype(np.float32) + np.float32(r) * 0.01
        logits[r, cols[149:]] = np.float32(4.0)
    hist = rng.randint(0, vocab, size=(rows, 32)).astype(np.int64)
    offsets = np.arange(rows + 1, dtype=np.int64) * 32
    seeds = np.arange(rows, dtype=np.uint64) + 5
    for top_p, penalty in [(0.9, 1.0), (1.0, 1.0), (0.6, 1.1)]:
        cfg = ol.make_config(max_new_tokens=1, do_sample=True, temperature=1.3, top_k=150, top_p=top_p,
                             repetition_penalty=penalty)
        (tokens, logp, status, diag), want = gh.check_rows_against_oracle(logits, hist, offsets, cfg, seeds)
        assert (status == 0).all()
        assert (diag["survivors"] == want["survivors"]).all()
        if penalty == 1.0 and top_p == 1.0:
            assert (diag["survivors"] == 549).all()


def test_the_promise_of_complete_inputs_changes_no_answer():
    """With psx_b200_ctx_inputs_are_ready a row pass runs ahead of the survivor stage of the call
    before it: three different batches enqueued back to back give what they give one at a time."""
    import torch
    w = WORKLOADS["c2"]
    cfg = gh.psx_config(workload_rows.config_of(w))
    batches = []
    for b in range(3):
        logits, hist, offsets, seeds = workload_rows.build("c2", np.arange(16 * b, 16 * b + 16))
        batches.append((torch.from_numpy(logits).cuda(), torch.from_numpy(hist.ravel().astype(np.int64)).cuda(),
                        torch.from_numpy(offsets.astype(np.int64)).cuda(),
                        torch.from_numpy(psx.uniforms_mt19937_64(seeds)).cuda()))
    context = gh.ctx()
    alone = []
    for logits, hist, offsets, u in batches:
        out = context.sample_rows(logits, hist, offsets, cfg, u)
        torch.cuda.synchronize()
        alone.append((out["tokens"].cpu().numpy(), out["log_probs"].cpu().numpy()))
    context.inputs_are_ready(True)
    try:
        for _ in range(3):
            outs = [context.sample_rows(logits, hist, offsets, cfg, u) for logits, hist, offsets, u in batches]
            torch.cuda.synchronize()
            for out, (tokens, logp) in zip(outs, alone):
                assert out["status"].cpu().numpy().tolist() == [0] * 16
                assert out["tokens"].cpu().numpy().tolist() == tokens.tolist()
                assert out["log_probs"].cpu().numpy().tobytes() == logp.tobytes()
    finally:
        context.inputs_are_ready(False)


def test_contexts_in_flight_on_their_own_streams_change_no_answer():
    """Three contexts, each with its own stream, scratch and outputs, fed round-robin the way the
    benchmark feeds them: the row pass of one batch overlaps the survivor stage of another, and every
    batch gets what it gets alone (checked against the restatement too)."""
    import torch
    w = WORKLOADS["c2"]
    config = workload_rows.config_of(w)
    cfg = gh.psx_config(config)
    batches, expected = [], []
    for b in range(6):
        logits, hist, offsets, seeds = workload_rows.build("c2", np.arange(8 * b, 8 * b + 8))
        expected.append(ol.rows("oracle", logits, hist.ravel(), offsets, config, seeds))
        batches.append((torch.from_numpy(logits).cuda(), torch.from_numpy(hist.ravel().astype(np.int64)).cuda(),
                        torch.from_numpy(offsets.astype(np.int64)).cuda(),
                        torch.from_numpy(psx.uniforms_mt19937_64(seeds)).cuda()))
    torch.cuda.synchronize()
    contexts = [psx.Context(0) for _ in range(3)]
    streams = [torch.cuda.Stream() for _ in contexts]
    try:
        for c in contexts:
            c.inputs_are_ready(True)
        for _ in range(3):
            outs = []
            for i, (logits, hist, offsets, u) in enumerate(batches):
                c = i % len(contexts)
                outs.append(contexts[c].sample_rows(logits, hist, offsets, cfg, u, stream=streams[c].cuda_stream))
            torch.cuda.synchronize()
            for out, want in zip(outs, expected):
                assert out["status"].cpu().numpy().tolist() == [0] * 8
                assert out["tokens"].cpu().numpy().tolist() == want["token"].tolist()
                np.testing.assert_allclose(out["log_probs"].cpu().numpy(), want["log_prob"], rtol=1e-5)
    finally:
        for c in contexts:
            c.close()


def test_contexts_with_different_plans_do_not_lower_each_others_limits():
    """A full-vocabulary top-p (large survivor-stage shared memory) in one context, a small top-k in a
    context created after it, then the first again: the kernels' limits belong to the process."""
    w = WORKLOADS["c3"]
    logits, hist, offsets, seeds = workload_rows.build("c3", np.arange(6))
    wide = workload_rows.config_of(w)
    narrow = ol.make_config(max_new_tokens=1, do_sample=True, top_k=5, temperature=0.9)
    u = psx.uniforms_mt19937_64(seeds)
    first, second = psx.Context(0), None
    try:
        a = gh.sample_on_gpu(logits, hist.ravel(), offsets, wide, u, context=first)
        second = psx.Context(0)
        b = gh.sample_on_gpu(logits, hist.ravel(), offsets, narrow, u, context=second)
        again = gh.sample_on_gpu(logits, hist.ravel(), offsets, wide, u, context=first)
    finally:
        first.close()
        if second is not None:
            second.close()
    assert a[0].tolist() == ol.rows("oracle", logits, hist.ravel(), offsets, wide, seeds)["token"].tolist()
    assert b[0].tolist() == ol.rows("oracle", logits, hist.ravel(), offsets, narrow, seeds)["token"].tolist()
    assert again[0].tolist() == a[0].tolist() and again[1].tobytes() == a[1].tobytes()


def test_a_prepared_call_enqueues_the_same_call_again():
    """Context.bind_sample_rows converts the arguments once; calling the result twice gives what
    sample_rows gives, and new contents of the same buffers are seen by the next call."""
    import torch
    w = WORKLOADS["c1"]
    cfg = workload_rows.config_of(w)
    logits, hist, offsets, seeds = workload_rows.build("c1", np.arange(10))
    other = workload_rows.build("c1", np.arange(10, 20))[0]
    d_logits = torch.from_numpy(logits).cuda()
    d_hist = torch.from_numpy(hist.ravel().astype(np.int64)).cuda()
    d_off = torch.from_numpy(offsets.astype(np.int64)).cuda()
    d_u = torch.from_numpy(psx.uniforms_mt19937_64(seeds)).cuda()
    context = gh.ctx()
    config = gh.psx_config(cfg)
    plain = context.sample_rows(d_logits, d_hist, d_off, config, d_u)
    torch.cuda.synchronize()
    want = plain["tokens"].cpu().numpy().tolist()
    call = context.bind_sample_rows(d_logits, d_hist, d_off, config, d_u)
    for _ in range(2):
        out = call()
        torch.cuda.synchronize()
        assert out["tokens"].cpu().numpy().tolist() == want
        assert out["log_probs"].cpu().numpy().tobytes() == plain["log_probs"].cpu().numpy().tobytes()
    d_logits.copy_(torch.from_numpy(other))
    out = call()
    torch.cuda.synchronize()
    expect = ol.rows("oracle", other, hist.ravel(), offsets, cfg, seeds)
    assert out["tokens"].cpu().numpy().tolist() == expect["token"].tolist()
