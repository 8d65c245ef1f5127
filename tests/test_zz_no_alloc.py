"""psx_b200_sample_rows_static: the sampling step for callers that are not allowed to allocate
device memory (a decode loop inside a server whose memory pool already owns the GPU, or a loop that
cannot afford cudaMalloc's device-wide synchronisation).  Its scratch is a fixed array inside the
library, shared by all calls, so the test calls it twice in a row -- the second call finds the
first call's leftovers in the array -- and checks both against the regular entry point on the same
inputs and against the CPU restatement of the reference: token ids equal, log-probs within the 1e-5
relative tolerance of the other GPU tests.
Collected last (the file name sorts after the others), so a failure here cannot hide theirs."""
import numpy as np
import pytest

import gpu_harness as gh
import oracle_lib as ol
import pulsatrix_b200 as psx
import workload_rows
from pulsatrix_b200.workloads import WORKLOADS

pytestmark = pytest.mark.gpu


def _run_both(logits, hist, offsets, cfg, seeds, num_new_tokens=0, shift=0, pad_columns=0, check_oracle=True):
    """(regular entry point's outputs, static entry point's outputs), each (tokens, log-probs, status);
    rows the static one answered are also compared with the CPU restatement of the reference."""
    import torch
    rows, vocab = logits.shape
    stride = vocab + pad_columns
    flat = torch.full((rows * stride + shift + 8,), float("nan"), dtype=torch.float32, device="cuda")
    d_logits = flat[shift: shift + rows * stride].view(rows, stride)[:, :vocab]
    d_logits.copy_(torch.from_numpy(logits))
    d_hist = torch.from_numpy(np.ascontiguousarray(hist).ravel()).cuda()
    d_off = torch.from_numpy(offsets).cuda()
    d_u = torch.from_numpy(psx.uniforms_mt19937_64(seeds)).cuda()
    config = gh.psx_config(cfg, num_new_tokens)
    want = gh.ctx().sample_rows(d_logits, d_hist, d_off, config, d_u, vocab=vocab)
    torch.cuda.synchronize()
    tokens = torch.full((rows,), -7, dtype=torch.int64, device="cuda")
    log_probs = torch.zeros(rows, dtype=torch.float32, device="cuda")
    status = torch.full((rows,), -7, dtype=torch.int32, device="cuda")
    psx.sample_rows_static(d_logits, d_hist, d_off, config, d_u, tokens, log_probs, status, vocab=vocab)
    torch.cuda.synchronize()
    if check_oracle:
        oracle_cfg = cfg
        if num_new_tokens:
            eos = [cfg.eos_token_ids[i] for i in range(cfg.num_eos_token_ids)]
            oracle_cfg = ol.make_config(max_new_tokens=1, do_sample=bool(cfg.do_sample), temperature=cfg.temperature,
                                        top_k=cfg.top_k, top_p=cfg.top_p, min_p=cfg.min_p,
                                        repetition_penalty=cfg.repetition_penalty, eos_token_ids=eos,
                                        min_new_tokens=max(0, cfg.min_new_tokens - num_new_tokens))
        ref = ol.rows("oracle", logits, np.ascontiguousarray(hist, dtype=np.int64).ravel(), offsets, oracle_cfg, seeds,
                      threads=8)
        ok = status.cpu().numpy() == 0
        assert tokens.cpu().numpy()[ok].tolist() == ref["token"][ok].tolist()
        got_lp = log_probs.cpu().numpy()[ok]
        assert (np.abs(got_lp - ref["log_prob"][ok]) <= 1e-5 * np.abs(ref["log_prob"][ok]) + 1e-9).all()
    return ((want["tokens"].cpu().numpy(), want["log_probs"].cpu().numpy(), want["status"].cpu().numpy()),
            (tokens.cpu().numpy(), log_probs.cpu().numpy(), status.cpu().numpy()))


def test_static_entry_point_matches_the_regular_one_on_two_calls_in_a_row():
    # First call: 48 rows of C2 (480 parts).  Second call: a different, smaller batch with other
    # settings, which reuses the front of the same scratch array while the rest still holds call one.
    w = WORKLOADS["c2"]
    first = workload_rows.build("c2", np.arange(48))
    want, got = _run_both(first[0], first[1], first[2], workload_rows.config_of(w), first[3])
    assert (want[2] == 0).all() and (got[2] == 0).all()
    assert got[0].tolist() == want[0].tolist()
    assert (np.abs(got[1] - want[1]) <= 1e-5 * np.abs(want[1]) + 1e-9).all()

    w3 = WORKLOADS["c3"]
    second = workload_rows.build("c3", np.arange(20))
    want, got = _run_both(second[0], second[1], second[2], workload_rows.config_of(w3), second[3])
    assert (want[2] == 0).all() and (got[2] == 0).all()
    assert got[0].tolist() == want[0].tolist()
    assert (np.abs(got[1] - want[1]) <= 1e-5 * np.abs(want[1]) + 1e-9).all()

    # ... and the first batch once more, now over the second call's leftovers.
    want, got = _run_both(first[0], first[1], first[2], workload_rows.config_of(w), first[3])
    assert got[0].tolist() == want[0].tolist() and (got[2] == 0).all()
    assert (np.abs(got[1] - want[1]) <= 1e-5 * np.abs(want[1]) + 1e-9).all()


def test_static_entry_point_refuses_what_its_scratch_cannot_hold():
    import torch
    rows, vocab = 1025, 64  # 1025 parts: one more than the built-in scratch holds
    logits = torch.zeros((rows, vocab), device="cuda")
    tokens = torch.zeros(rows, dtype=torch.int64, device="cuda")
    log_probs = torch.zeros(rows, dtype=torch.float32, device="cuda")
    status = torch.zeros(rows, dtype=torch.int32, device="cuda")
    with pytest.raises(psx.PsxError) as err:
        psx.sample_rows_static(logits, None, None, psx.SamplingConfig.make(), None, tokens, log_probs, status)
    assert err.value.status == 4 and "1025 parts" in str(err.value) and "1024" in str(err.value)
    with pytest.raises(psx.PsxError) as err:  # settings are checked like everywhere else
        psx.sample_rows_static(logits[:4], None, None, psx.SamplingConfig.make(top_p=0.0), None, tokens, log_probs,
                               status)
    assert err.value.status == 1 and "top_p" in str(err.value)
    # greedy on a small batch, no history needed
    small = torch.randn((4, 3000), device="cuda", generator=torch.Generator(device="cuda").manual_seed(3))
    psx.sample_rows_static(small, None, None, psx.SamplingConfig.make(), None, tokens[:4], log_probs[:4], status[:4])
    torch.cuda.synchronize()
    assert tokens[:4].tolist() == small.argmax(dim=1).tolist() and (status[:4] == 0).all()


def test_static_entry_point_follows_the_regular_plan_on_a_large_top_k():
    # top_k = 200 over a 151,936-wide row needs the larger survivor-stage capacities of the regular plan.
    w = WORKLOADS["c2"]
    rows = workload_rows.build("c2", np.arange(12))
    cfg = ol.make_config(max_new_tokens=1, do_sample=True, temperature=0.9, top_k=200, top_p=0.95,
                         repetition_penalty=w.repetition_penalty)
    want, got = _run_both(rows[0], rows[1], rows[2], cfg, rows[3])
    assert got[2].tolist() == want[2].tolist() and (got[2] == 0).all()
    assert got[0].tolist() == want[0].tolist()


def test_static_entry_point_bans_eos_ids_and_forgets_them_again():
    import torch
    rng = np.random.default_rng(11)
    rows, vocab, hlen = 6, 40003, 40
    logits, hist = ol.synth_rows(np.arange(rows) + 700, vocab, 2.0, 1.0, hlen)
    offsets = np.arange(rows + 1, dtype=np.int64) * hlen
    seeds = np.arange(rows, dtype=np.uint64) + 5
    eos = [int(np.argmax(logits[r])) for r in range(3)] + [vocab + 3, -2]  # the first rows' maxima, two ids outside the row
    banned = ol.make_config(max_new_tokens=4, do_sample=True, temperature=0.8, top_k=30, top_p=0.9, repetition_penalty=1.3,
                            eos_token_ids=eos, min_new_tokens=3)
    # an odd base address and an odd stride: rows start off the 16-byte boundaries
    want, got = _run_both(logits, hist, offsets, banned, seeds, num_new_tokens=1, shift=3, pad_columns=5)
    assert (got[2] == 0).all() and got[0].tolist() == want[0].tolist()
    assert not set(got[0].tolist()) & set(eos)
    # the same rows once the ban is over: the ids left in the built-in array by the call before must not count
    want, got = _run_both(logits, hist, offsets, banned, seeds, num_new_tokens=3, shift=1, pad_columns=2)
    assert (got[2] == 0).all() and got[0].tolist() == want[0].tolist()
    # more banned ids than the built-in array holds
    many = ol.make_config(max_new_tokens=4, do_sample=False, eos_token_ids=list(range(257)), min_new_tokens=2)
    d = torch.from_numpy(logits).cuda()
    out = [torch.zeros(rows, dtype=t, device="cuda") for t in (torch.int64, torch.float32, torch.int32)]
    with pytest.raises(psx.PsxError) as err:
        psx.sample_rows_static(d, None, None, gh.psx_config(many), None, *out)
    assert err.value.status == 4 and "256" in str(err.value)
    del rng


def test_static_entry_point_with_enough_rows_for_the_survivor_stage_by_warps():
    # 300 rows of one part each: the launch goes through the warp-per-row survivor kernel and the block
    # kernel behind it; some rows tie 200 logits at the k-th value, more than a warp's list holds.
    logits, hist = ol.synth_rows(np.arange(300) + 6000, 15001, 2.5, 1.0, 24)
    offsets = np.arange(301, dtype=np.int64) * 24
    seeds = np.arange(300, dtype=np.uint64) + 6000
    rng = np.random.RandomState(9)
    for r in range(0, 300, 37):
        order = np.argsort(-logits[r])
        logits[r, rng.choice(order[30:], 200, replace=False)] = logits[r, order[9]]
    for settings in (dict(do_sample=True, temperature=0.9, top_k=16, top_p=0.9, repetition_penalty=1.1), dict(do_sample=False)):
        cfg = ol.make_config(max_new_tokens=1, **settings)
        want, got = _run_both(logits, hist, offsets, cfg, seeds)
        assert (want[2] == 0).all() and (got[2] == 0).all()
        assert got[0].tolist() == want[0].tolist()
