"""The bounded device-side wait: a row pass whose copies never complete gives up instead of hanging.

Nothing faults and nothing hangs here: the test hook makes the kernel announce 16 bytes more per
chunk than its copies deliver, so the copies themselves finish and only the barrier stays open; the
wait limit is set to two milliseconds; the kernel returns, every row reports
PSX_ROW_DEVICE_TIMEOUT, and the same context answers the next ordinary call correctly."""
import numpy as np
import pytest

import gpu_harness as gh
import oracle_lib as ol
import pulsatrix_b200 as psx

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_reports_a_timeout_and_the_context_stays_usable():
    import torch
    rows, vocab, hlen = 3, 20011, 16
    logits, hist = ol.synth_rows(np.arange(rows) + 40, vocab, 2.0, 1.1, hlen)
    offsets = np.arange(rows + 1, dtype=np.int64) * hlen
    seeds = np.arange(rows, dtype=np.uint64)
    cfg = ol.make_config(max_new_tokens=1, do_sample=True, temperature=0.8, top_k=10, top_p=0.9, repetition_penalty=1.2)
    uniforms = psx.uniforms_mt19937_64(seeds)
    context = psx.Context(0)
    context.set_wait_limit(2_000_000)
    context.test_short_copy(True)
    tokens, logp, status, _ = gh.sample_on_gpu(logits, hist.ravel(), offsets, cfg, uniforms, context=context)
    assert status.tolist() == [psx.ROW_DEVICE_TIMEOUT] * rows and tokens.tolist() == [-1] * rows
    # the host entry point names the failure
    with pytest.raises(psx.PsxError) as err:
        context.sample_rows_host(logits, hist.ravel(), offsets, gh.psx_config(cfg), uniforms)
    assert err.value.status == psx.ERR_ROW_FAILED and "wait" in str(err.value) and "ran out" in str(err.value)
    # back to normal: same context, same rows
    context.test_short_copy(False)
    context.set_wait_limit(1_000_000_000)
    want = ol.rows("oracle", logits, hist.ravel(), offsets, cfg, seeds)
    tokens, logp, status, _ = gh.sample_on_gpu(logits, hist.ravel(), offsets, cfg, uniforms, context=context)
    assert (status == 0).all() and tokens.tolist() == want["token"].tolist()
    assert np.allclose(logp, want["log_prob"], rtol=1e-5, atol=0)
    assert torch.cuda.is_available()
    context.close()
