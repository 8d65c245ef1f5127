"""Helpers shared by the GPU tests: run rows through the C ABI on cuda:0 and through the CPU
checker on the same inputs."""
from __future__ import annotations

import numpy as np

import oracle_lib as ol
import pulsatrix_b200 as psx

_ctx = None


def ctx():
    global _ctx
    if _ctx is None:
        _ctx = psx.Context(0)
    return _ctx


def psx_config(cfg, num_new_tokens=0):
    """A psx_sampling_config with the same settings as a checker config."""
    eos = [cfg.eos_token_ids[i] for i in range(cfg.num_eos_token_ids)]
    return psx.SamplingConfig.make(do_sample=bool(cfg.do_sample), temperature=cfg.temperature, top_k=cfg.top_k,
                                   top_p=cfg.top_p, min_p=cfg.min_p, repetition_penalty=cfg.repetition_penalty,
                                   min_new_tokens=cfg.min_new_tokens, num_new_tokens=num_new_tokens,
                                   eos_token_ids=eos)


def sample_on_gpu(logits, hist_flat, offsets, cfg, uniforms, num_new_tokens=0, pad_columns=0, shift=0, context=None):
    """Device-resident call.  pad_columns widens the row stride, shift offsets the base pointer by
    that many floats, so rows need not start on a 16-byte boundary; context: the shared one if None."""
    import torch
    rows, vocab = logits.shape
    stride = vocab + pad_columns
    flat = torch.full((rows * stride + shift + 8,), float("nan"), dtype=torch.float32, device="cuda")
    view = flat[shift: shift + rows * stride].view(rows, stride)
    view[:, :vocab] = torch.from_numpy(np.ascontiguousarray(logits)).cuda()
    d_hist = torch.from_numpy(np.ascontiguousarray(hist_flat, dtype=np.int64)).cuda() if hist_flat is not None else None
    d_off = torch.from_numpy(np.ascontiguousarray(offsets, dtype=np.int64)).cuda() if offsets is not None else None
    d_u = torch.from_numpy(np.ascontiguousarray(uniforms, dtype=np.float64)).cuda() if uniforms is not None else None
    out = (context or ctx()).sample_rows(view, d_hist, d_off, psx_config(cfg, num_new_tokens), d_u, vocab=vocab)
    torch.cuda.synchronize()
    return (out["tokens"].cpu().numpy(), out["log_probs"].cpu().numpy(), out["status"].cpu().numpy(),
            psx.Context.diag_to_numpy(out["diag"]))


def check_rows_against_oracle(logits, hist, offsets, cfg, seeds, *, expect_ok=True, **gpu_kwargs):
    """Runs the same rows on the GPU and through the CPU restatement; tokens must be equal and
    log-probs within 1e-5 relative.  Returns (gpu outputs, oracle infos)."""
    uniforms = psx.uniforms_mt19937_64(seeds)
    hist_flat = np.ascontiguousarray(hist, dtype=np.int64).ravel()
    tokens, logp, status, diag = sample_on_gpu(logits, hist_flat, offsets, cfg, uniforms, **gpu_kwargs)
    # The checker's rows are step 0 of Generate(); a later step only changes whether the EOS ban
    # still holds (src/generation.cpp:69), which min_new_tokens - num_new_tokens expresses.
    oracle_cfg = cfg
    if gpu_kwargs.get("num_new_tokens", 0):
        eos = [cfg.eos_token_ids[i] for i in range(cfg.num_eos_token_ids)]
        oracle_cfg = ol.make_config(max_new_tokens=1, do_sample=bool(cfg.do_sample), temperature=cfg.temperature,
                                    top_k=cfg.top_k, top_p=cfg.top_p, min_p=cfg.min_p,
                                    repetition_penalty=cfg.repetition_penalty, eos_token_ids=eos,
                                    min_new_tokens=max(0, cfg.min_new_tokens - gpu_kwargs["num_new_tokens"]))
    want = ol.rows("oracle", logits, hist_flat, offsets, oracle_cfg, seeds, threads=8)
    if expect_ok:
        assert (status == 0).all(), f"row status {status[status != 0][:8]} at rows {np.nonzero(status)[0][:8]}"
    ok = status == 0
    decided = status != psx.ROW_TOO_WIDE
    assert (status[decided] == want["status"][decided]).all(), (status, want["status"])
    bad = np.nonzero(tokens[ok] != want["token"][ok])[0]
    assert bad.size == 0, (f"token mismatch at rows {np.nonzero(ok)[0][bad][:8]}: gpu {tokens[ok][bad][:8]} "
                           f"oracle {want['token'][ok][bad][:8]} draw margins {want['draw_margin'][ok][bad][:8]} "
                           f"top-p margins {want['top_p_margin'][ok][bad][:8]}")
    err = np.abs(logp[ok] - want["log_prob"][ok]) - 1e-5 * np.abs(want["log_prob"][ok])
    assert err.size == 0 or err.max() <= 1e-9, f"log-prob error beyond 1e-5 relative by {err.max()}"
    if cfg.do_sample:
        assert (diag["survivors"][ok] == want["survivors"][ok]).all()
    return (tokens, logp, status, diag), want
