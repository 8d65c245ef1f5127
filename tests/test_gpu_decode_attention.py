"""Attention of the new positions over the KV cache (psx_b200_decode_attention) against the CPU restatement
of MultiHeadAttentionModule::forward_cached's core (src/multihead_attention_module.cpp:562-586), which
tests/test_oracle_pins.py pins to the compiled reference: within the reference's own CPU/GPU equivalence
tolerance, 1e-4 (tests/backend_primitive_equivalence_cases.hpp:22).  Grouped-query heads, several new
positions, causal masks with a cache offset, sliding windows, key padding, fully masked rows, caches of one
position and of thousands (several slices per head)."""
import numpy as np
import pytest

import gpu_harness as gh
import oracle_lib as ol
import pulsatrix_b200 as psx

pytestmark = pytest.mark.gpu
TOLERANCE = 1e-4


def _case(batch, heads, kv_heads, q_len, d, cached, max_len, seed, causal=True, window=0, padding=False, scale=None):
    import torch
    rng = np.random.RandomState(seed)
    q = rng.randn(batch, heads, q_len, d).astype(np.float32)
    keys = rng.randn(batch, kv_heads, max_len, d).astype(np.float32)
    values = rng.randn(batch, kv_heads, max_len, d).astype(np.float32)
    total = cached + q_len
    keys[:, :, total:] = np.nan   # what lies beyond the cached positions must never be read into a result
    values[:, :, total:] = np.nan
    keep = None
    if padding:
        keep = (rng.rand(batch, total) > 0.3).astype(np.float32)
        keep[0, :] = 0.0          # a fully masked batch entry: uniform attention, as the reference gives
    scale = float(1.0 / np.sqrt(np.float32(d))) if scale is None else scale
    want = ol.decode_attention("oracle", q, np.nan_to_num(keys), np.nan_to_num(values), cached, scale, causal, window, keep)
    got, status = gh.ctx().decode_attention(torch.from_numpy(q).cuda(), torch.from_numpy(keys).cuda(), torch.from_numpy(values).cuda(),
                                            cached, scale=scale, causal=causal, window=window,
                                            key_keep=None if keep is None else torch.from_numpy(keep).cuda())
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    got = got.cpu().numpy()
    assert np.isfinite(got).all()
    err = np.abs(got - want) / np.maximum(1.0, np.abs(want))
    assert err.max() <= TOLERANCE, (err.max(), np.unravel_index(err.argmax(), err.shape))


@pytest.mark.parametrize("cached", [0, 1, 31, 32, 33, 127, 1000, 4097])
def test_one_new_position_over_caches_of_every_length(cached):
    _case(batch=3, heads=8, kv_heads=2, q_len=1, d=64, cached=cached, max_len=cached + 5, seed=cached)


@pytest.mark.parametrize("heads,kv_heads,q_len,d", [(4, 4, 1, 128), (8, 1, 1, 64), (16, 2, 1, 128), (6, 3, 2, 32), (4, 2, 4, 96),
                                                    (2, 2, 8, 4), (12, 12, 3, 80), (4, 2, 1, 256), (8, 8, 1, 160), (2, 1, 2, 192), (8, 1, 1, 256)])
def test_head_layouts_and_several_new_positions(heads, kv_heads, q_len, d):
    _case(batch=2, heads=heads, kv_heads=kv_heads, q_len=q_len, d=d, cached=300, max_len=512, seed=heads * 100 + d)


def test_masks():
    _case(batch=2, heads=4, kv_heads=2, q_len=2, d=64, cached=500, max_len=600, seed=1, causal=True, window=64)
    _case(batch=3, heads=4, kv_heads=4, q_len=1, d=64, cached=200, max_len=256, seed=2, causal=True, padding=True)
    _case(batch=2, heads=4, kv_heads=1, q_len=2, d=32, cached=90, max_len=128, seed=3, causal=False)
    _case(batch=2, heads=2, kv_heads=2, q_len=3, d=64, cached=40, max_len=64, seed=4, causal=False, padding=True, scale=0.3)


def test_many_slices_and_many_heads():
    _case(batch=1, heads=8, kv_heads=8, q_len=1, d=128, cached=20000, max_len=20001, seed=5)    # few heads, long cache: slices
    _case(batch=40, heads=16, kv_heads=8, q_len=1, d=128, cached=700, max_len=768, seed=6)      # many heads: one slice each


def test_bad_arguments_are_refused():
    import torch
    ctx = gh.ctx()
    q = torch.zeros((1, 6, 1, 64), device="cuda")
    kv = torch.zeros((1, 4, 16, 64), device="cuda")
    with pytest.raises(psx.PsxError):   # heads not a multiple of kv_heads
        ctx.decode_attention(q, kv, kv, 3)
    q = torch.zeros((1, 4, 1, 64), device="cuda")
    with pytest.raises(psx.PsxError):   # the cache is full
        ctx.decode_attention(q, kv, kv, 16)
    q = torch.zeros((1, 16, 4, 64), device="cuda")
    kv = torch.zeros((1, 1, 64, 64), device="cuda")
    with pytest.raises(psx.PsxError) as e:   # 64 query rows per kv head
        ctx.decode_attention(q, kv, kv, 8)
    assert e.value.status == psx.ERR_UNSUPPORTED
