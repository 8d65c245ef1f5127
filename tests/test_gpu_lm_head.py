"""The language-model head on the device (psx_b200_lm_head_logits / psx_b200_lm_head_sample_rows).

Against the reference's own tiny Hugging Face models (tests/golden/hf_tiny_heads.npz, made by
tests/golden/make_golden.py --tiny-heads from the compiled reference: per greedy step the head's
input, the reference's logits and its token -- the tokens are those of its
CausalLMTest.GreedyGenerationMatchesTransformers, tests/causal_lm_test.cpp:270-278): the logits must
be the reference's bit for bit and the greedy tokens equal.  Against a numpy emulation of the
reference's loop (one float accumulator per logit, ascending feature order, product and sum each
rounded, src/cpu_backend.cpp:188-196) on larger shapes, both weight layouts: bit-exact."""
from pathlib import Path

import numpy as np
import pytest

import gpu_harness as gh
import oracle_lib as ol
import pulsatrix_b200 as psx

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden" / "hf_tiny_heads.npz"
MODELS = ["llama", "qwen2", "qwen3", "gemma3"]


def reference_head(hidden, weight_vocab_by_d):
    """The reference's loop, vectorised over the vocabulary: acc = fl(acc + fl(h[p] * w[:, p])) for p ascending."""
    rows, d = hidden.shape
    out = np.zeros((rows, weight_vocab_by_d.shape[0]), dtype=np.float32)
    for m in range(rows):
        acc = np.zeros(weight_vocab_by_d.shape[0], dtype=np.float32)
        for p in range(d):
            acc = (acc + (hidden[m, p] * weight_vocab_by_d[:, p]).astype(np.float32)).astype(np.float32)
        out[m] = acc
    return out


@pytest.mark.parametrize("name", MODELS)
def test_tiny_model_heads_give_the_references_logits_and_tokens(name):
    import torch
    gold = np.load(GOLDEN)
    weight, tied = gold[f"{name}_weight"], bool(gold[f"{name}_tied"])
    hidden, logits, tokens = gold[f"{name}_hidden"], gold[f"{name}_logits"], gold[f"{name}_tokens"]
    d_weight = torch.from_numpy(weight).cuda()
    d_hidden = torch.from_numpy(hidden).cuda()
    ctx = gh.ctx()
    got = ctx.lm_head_logits(d_hidden, d_weight, vocab_by_d=tied).cpu().numpy()  # all eight steps as a batch
    assert got.view(np.uint32).tolist() == logits.view(np.uint32).tolist()
    # the decode loop: head and greedy draw in one call per token, the row never leaves the device
    sequence = gold["prompt"].tolist()
    greedy = psx.SamplingConfig.make()
    for step in range(len(tokens)):
        history = torch.tensor(sequence, dtype=torch.int64, device="cuda")
        offsets = torch.tensor([0, len(sequence)], dtype=torch.int64, device="cuda")
        out = ctx.lm_head_sample_rows(d_hidden[step:step + 1], d_weight, history, offsets, greedy, None, vocab_by_d=tied)
        torch.cuda.synchronize()
        assert int(out["status"][0]) == 0
        token = int(out["tokens"][0])
        assert token == int(tokens[step])
        want = ol.rows("oracle", logits[step:step + 1], np.array(sequence, dtype=np.int64), np.array([0, len(sequence)]),
                       ol.make_config(max_new_tokens=1), np.zeros(1, dtype=np.uint64))
        assert abs(float(out["log_probs"][0]) - float(want["log_prob"][0])) <= 1e-5 * abs(float(want["log_prob"][0])) + 1e-9
        sequence.append(token)


@pytest.mark.parametrize("rows,d,vocab", [(1, 64, 1000), (3, 100, 5001), (8, 257, 4099), (17, 96, 3000), (64, 128, 2500),
                                          (70, 33, 777), (2, 2048, 20011)])
@pytest.mark.parametrize("vocab_by_d", [True, False])
def test_head_equals_the_references_loop_bit_for_bit(rows, d, vocab, vocab_by_d):
    import torch
    rng = np.random.RandomState(rows * 7 + d)
    hidden = rng.randn(rows, d).astype(np.float32)
    weight = (rng.randn(vocab, d) * 0.05).astype(np.float32)
    hidden[0, 0] = -0.0
    want = reference_head(hidden, weight)
    layout = weight if vocab_by_d else np.ascontiguousarray(weight.T)
    got = gh.ctx().lm_head_logits(torch.from_numpy(hidden).cuda(), torch.from_numpy(layout).cuda(), vocab_by_d=vocab_by_d)
    assert got.cpu().numpy().view(np.uint32).tolist() == want.view(np.uint32).tolist()


def test_head_and_sampling_in_one_call_match_sampling_the_references_logits():
    import torch
    rng = np.random.RandomState(4)
    rows, d, vocab, hlen = 12, 160, 30011, 20
    hidden = rng.randn(rows, d).astype(np.float32)
    weight = (rng.randn(vocab, d) * 0.3).astype(np.float32)
    logits = reference_head(hidden, weight)
    hist = rng.randint(0, vocab, size=(rows, hlen)).astype(np.int64)
    offsets = np.arange(rows + 1, dtype=np.int64) * hlen
    seeds = np.arange(rows, dtype=np.uint64) + 50
    cfg = ol.make_config(max_new_tokens=1, do_sample=True, temperature=0.8, top_k=40, top_p=0.9, repetition_penalty=1.2)
    want = ol.rows("oracle", logits, hist.ravel(), offsets, cfg, seeds)
    out = gh.ctx().lm_head_sample_rows(torch.from_numpy(hidden).cuda(), torch.from_numpy(weight).cuda(),
                                       torch.from_numpy(hist.ravel()).cuda(), torch.from_numpy(offsets).cuda(),
                                       gh.psx_config(cfg), torch.from_numpy(psx.uniforms_mt19937_64(seeds)).cuda())
    torch.cuda.synchronize()
    assert (out["status"].cpu().numpy() == 0).all()
    assert out["tokens"].cpu().numpy().tolist() == want["token"].tolist()
    assert np.allclose(out["log_probs"].cpu().numpy(), want["log_prob"], rtol=1e-5, atol=0)
