"""Pins the CPU checker: the plain-C restatement (oracle/psx_oracle.c) against the reference's own
known-answer vectors, against the reference compiled from its sources (oracle/_ref), and against
the committed golden fixtures.  CPU only.

The cases restate the reference's tests for this path: tests/generation_test.cpp:66-245,
tests/top_k_test.cpp:49-144, tests/backend_primitive_equivalence_cases.hpp:345-375,
tests/determinism_test.cpp:41-53, tests/sampler_test.cpp:20-77.
"""
import ctypes as C
import json
import math
from pathlib import Path

import numpy as np
import pytest

import oracle_lib as ol
import workload_rows
from pulsatrix_b200.workloads import WORKLOADS

GOLDEN = Path(__file__).resolve().parent / "golden"
KINDS = ["oracle"] + (["reference"] if ol.reference_available() else [])
needs_reference = pytest.mark.skipif(not ol.reference_available(), reason="compiled reference not present")


def _special(v):
    return {"ninf": -math.inf, "inf": math.inf, "nan": math.nan}.get(v, v) if isinstance(v, str) else v


def _floats(xs):
    return np.array([_special(x) for x in xs], dtype=np.float32)


# ---- ProcessLogits vs the Hugging Face vectors (tests/generation_test.cpp:66-106) --------------

HF = json.loads((GOLDEN / "hf_logit_processing.json").read_text())


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("case", HF["cases"], ids=lambda c: c["name"])
def test_logit_processing_matches_hugging_face(kind, case):
    cfg = ol.make_config(**case["config"])
    rc, out = ol.process_logits(kind, HF["logits"], HF["tokens"], case["num_new_tokens"], cfg)
    assert rc == ol.OK
    expected = _floats(case["expected"])
    inf = np.isinf(expected)
    assert (out[inf] == expected[inf]).all()
    assert np.abs(out[~inf] - expected[~inf]).max() <= 1e-5


# ---- Generate (tests/generation_test.cpp:115-181, 224-245) -------------------------------------

def _bigram_row(last):
    row = np.zeros(5, dtype=np.float32)
    row[(last + 1) % 5] = 4.0
    return row


def _bigram_table(first, n):
    """Rows of the bigram model along its greedy path from token `first`."""
    rows, last = [], first
    for _ in range(n):
        rows.append(_bigram_row(last))
        last = (last + 1) % 5
    return np.stack(rows)


@pytest.mark.parametrize("kind", KINDS)
def test_greedy_follows_the_model_and_stops_at_eos(kind):
    cfg = ol.make_config(max_new_tokens=10, eos_token_ids=[4])
    rc, tokens, logp, eos = ol.generate_table(kind, _bigram_table(1, 10), [1], cfg, 0)
    assert rc == ol.OK
    assert tokens.tolist() == [1, 2, 3, 4]
    assert eos
    assert len(logp) == 3
    assert abs(logp[0] - (4.0 - math.log(math.exp(4.0) + 4.0))) <= 1e-6

    cfg = ol.make_config(max_new_tokens=7)
    rc, tokens, logp, eos = ol.generate_table(kind, _bigram_table(1, 7), [1], cfg, 0)
    assert tokens.tolist()[1:] == [2, 3, 4, 0, 1, 2, 3]
    assert not eos


@pytest.mark.parametrize("kind", KINDS)
def test_min_new_tokens_holds_off_eos(kind):
    # EOS (2) is banned for the first 3 tokens; with it gone every other token ties at 0 and the
    # lowest index wins, so the path is 1 -> 0 -> 1 -> 0 -> then 1 -> 2 once the ban lifts.
    cfg = ol.make_config(max_new_tokens=10, eos_token_ids=[2])
    rc, tokens, _, eos = ol.generate_table(kind, _bigram_table(1, 10), [1], cfg, 0)
    assert tokens.tolist() == [1, 2] and eos
    cfg = ol.make_config(max_new_tokens=10, eos_token_ids=[2], min_new_tokens=3)
    table = np.stack([_bigram_row(t) for t in [1, 0, 1, 0, 1, 0, 1, 0, 1, 0]])
    rc, tokens, _, eos = ol.generate_table(kind, table, [1], cfg, 0)
    assert rc == ol.OK
    new = tokens.tolist()[1:]
    assert len(new) >= 4 and new[0] != 2 and new[0] == 0 and eos


@pytest.mark.parametrize("kind", KINDS)
def test_sampling_is_seeded_and_follows_the_distribution(kind):
    fixed = np.array([0.0, 1.0, 2.0, -1.0], dtype=np.float32)
    n = 40000
    cfg = ol.make_config(max_new_tokens=n, do_sample=True, temperature=0.5)
    table = np.tile(fixed, (n, 1))
    rc, tokens, _, _ = ol.generate_table(kind, table, [0], cfg, 17)
    assert rc == ol.OK
    new = tokens[1:]
    p = np.exp(2.0 * fixed.astype(np.float64))
    p /= p.sum()
    for t in range(4):
        assert abs((new == t).mean() - p[t]) <= 0.01
    cfg = ol.make_config(max_new_tokens=50, do_sample=True, temperature=0.5)
    a = ol.generate_table(kind, table[:50], [0], cfg, 17)[1]
    b = ol.generate_table(kind, table[:50], [0], cfg, 17)[1]
    c = ol.generate_table(kind, table[:50], [0], cfg, 18)[1]
    assert (a == b).all() and not (a == c).all()
    cfg = ol.make_config(max_new_tokens=50, do_sample=True, temperature=0.5, top_k=1)
    assert (ol.generate_table(kind, table[:50], [0], cfg, 17)[1][1:] == 2).all()


@needs_reference
def test_sampled_chain_matches_the_reference_token_for_token():
    rng = np.random.RandomState(5)
    table = (rng.randn(200, 300) * 2.0).astype(np.float32)
    for seed, kw in [(3, dict(top_k=5)), (9, dict(top_p=0.7, temperature=0.6, repetition_penalty=1.3)),
                     (11, dict(min_p=0.02, temperature=1.4)), (12, dict())]:
        cfg = ol.make_config(max_new_tokens=200, do_sample=True, eos_token_ids=[7], min_new_tokens=20, **kw)
        a = ol.generate_table("oracle", table, [1, 2, 3], cfg, seed)
        b = ol.generate_table("reference", table, [1, 2, 3], cfg, seed)
        assert a[0] == b[0] == ol.OK
        assert a[1].tolist() == b[1].tolist()
        assert (a[2] == b[2]).all()
        assert a[3] == b[3]


@pytest.mark.parametrize("kind", KINDS)
def test_rejects_bad_input(kind):
    table = _bigram_table(1, 4)
    assert ol.generate_table(kind, table, [], ol.make_config(), 0)[0] == ol.EMPTY_PROMPT
    for bad in (dict(temperature=0.0), dict(top_p=0.0), dict(top_k=-1), dict(min_p=1.5), dict(repetition_penalty=0.0),
                dict(temperature=math.inf), dict(max_new_tokens=-1)):
        assert ol.generate_table(kind, table, [1], ol.make_config(**bad), 0)[0] == ol.BAD_CONFIG
    nan_table = np.array([[0.0, math.nan]], dtype=np.float32)
    assert ol.generate_table(kind, nan_table, [1], ol.make_config(), 0)[0] == ol.NON_FINITE
    inf_table = np.array([[0.0, -math.inf]], dtype=np.float32)
    assert ol.generate_table(kind, inf_table, [1], ol.make_config(), 0)[0] == ol.NON_FINITE
    banned = ol.make_config(min_new_tokens=1, eos_token_ids=[0, 1, 2, 3, 4])
    assert ol.generate_table(kind, table, [1], banned, 0)[0] == ol.ALL_REMOVED


def test_mt19937_64_is_the_standard_engine():
    # ISO C++ [rand.predef]: the 10000th value of a default-seeded mt19937_64.
    class Mt(C.Structure):
        _fields_ = [("mt", C.c_uint64 * 312), ("index", C.c_int)]

    g = Mt()
    ol.oracle().psxo_mt_seed(C.byref(g), C.c_uint64(5489))
    for _ in range(9999):
        ol.oracle().psxo_mt_next(C.byref(g))
    assert ol.oracle().psxo_mt_next(C.byref(g)) == 9981545732273789042


# ---- random cross-checks of the restatement against the compiled reference ----------------------

@needs_reference
@pytest.mark.parametrize("seed", range(6))
def test_process_logits_matches_the_reference_on_random_rows(seed):
    rng = np.random.RandomState(100 + seed)
    for _ in range(40):
        vocab = int(rng.choice([1, 2, 3, 17, 64, 257, 1000]))
        logits = (rng.randn(vocab) * rng.choice([0.5, 2.0, 6.0])).astype(np.float32)
        if rng.rand() < 0.5:  # quantise so that ties are common
            logits = np.round(logits * 2) / 2
        tokens = rng.randint(-3, vocab + 3, size=rng.randint(0, 40))
        cfg = ol.make_config(do_sample=bool(rng.rand() < 0.85), temperature=float(rng.choice([0.3, 0.7, 1.0, 1.7])),
                             top_k=int(rng.choice([0, 1, 2, 5, 50, vocab, vocab + 5])),
                             top_p=float(rng.choice([1.0, 0.95, 0.5, 0.1])),
                             min_p=float(rng.choice([0.0, 0.0, 0.05, 0.5])),
                             repetition_penalty=float(rng.choice([1.0, 1.2, 0.8])),
                             min_new_tokens=int(rng.choice([0, 3])), eos_token_ids=rng.randint(0, vocab, size=2))
        num_new = int(rng.randint(0, 5))
        ra, a = ol.process_logits("oracle", logits, tokens, num_new, cfg)
        rb, b = ol.process_logits("reference", logits, tokens, num_new, cfg)
        assert ra == rb == ol.OK
        assert a.tobytes() == b.tobytes()


# ---- top-k (tests/top_k_test.cpp, tests/backend_primitive_equivalence_cases.hpp:345-375) -------

TOPK = json.loads((GOLDEN / "top_k_cases.json").read_text())


def _same(a, b):
    a, b = np.asarray(a, dtype=np.float32), np.asarray(b, dtype=np.float32)
    return a.shape == b.shape and bool(((a == b) | (np.isnan(a) & np.isnan(b))).all())


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("case", TOPK["cases"], ids=lambda c: c["name"])
def test_top_k_known_answers(kind, case):
    values, indices = ol.top_k_rows(kind, _floats(case["row"])[None, :], case["k"], case["largest"])
    assert _same(values[0], _floats(case["values"]))
    assert indices[0].tolist() == case["indices"]


def tie_heavy_values(n, seed):
    """The reference tests' coarse 9-level values (tests/top_k_test.cpp:36-43)."""
    out = np.zeros(n, dtype=np.float32)
    for i in range(n):
        seed = (seed * 1664525 + 1013904223) & 0xFFFFFFFF
        out[i] = (int((seed >> 16) % 9) - 4) * 0.5
    return out


def stable_order(row, largest):
    """NaN above every number, equal values keep the lower index: a stable sort on a rank key."""
    key = np.where(np.isnan(row), np.inf, row.astype(np.float64))
    key = np.where(np.isnan(row), 2.0, np.where(np.isposinf(row), 1.0, 0.0)) * 1e300 + np.where(np.isfinite(row), key, 0)
    key = np.where(np.isneginf(row), -1e300, key)
    return np.argsort(-key if largest else key, kind="stable")


@pytest.mark.parametrize("kind", KINDS)
def test_top_k_matches_a_stable_sort_row_by_row(kind):
    rows, cols = 37, 53
    v = tie_heavy_values(rows * cols, 11)
    v[5] = np.nan
    v[cols + 9] = -np.inf
    x = v.reshape(rows, cols)
    for largest in (True, False):
        for k in (1, 4, 17, cols):
            values, indices = ol.top_k_rows(kind, x, k, largest)
            for r in range(rows):
                order = stable_order(x[r], largest)[:k]
                assert indices[r].tolist() == order.tolist()
                assert _same(values[r], x[r][order])


@needs_reference
def test_top_k_rows_restatement_equals_the_reference_bit_for_bit():
    rng = np.random.RandomState(41)
    x = ((rng.randint(0, 9, size=(300, 129)) - 4) * 0.5).astype(np.float32)
    x[0, 3] = np.nan
    x[1, 7] = np.inf
    x[2, 1] = -np.inf
    x[3, 0] = -0.0
    for largest in (True, False):
        for k in (1, 7, 129):
            va, ia = ol.top_k_rows("oracle", x, k, largest)
            vb, ib = ol.top_k_rows("reference", x, k, largest)
            assert (ia == ib).all()
            assert _same(va, vb)
            assert (np.signbit(va) == np.signbit(vb)).all()


# ---- seed streams (tests/determinism_test.cpp:41-53, src/portable_random.hpp) -------------------

@needs_reference
def test_seed_streams_match_the_reference():
    for seed in (0, 5, 2**63 + 11):
        ol.oracle().psxo_set_seed(C.c_uint64(seed))
        ol.reference().psxref_set_seed(C.c_uint64(seed))
        a = [ol.oracle().psxo_next_seed() for _ in range(20)]
        b = [ol.reference().psxref_next_seed() for _ in range(20)]
        assert a == b and len(set(a)) == 20
    n = 64
    words = np.zeros(n, dtype=np.uint64)
    uni = np.zeros(n, dtype=np.float64)
    gau = np.zeros(n, dtype=np.float64)
    ol.reference().psxref_portable_streams(C.c_uint64(99), C.c_int64(n), words.ctypes.data_as(C.c_void_p),
                                           uni.ctypes.data_as(C.c_void_p), gau.ctypes.data_as(C.c_void_p))

    class Rng(C.Structure):
        _fields_ = [("state", C.c_uint64)]

    a, b, c = Rng(99), Rng(99), Rng(99)
    for i in range(n):
        assert ol.oracle().psxo_prng_next(C.byref(a)) == int(words[i])
        assert ol.oracle().psxo_prng_uniform(C.byref(b)) == uni[i]
        assert ol.oracle().psxo_prng_gaussian(C.byref(c)) == gau[i]


# ---- the five workloads against the committed fixtures ------------------------------------------

@pytest.mark.parametrize("name", list(WORKLOADS))
def test_restatement_reproduces_the_golden_rows(name):
    w = WORKLOADS[name]
    gold = np.load(GOLDEN / f"workload_{name}.npz")
    assert len(gold["token"]) == w.rows
    rng = np.random.RandomState(1)
    ids = np.sort(rng.choice(w.rows, size=min(w.rows, 6 if w.vocab > 100000 else 12), replace=False))
    logits, hist, offsets, seeds = workload_rows.build(name, ids)
    assert [workload_rows.logits_checksum(r) for r in logits] == gold["checksum"][ids].tolist()
    got = ol.rows("oracle", logits, hist, offsets, workload_rows.config_of(w), seeds, threads=4)
    assert (got["status"] == 0).all()
    assert got["token"].tolist() == gold["token"][ids].tolist()
    assert (got["log_prob"] == gold["log_prob"][ids]).all()
    assert got["survivors"].tolist() == gold["survivors"][ids].tolist()
    if w.do_sample:
        assert np.allclose(got["u"], ol.mt_uniforms(seeds), rtol=0, atol=0)


# ---- the float row primitives beside the path (src/cpu_backend.cpp:292-338,459-466) ---------------------

@pytest.mark.parametrize("kind", KINDS)
def test_row_primitives_known_answers(kind):
    x = np.array([[0.0, 0.0, 0.0, 0.0], [1.0, 2.0, 3.0, 4.0], [-1e30, 5.0, 5.0, -np.inf]], dtype=np.float32)
    y = ol.row_primitive(kind, "softmax_rows", x)
    assert y[0].tolist() == [0.25] * 4
    e = np.exp(x[1].astype(np.float64) - 4.0)
    assert np.allclose(y[1], e / e.sum(), rtol=1e-6)
    assert y[2].tolist() == [0.0, 0.5, 0.5, 0.0]
    lse = ol.row_primitive(kind, "logsumexp_rows", x)
    assert np.allclose(lse, [np.log(4.0), 4.0 + np.log(e.sum()), 5.0 + np.log(2.0)], rtol=1e-6)
    table = np.arange(12, dtype=np.float32).reshape(4, 3)
    got = ol.row_primitive(kind, "gather_rows", table, np.array([3.0, 0.0, 3.0, 1.0], dtype=np.float32))
    assert got.tolist() == table[[3, 0, 3, 1]].tolist()


@needs_reference
def test_row_primitive_restatements_equal_the_reference_bit_for_bit():
    rng = np.random.RandomState(5)
    for rows, cols in [(3, 1), (5, 17), (2, 1000), (4, 4097)]:
        x = (rng.randn(rows, cols) * 4).astype(np.float32)
        for name in ("softmax_rows", "logsumexp_rows"):
            assert ol.row_primitive("oracle", name, x).tobytes() == ol.row_primitive("reference", name, x).tobytes()
    table = rng.randn(50, 7).astype(np.float32)
    idx = rng.randint(0, 50, size=31).astype(np.float32)
    assert ol.row_primitive("oracle", "gather_rows", table, idx).tobytes() == \
        ol.row_primitive("reference", "gather_rows", table, idx).tobytes()


@needs_reference
def test_decode_attention_restatement_equals_the_reference_bit_for_bit():
    """psxo_decode_attention against the reference's own CPUBackend calls of forward_cached's core
    (src/multihead_attention_module.cpp:562-586): grouped-query heads, new positions, every mask."""
    rng = np.random.RandomState(11)
    cases = [dict(batch=2, heads=4, kv_heads=2, q_len=1, d=16, cached=37, max_len=48, causal=True, window=0, padding=False),
             dict(batch=1, heads=6, kv_heads=3, q_len=3, d=8, cached=20, max_len=32, causal=True, window=7, padding=True),
             dict(batch=3, heads=2, kv_heads=2, q_len=2, d=12, cached=0, max_len=4, causal=False, window=0, padding=True),
             dict(batch=2, heads=8, kv_heads=1, q_len=1, d=64, cached=300, max_len=301, causal=True, window=0, padding=False)]
    for c in cases:
        q = rng.randn(c["batch"], c["heads"], c["q_len"], c["d"]).astype(np.float32)
        keys = rng.randn(c["batch"], c["kv_heads"], c["max_len"], c["d"]).astype(np.float32)
        values = rng.randn(c["batch"], c["kv_heads"], c["max_len"], c["d"]).astype(np.float32)
        keep = None
        if c["padding"]:
            keep = (rng.rand(c["batch"], c["cached"] + c["q_len"]) > 0.4).astype(np.float32)
            keep[0, :] = 0.0  # a fully masked entry: every score is the lowest float, the softmax uniform
        scale = float(1.0 / np.sqrt(np.float32(c["d"])))
        a = ol.decode_attention("oracle", q, keys, values, c["cached"], scale, c["causal"], c["window"], keep)
        b = ol.decode_attention("reference", q, keys, values, c["cached"], scale, c["causal"], c["window"], keep)
        assert a.tobytes() == b.tobytes()
        if keep is not None and not c["causal"]:
            total = c["cached"] + c["q_len"]
            assert np.allclose(a[0, 0, 0], values[0, 0, :total].mean(axis=0), rtol=1e-5, atol=1e-6)  # uniform over all positions
