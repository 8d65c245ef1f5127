"""Regenerates tests/golden/workload_<name>.npz from the reference itself.

Run where the reference checkout is present (it is compiled in place into oracle/_ref by
oracle/Makefile):  python tests/golden/make_golden.py            (the five workloads)
                   python tests/golden/make_golden.py --tiny-heads   (hf_tiny_heads.npz, see tiny_heads)

For every row of the five workloads it stores what the reference's own Generate() decided
(token id, log-prob, status), what the plain-C restatement reports beside it (survivor count,
distance of the draw from its CDF bucket edges, distance of the top-p walk from its cut), and a
checksum of the generated logits so a drifting generator is noticed.  Inputs are not stored: the
seeded generator rebuilds them.
"""
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path[:0] = [str(HERE.parent.parent), str(HERE.parent)]

import oracle_lib  # noqa: E402
import workload_rows  # noqa: E402
from pulsatrix_b200.workloads import WORKLOADS  # noqa: E402


# The reference's own tiny Hugging Face models (tests/fixtures/hf_tiny/<name> of its checkout), the
# prompt and the tokens of its CausalLMTest.GreedyGenerationMatchesTransformers
# (tests/causal_lm_test.cpp:246,270-278).
TINY_MODELS = {"llama": [42, 41, 15, 6, 29, 45, 29, 50], "qwen2": [1, 46, 58, 57, 20, 11, 58, 25],
               "qwen3": [26, 16, 58, 16, 58, 16, 52, 0], "gemma3": [8, 30, 30, 30, 30, 30, 30, 30]}
TINY_PROMPT = [3, 17, 42, 5, 60, 8]


def tiny_heads():
    """tests/golden/hf_tiny_heads.npz: per model the head's weight matrix, and per greedy step the
    head's input, the reference's logits and its token -- what the device head is checked against."""
    import ctypes as C
    lib = oracle_lib.reference()
    out = {}
    steps = 8
    prompt = np.array(TINY_PROMPT, dtype=np.int64)
    for name, expected in TINY_MODELS.items():
        directory = oracle_lib.REFERENCE_CHECKOUT / "tests" / "fixtures" / "hf_tiny" / name
        d, vocab, tied = C.c_int64(), C.c_int64(), C.c_int32()
        weight = np.zeros(1 << 20, dtype=np.float32)
        hidden = np.zeros(steps * 4096, dtype=np.float32)
        logits = np.zeros(steps * 4096, dtype=np.float32)
        tokens = np.zeros(steps, dtype=np.int64)
        generated = np.zeros(steps, dtype=np.int64)
        ptr = lambda a: a.ctypes.data_as(C.c_void_p)  # noqa: E731
        rc = lib.psxref_tiny_lm(str(directory).encode(), ptr(prompt), C.c_int64(len(prompt)), C.c_int64(steps), C.byref(d),
                                C.byref(vocab), C.byref(tied), ptr(weight), C.c_int64(weight.size), ptr(hidden), ptr(logits),
                                ptr(tokens), ptr(generated))
        assert rc == 0, (name, rc)
        d, vocab = d.value, vocab.value
        assert generated.tolist() == expected == tokens.tolist(), (name, generated, tokens)
        shape = (vocab, d) if tied.value else (d, vocab)
        out[f"{name}_weight"] = weight[: d * vocab].reshape(shape).copy()
        out[f"{name}_tied"] = np.array(tied.value)
        out[f"{name}_hidden"] = hidden[: steps * d].reshape(steps, d).copy()
        out[f"{name}_logits"] = logits[: steps * vocab].reshape(steps, vocab).copy()
        out[f"{name}_tokens"] = tokens.copy()
        print(name, "d", d, "vocab", vocab, "tied", tied.value, "tokens", tokens.tolist())
    out["prompt"] = prompt
    np.savez_compressed(HERE / "hf_tiny_heads.npz", **out)


def main():
    if "--tiny-heads" in sys.argv or "--all" in sys.argv:
        tiny_heads()
        if "--all" not in sys.argv:
            return
    for name, w in WORKLOADS.items():
        out = {k: [] for k in ("token", "log_prob", "status", "survivors", "draw_margin", "top_p_margin", "u",
                               "checksum")}
        cfg = workload_rows.config_of(w)
        for start in range(0, w.rows, 64):
            ids = np.arange(start, min(start + 64, w.rows))
            logits, hist, offsets, seeds = workload_rows.build(name, ids)
            ref = oracle_lib.rows("reference", logits, hist, offsets, cfg, seeds, threads=8)
            orc = oracle_lib.rows("oracle", logits, hist, offsets, cfg, seeds, threads=8)
            assert (ref["token"] == orc["token"]).all(), f"{name}: restatement and reference disagree on a token"
            assert (ref["log_prob"] == orc["log_prob"]).all(), f"{name}: log-probs differ"
            assert (ref["status"] == 0).all()
            out["token"].append(ref["token"])
            out["log_prob"].append(ref["log_prob"])
            out["status"].append(ref["status"])
            for k in ("survivors", "draw_margin", "top_p_margin", "u"):
                out[k].append(orc[k])
            out["checksum"].append(np.array([workload_rows.logits_checksum(row) for row in logits], dtype=np.uint64))
        arrays = {k: np.concatenate(v) for k, v in out.items()}
        np.savez_compressed(HERE / f"workload_{name}.npz", **arrays)
        print(name, "rows", w.rows, "min draw margin", arrays["draw_margin"].min(), "min top-p margin",
              arrays["top_p_margin"].min(), "max survivors", arrays["survivors"].max())


if __name__ == "__main__":
    main()
