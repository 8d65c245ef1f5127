"""ctypes bindings for the two CPU checkers under oracle/ (test infrastructure).

`oracle()` loads oracle/libpsx_oracle.so, the plain-C restatement; it is built on demand with
gcc.  `reference()` loads oracle/_ref/libpsx_ref.so, the reference's own sources compiled in
place; it is built on demand when the reference checkout is present and is otherwise used as
shipped (or reported missing, and the tests that need it skip).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
ORACLE_DIR = ROOT / "oracle"
# The reference checkout: PSX_REFERENCE_DIR, else a directory named `reference` beside this repository.
REFERENCE_CHECKOUT = Path(os.environ.get("PSX_REFERENCE_DIR") or ROOT.parent / "reference")

OK, BAD_CONFIG, EMPTY_PROMPT, EMPTY_LOGITS, NON_FINITE, ALL_REMOVED = range(6)


class Config(C.Structure):
    """psxo_config: GenerationConfig flattened to C (include/pulsatrix/generation.hpp:29-52)."""

    _fields_ = [
        ("max_new_tokens", C.c_int64),
        ("min_new_tokens", C.c_int64),
        ("eos_token_ids", C.POINTER(C.c_int64)),
        ("num_eos_token_ids", C.c_int64),
        ("do_sample", C.c_int32),
        ("temperature", C.c_float),
        ("top_k", C.c_int64),
        ("top_p", C.c_float),
        ("min_p", C.c_float),
        ("repetition_penalty", C.c_float),
    ]


class StepInfo(C.Structure):
    _fields_ = [
        ("token", C.c_int64),
        ("log_prob", C.c_float),
        ("status", C.c_int32),
        ("survivors", C.c_int64),
        ("u", C.c_double),
        ("draw_margin", C.c_double),
        ("top_p_margin", C.c_double),
    ]


STEP_INFO_DTYPE = np.dtype(
    {
        "names": ["token", "log_prob", "status", "survivors", "u", "draw_margin", "top_p_margin"],
        "formats": ["<i8", "<f4", "<i4", "<i8", "<f8", "<f8", "<f8"],
        "offsets": [StepInfo.token.offset, StepInfo.log_prob.offset, StepInfo.status.offset,
                    StepInfo.survivors.offset, StepInfo.u.offset, StepInfo.draw_margin.offset,
                    StepInfo.top_p_margin.offset],
        "itemsize": C.sizeof(StepInfo),
    }
)


def make_config(max_new_tokens=32, min_new_tokens=0, eos_token_ids=(), do_sample=False, temperature=1.0,
                top_k=0, top_p=1.0, min_p=0.0, repetition_penalty=1.0):
    """A psxo_config with GenerationConfig's defaults; keeps the EOS array alive on the object."""
    eos = np.asarray(list(eos_token_ids), dtype=np.int64)
    cfg = Config(max_new_tokens, min_new_tokens, eos.ctypes.data_as(C.POINTER(C.c_int64)), len(eos),
                 int(do_sample), temperature, top_k, top_p, min_p, repetition_penalty)
    cfg._eos_keepalive = eos
    return cfg


def _ptr(a, ctype):
    return a.ctypes.data_as(C.POINTER(ctype))


def _build(target: str) -> None:
    subprocess.run(["make", "-C", str(ORACLE_DIR), "-j8", target, f"REF={REFERENCE_CHECKOUT}"], check=True,
                   stdout=subprocess.DEVNULL)


_oracle = None
_reference = None


def oracle():
    global _oracle
    if _oracle is None:
        _build("oracle")
        lib = C.CDLL(str(ORACLE_DIR / "libpsx_oracle.so"))
        lib.psxo_next_seed.restype = C.c_uint64
        lib.psxo_mt_next.restype = C.c_uint64
        lib.psxo_mt_uniform.restype = C.c_double
        lib.psxo_prng_next.restype = C.c_uint64
        lib.psxo_prng_uniform.restype = C.c_double
        lib.psxo_prng_gaussian.restype = C.c_double
        _oracle = lib
    return _oracle


def reference_available() -> bool:
    return (ORACLE_DIR / "_ref" / "libpsx_ref.so").exists() or (REFERENCE_CHECKOUT / "src" / "generation.cpp").exists()


def reference():
    global _reference
    if _reference is None:
        if (REFERENCE_CHECKOUT / "src" / "generation.cpp").exists():
            _build("ref")
        lib = C.CDLL(str(ORACLE_DIR / "_ref" / "libpsx_ref.so"))
        lib.psxref_next_seed.restype = C.c_uint64
        _reference = lib
    return _reference


# ---- thin numpy wrappers ----------------------------------------------------------------------

def process_logits(lib_kind, logits, tokens, num_new_tokens, cfg):
    """ProcessLogits through the restatement ('oracle') or the compiled reference ('reference')."""
    out = np.array(logits, dtype=np.float32)
    toks = np.asarray(tokens, dtype=np.int64)
    if lib_kind == "oracle":
        rc = oracle().psxo_process_logits(_ptr(out, C.c_float), C.c_int64(out.size), _ptr(toks, C.c_int64),
                                          C.c_int64(toks.size), C.c_int64(num_new_tokens), C.byref(cfg), None)
    else:
        rc = reference().psxref_process_logits(_ptr(out, C.c_float), C.c_int64(out.size), _ptr(toks, C.c_int64),
                                               C.c_int64(toks.size), C.c_int64(num_new_tokens), C.byref(cfg))
    return rc, out


def rows(lib_kind, logits, hist, offsets, cfg, seeds, threads=8):
    """Independent rows, one Generate(max_new_tokens=1, seed) each.  Returns a structured array."""
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    n_rows, vocab = logits.shape
    hist = np.ascontiguousarray(hist, dtype=np.int64)
    offsets = np.ascontiguousarray(offsets, dtype=np.int64)
    seeds = np.ascontiguousarray(seeds, dtype=np.uint64)
    infos = np.zeros(n_rows, dtype=STEP_INFO_DTYPE)
    fn = oracle().psxo_rows if lib_kind == "oracle" else reference().psxref_rows
    fn(_ptr(logits, C.c_float), C.c_int64(n_rows), C.c_int64(vocab), C.c_int64(vocab), _ptr(hist, C.c_int64),
       _ptr(offsets, C.c_int64), C.byref(cfg), _ptr(seeds, C.c_uint64), C.c_int(threads),
       infos.ctypes.data_as(C.c_void_p))
    return infos


def generate_table(lib_kind, logits_steps, prompt, cfg, seed):
    """Generate() with the model given as a (steps, vocab) table.  seed=None -> global stream
    (reference only)."""
    logits_steps = np.ascontiguousarray(logits_steps, dtype=np.float32)
    steps, vocab = logits_steps.shape
    prompt = np.asarray(prompt, dtype=np.int64)
    tokens = np.zeros(prompt.size + max(cfg.max_new_tokens, 0) + 1, dtype=np.int64)
    logp = np.zeros(max(cfg.max_new_tokens, 0) + 1, dtype=np.float32)
    n_new = C.c_int64(0)
    eos = C.c_int32(0)
    if lib_kind == "oracle":
        rc = oracle().psxo_generate_table(_ptr(logits_steps, C.c_float), C.c_int64(vocab), _ptr(prompt, C.c_int64),
                                          C.c_int64(prompt.size), C.byref(cfg), C.c_uint64(seed),
                                          _ptr(tokens, C.c_int64), _ptr(logp, C.c_float), C.byref(n_new),
                                          C.byref(eos), None)
    else:
        rc = reference().psxref_generate_table(_ptr(logits_steps, C.c_float), C.c_int64(vocab),
                                               _ptr(prompt, C.c_int64), C.c_int64(prompt.size), C.byref(cfg),
                                               C.c_int32(seed is not None), C.c_uint64(seed or 0),
                                               _ptr(tokens, C.c_int64), _ptr(logp, C.c_float), C.byref(n_new),
                                               C.byref(eos))
    n = n_new.value
    return rc, tokens[: prompt.size + n].copy(), logp[:n].copy(), bool(eos.value)


def top_k_rows(lib_kind, x, k, largest=True):
    x = np.ascontiguousarray(x, dtype=np.float32)
    n_rows, cols = x.shape
    values = np.zeros((n_rows, k), dtype=np.float32)
    indices = np.zeros((n_rows, k), dtype=np.float32)
    fn = oracle().psxo_top_k_rows if lib_kind == "oracle" else reference().psxref_top_k_rows
    fn(_ptr(x, C.c_float), _ptr(values, C.c_float), _ptr(indices, C.c_float), C.c_int64(n_rows), C.c_int64(cols),
       C.c_int64(k), C.c_int(int(largest)))
    return values, indices


def row_primitive(lib_kind, name, *arrays):
    """softmax_rows / logsumexp_rows (x) or gather_rows (table, indices) through a CPU checker."""
    lib = oracle() if lib_kind == "oracle" else reference()
    prefix = "psxo_" if lib_kind == "oracle" else "psxref_"
    fn = getattr(lib, prefix + name)
    if name == "gather_rows":
        table, indices = (np.ascontiguousarray(a, dtype=np.float32) for a in arrays)
        out = np.empty((indices.shape[0], table.shape[1]), dtype=np.float32)
        fn(_ptr(table, C.c_float), _ptr(indices, C.c_float), _ptr(out, C.c_float), C.c_int64(indices.shape[0]),
           C.c_int64(table.shape[1]))
        return out
    x = np.ascontiguousarray(arrays[0], dtype=np.float32)
    out = np.empty_like(x) if name == "softmax_rows" else np.empty(x.shape[0], dtype=np.float32)
    fn(_ptr(x, C.c_float), _ptr(out, C.c_float), C.c_int64(x.shape[0]), C.c_int64(x.shape[1]))
    return out


def decode_attention(lib_kind, q, keys, values, cached, scale, causal=True, window=0, key_keep=None):
    """Attention of the new positions over the KV cache through a CPU checker.  q: (batch, heads, q_len, d);
    keys / values: (batch, kv_heads, max_len, d)."""
    lib = oracle() if lib_kind == "oracle" else reference()
    fn = getattr(lib, ("psxo_" if lib_kind == "oracle" else "psxref_") + "decode_attention")
    q = np.ascontiguousarray(q, dtype=np.float32)
    keys = np.ascontiguousarray(keys, dtype=np.float32)
    values = np.ascontiguousarray(values, dtype=np.float32)
    keep = None if key_keep is None else np.ascontiguousarray(key_keep, dtype=np.float32)
    batch, heads, q_len, d = q.shape
    out = np.empty_like(q)
    fn.restype = None
    fn(_ptr(q, C.c_float), _ptr(keys, C.c_float), _ptr(values, C.c_float), _ptr(keep, C.c_float) if keep is not None else None,
       _ptr(out, C.c_float), C.c_int64(batch), C.c_int64(heads), C.c_int64(keys.shape[1]), C.c_int64(q_len), C.c_int64(d),
       C.c_int64(cached), C.c_int64(keys.shape[2]), C.c_float(scale), C.c_int(int(bool(causal))), C.c_int64(window))
    return out


def mt_uniforms(seeds):
    """First uniform of std::mt19937_64(seed) for each seed: (engine() >> 11) * 2^-53."""
    lib = oracle()

    class Mt(C.Structure):
        _fields_ = [("mt", C.c_uint64 * 312), ("index", C.c_int)]

    out = np.zeros(len(seeds), dtype=np.float64)
    g = Mt()
    for i, s in enumerate(seeds):
        lib.psxo_mt_seed(C.byref(g), C.c_uint64(int(s)))
        out[i] = lib.psxo_mt_uniform(C.byref(g))
    return out


def synth_rows(row_seeds, vocab, sigma, zeta, history_len):
    """Rows of the synthetic workload, one per generator seed in row_seeds."""
    lib = oracle()
    n_rows = len(row_seeds)
    logits = np.zeros((n_rows, vocab), dtype=np.float32)
    hist = np.zeros((n_rows, max(history_len, 0)), dtype=np.int64)
    for r, seed in enumerate(row_seeds):
        lib.psxo_synth_row(C.c_uint64(int(seed)), C.c_int64(vocab), C.c_double(sigma), C.c_double(zeta),
                           _ptr(logits[r], C.c_float), C.c_int64(history_len),
                           _ptr(hist[r], C.c_int64) if history_len > 0 else None)
    return logits, hist
