"""ctypes binding of include/psx_b200.h.  Device memory comes from torch tensors; every compute
call goes through the C ABI into the CUDA kernels."""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import numpy as np

PACKAGE = Path(__file__).resolve().parent
ROW_OK, ROW_NON_FINITE, ROW_ALL_REMOVED, ROW_TOO_WIDE, ROW_DEVICE_TIMEOUT = 0, 4, 5, 16, 32
OK, ERR_BAD_ARGUMENT, ERR_CUDA, ERR_ROW_FAILED, ERR_UNSUPPORTED = range(5)

EXPORTS = [
    "psx_b200_version", "psx_b200_last_error", "psx_b200_ctx_create", "psx_b200_ctx_destroy", "psx_b200_ctx_stream",
    "psx_b200_sync", "psx_b200_launch_count", "psx_b200_ctx_enable_timing", "psx_b200_ctx_read_timing", "psx_b200_ctx_inputs_are_ready",
    "psx_b200_ctx_set_wait_limit", "psx_b200_test_short_copy", "psx_b200_sample_rows", "psx_b200_sample_rows_host", "psx_b200_row_pass_only", "psx_b200_sample_rows_static", "psx_b200_read_only_pass", "psx_b200_process_logits", "psx_b200_process_logits_host",
    "psx_b200_shard_record_bytes", "psx_b200_shard_scan", "psx_b200_shard_merge", "psx_b200_shard_merge_rows",
    "psx_b200_exchange_handle_bytes", "psx_b200_exchange_create", "psx_b200_exchange_open", "psx_b200_exchange_destroy",
    "psx_b200_exchange_sample", "psx_b200_exchange_results", "psx_b200_exchange_test_wait",
    "psx_b200_top_k_rows", "psx_b200_lm_head_logits", "psx_b200_lm_head_sample_rows", "psx_b200_softmax_rows", "psx_b200_logsumexp_rows", "psx_b200_gather_rows", "psx_b200_decode_attention",
    "psx_uniforms_mt19937_64", "psx_uniforms_portable",
]


class PsxError(RuntimeError):
    """A C entry point returned a non-zero psx_status.  `.status` holds it; the text is the
    library's message (the reference's own wording for its std::invalid_argument cases)."""

    def __init__(self, status, message):
        super().__init__(message)
        self.status = status


class SamplingConfig(C.Structure):
    """psx_sampling_config."""

    _fields_ = [
        ("min_new_tokens", C.c_int64),
        ("num_new_tokens", C.c_int64),
        ("eos_token_ids", C.POINTER(C.c_int64)),
        ("num_eos_token_ids", C.c_int64),
        ("do_sample", C.c_int32),
        ("temperature", C.c_float),
        ("top_k", C.c_int64),
        ("top_p", C.c_float),
        ("min_p", C.c_float),
        ("repetition_penalty", C.c_float),
    ]

    @classmethod
    def make(cls, do_sample=False, temperature=1.0, top_k=0, top_p=1.0, min_p=0.0, repetition_penalty=1.0,
             min_new_tokens=0, num_new_tokens=0, eos_token_ids=()):
        eos = np.asarray(list(eos_token_ids), dtype=np.int64)
        cfg = cls(min_new_tokens, num_new_tokens, eos.ctypes.data_as(C.POINTER(C.c_int64)), len(eos), int(do_sample),
                  temperature, top_k, top_p, min_p, repetition_penalty)
        cfg._keepalive = eos
        return cfg


class RowDiag(C.Structure):
    """psx_row_diag."""

    _fields_ = [("candidates", C.c_int32), ("survivors", C.c_int32), ("draw_margin", C.c_double),
                ("top_p_margin", C.c_double)]


ROW_DIAG_DTYPE = np.dtype({"names": ["candidates", "survivors", "draw_margin", "top_p_margin"],
                           "formats": ["<i4", "<i4", "<f8", "<f8"], "itemsize": C.sizeof(RowDiag)})

_lib = None


def library_path() -> Path:
    if os.environ.get("PSX_B200_LIBRARY"):  # a variant build (see build.py)
        return Path(os.environ["PSX_B200_LIBRARY"])
    if os.environ.get("PSX_B200_STAGE_CLOCKS") == "1":  # the profiling build (see build.py)
        return PACKAGE / "libpsx_b200_clocks.so"
    return PACKAGE / "libpsx_b200.so"


def library():
    """Loads libpsx_b200.so.  Raises when it has not been built: there is nothing to fall back to."""
    global _lib
    if _lib is None:
        path = library_path()
        if not path.exists():
            raise ImportError(f"{path} is missing: build it with `python -m pulsatrix_b200.build` (needs nvcc)")
        lib = C.CDLL(str(path))
        lib.psx_b200_version.restype = C.c_char_p
        lib.psx_b200_last_error.restype = C.c_char_p
        lib.psx_b200_ctx_stream.restype = C.c_void_p
        lib.psx_b200_ctx_stream.argtypes = [C.c_void_p]
        lib.psx_b200_ctx_destroy.argtypes = [C.c_void_p]
        lib.psx_b200_launch_count.restype = C.c_uint64
        lib.psx_b200_launch_count.argtypes = [C.c_void_p]
        lib.psx_b200_shard_record_bytes.restype = C.c_size_t
        lib.psx_b200_shard_record_bytes.argtypes = [C.c_void_p]
        lib.psx_b200_ctx_create.argtypes = [C.c_int, C.c_void_p]
        lib.psx_b200_sync.argtypes = [C.c_void_p, C.c_void_p]
        lib.psx_b200_ctx_enable_timing.argtypes = [C.c_void_p, C.c_int]
        lib.psx_b200_ctx_inputs_are_ready.argtypes = [C.c_void_p, C.c_int]
        lib.psx_b200_ctx_set_wait_limit.argtypes = [C.c_void_p, C.c_uint64]
        lib.psx_b200_test_short_copy.argtypes = [C.c_void_p, C.c_int]
        lib.psx_b200_ctx_read_timing.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        ptr, i64 = C.c_void_p, C.c_int64
        lib.psx_b200_sample_rows.argtypes = [ptr, ptr, ptr, i64, i64, i64, ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr]
        lib.psx_b200_sample_rows_static.argtypes = [ptr, ptr, i64, i64, i64, ptr, ptr, ptr, ptr, ptr, ptr, ptr]
        lib.psx_b200_read_only_pass.argtypes = [ptr, ptr, C.c_size_t, ptr]
        lib.psx_b200_process_logits.argtypes = [ptr, ptr, ptr, i64, i64, i64, ptr, ptr, ptr, ptr]
        lib.psx_b200_process_logits_host.argtypes = [ptr, ptr, i64, i64, i64, ptr, ptr, ptr, ptr]
        lib.psx_b200_row_pass_only.argtypes = [ptr, ptr, ptr, i64, i64, i64, ptr, ptr, ptr]
        lib.psx_b200_sample_rows_host.argtypes = [ptr, ptr, i64, i64, i64, ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr]
        lib.psx_b200_shard_scan.argtypes = [ptr, ptr, ptr, i64, i64, i64, i64, i64, ptr, ptr, ptr, ptr]
        lib.psx_b200_shard_merge.argtypes = [ptr, ptr, ptr, C.c_int32, i64, i64, ptr, ptr, ptr, ptr, ptr, ptr]
        lib.psx_b200_shard_merge_rows.argtypes = [ptr, ptr, ptr, C.c_int32, i64, i64, i64, i64, ptr, ptr, ptr, ptr, ptr, ptr]
        lib.psx_b200_exchange_handle_bytes.restype = C.c_size_t
        lib.psx_b200_exchange_handle_bytes.argtypes = []
        lib.psx_b200_exchange_create.argtypes = [ptr, C.c_int32, C.c_int32, i64, ptr, ptr, ptr]
        lib.psx_b200_exchange_open.argtypes = [ptr, ptr]
        lib.psx_b200_exchange_destroy.argtypes = [ptr]
        lib.psx_b200_exchange_destroy.restype = None
        lib.psx_b200_exchange_sample.argtypes = [ptr, ptr, ptr, i64, i64, i64, i64, ptr, ptr, ptr, ptr]
        lib.psx_b200_exchange_results.argtypes = [ptr, ptr, ptr]
        lib.psx_b200_exchange_test_wait.argtypes = [ptr, C.c_uint64, C.c_uint32]
        lib.psx_b200_top_k_rows.argtypes = [ptr, ptr, ptr, ptr, ptr, C.c_size_t, C.c_size_t, C.c_size_t, C.c_int]
        lib.psx_b200_lm_head_logits.argtypes = [ptr, ptr, ptr, i64, i64, ptr, i64, C.c_int32, ptr, i64]
        lib.psx_b200_lm_head_sample_rows.argtypes = [ptr, ptr, ptr, i64, i64, ptr, i64, C.c_int32, ptr, ptr, ptr, ptr, ptr, ptr,
                                                     ptr, ptr]
        lib.psx_b200_softmax_rows.argtypes = [ptr, ptr, ptr, ptr, C.c_size_t, C.c_size_t]
        lib.psx_b200_logsumexp_rows.argtypes = [ptr, ptr, ptr, ptr, C.c_size_t, C.c_size_t]
        lib.psx_b200_gather_rows.argtypes = [ptr, ptr, ptr, ptr, ptr, C.c_size_t, C.c_size_t]
        lib.psx_b200_decode_attention.argtypes = [ptr, ptr, ptr, ptr, ptr, ptr, ptr, i64, i64, i64, i64, i64, i64, i64, C.c_float, C.c_int32,
                                                  i64, ptr]
        lib.psx_uniforms_mt19937_64.argtypes = [ptr, i64, ptr]
        lib.psx_uniforms_portable.argtypes = [ptr, i64, ptr]
        _lib = lib
    return _lib


def _check(status):
    if status != OK:
        raise PsxError(status, library().psx_b200_last_error().decode())


def uniforms_mt19937_64(seeds) -> np.ndarray:
    """(std::mt19937_64(seed)() >> 11) * 2^-53 per seed: Generate()'s first draw."""
    seeds = np.ascontiguousarray(seeds, dtype=np.uint64)
    out = np.zeros(seeds.size, dtype=np.float64)
    library().psx_uniforms_mt19937_64(seeds.ctypes.data, seeds.size, out.ctypes.data)
    return out


def uniforms_portable(seeds) -> np.ndarray:
    seeds = np.ascontiguousarray(seeds, dtype=np.uint64)
    out = np.zeros(seeds.size, dtype=np.float64)
    library().psx_uniforms_portable(seeds.ctypes.data, seeds.size, out.ctypes.data)
    return out


def _dptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def read_only_pass(tensor, sink, stream=None):
    """Launches the read-only kernel over a contiguous cuda tensor (benchmark aid)."""
    if stream is None:
        import torch
        stream = torch.cuda.current_stream(tensor.device).cuda_stream
    _check(library().psx_b200_read_only_pass(C.c_void_p(stream), _dptr(tensor), tensor.numel() * tensor.element_size(),
                                             _dptr(sink)))


def sample_rows_static(logits, history_ids, history_offsets, config, uniforms, tokens, log_probs, status, stream=None,
                       vocab=None):
    """psx_b200_sample_rows_static: the sampling step without a context and without any device
    allocation (its scratch is a fixed array inside the library).  All tensors are the caller's:
    cuda inputs as for Context.sample_rows, and preallocated cuda outputs tokens (int64),
    log_probs (float32), status (int32).  Asynchronous on `stream` (default: torch's current)."""
    rows = logits.shape[0]
    vocab = logits.shape[1] if vocab is None else vocab
    if stream is None:
        import torch
        stream = torch.cuda.current_stream(logits.device).cuda_stream
    _check(library().psx_b200_sample_rows_static(
        C.c_void_p(stream), _dptr(logits), rows, vocab, logits.stride(0) if rows else vocab, _dptr(history_ids),
        _dptr(history_offsets), C.addressof(config), _dptr(uniforms), _dptr(tokens), _dptr(log_probs), _dptr(status)))


class Context:
    """A psx_ctx on one CUDA device."""

    def __init__(self, device: int = 0):
        self._lib = library()
        self._ctx = C.c_void_p()
        _check(self._lib.psx_b200_ctx_create(C.c_int(device), C.byref(self._ctx)))
        self.device = device

    def close(self):
        if self._ctx:
            self._lib.psx_b200_ctx_destroy(self._ctx)
            self._ctx = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def launches(self) -> int:
        return int(self._lib.psx_b200_launch_count(self._ctx))

    @property
    def stream(self) -> int:
        return int(self._lib.psx_b200_ctx_stream(self._ctx) or 0)

    def inputs_are_ready(self, ready=True):
        """Promise that the inputs of the calls that follow are complete before each call is made
        (see psx_b200_ctx_inputs_are_ready): the row pass then overlaps the kernel before it."""
        _check(self._lib.psx_b200_ctx_inputs_are_ready(self._ctx, int(ready)))

    def set_wait_limit(self, nanoseconds):
        """How long a kernel waits for one of its own copies before the row reports ROW_DEVICE_TIMEOUT."""
        _check(self._lib.psx_b200_ctx_set_wait_limit(self._ctx, int(nanoseconds)))

    def test_short_copy(self, on=True):
        """Test hook (psx_b200_test_short_copy): the row pass's waits for its chunks run out."""
        _check(self._lib.psx_b200_test_short_copy(self._ctx, int(on)))

    def enable_timing(self, on=True):
        _check(self._lib.psx_b200_ctx_enable_timing(self._ctx, int(on)))

    def read_timing(self):
        """(row-pass ms, survivor-stage ms, calls) summed over the calls since the last read."""
        scan, merge, calls = C.c_double(0), C.c_double(0), C.c_uint64(0)
        _check(self._lib.psx_b200_ctx_read_timing(self._ctx, C.addressof(scan), C.addressof(merge),
                                                  C.addressof(calls)))
        return scan.value, merge.value, calls.value

    def sync(self, stream=None):
        _check(self._lib.psx_b200_sync(self._ctx, C.c_void_p(stream) if stream else None))

    # ---- device-resident sampling ------------------------------------------------------------------
    def alloc_outputs(self, rows, with_diag=True):
        import torch
        dev = torch.device("cuda", self.device)
        out = {
            "tokens": torch.empty(rows, dtype=torch.int64, device=dev),
            "log_probs": torch.empty(rows, dtype=torch.float32, device=dev),
            "status": torch.empty(rows, dtype=torch.int32, device=dev),
            "diag": torch.empty(rows * C.sizeof(RowDiag), dtype=torch.uint8, device=dev) if with_diag else None,
        }
        return out

    def sample_rows(self, logits, history_ids, history_offsets, config, uniforms, out=None, stream=None, vocab=None):
        """logits: cuda float32 (rows, >=vocab) with unit column stride; history/uniforms: cuda
        tensors (int64 / float64) or None.  Asynchronous; returns the dict of output tensors."""
        rows = logits.shape[0]
        vocab = logits.shape[1] if vocab is None else vocab
        assert logits.stride(1) == 1 or rows == 0
        out = out or self.alloc_outputs(rows)
        if stream is None:
            import torch
            stream = torch.cuda.current_stream(logits.device).cuda_stream
        _check(self._lib.psx_b200_sample_rows(
            self._ctx, C.c_void_p(stream), _dptr(logits), rows, vocab, logits.stride(0) if rows else vocab,
            _dptr(history_ids), _dptr(history_offsets), C.addressof(config), _dptr(uniforms), _dptr(out["tokens"]),
            _dptr(out["log_probs"]), _dptr(out["status"]), _dptr(out["diag"])))
        return out

    def bind_sample_rows(self, logits, history_ids, history_offsets, config, uniforms, out=None, stream=None,
                         vocab=None):
        """sample_rows with its arguments converted once: returns a function of no arguments that
        enqueues the same call again (same buffers, same stream) and returns the output dict.  For
        loops over fixed buffers, where building the argument list costs as much as the launches."""
        rows = logits.shape[0]
        vocab = logits.shape[1] if vocab is None else vocab
        assert logits.stride(1) == 1 or rows == 0
        out = out or self.alloc_outputs(rows)
        if stream is None:
            import torch
            stream = torch.cuda.current_stream(logits.device).cuda_stream
        args = (self._ctx, C.c_void_p(stream), _dptr(logits), C.c_int64(rows), C.c_int64(vocab),
                C.c_int64(logits.stride(0) if rows else vocab), _dptr(history_ids), _dptr(history_offsets),
                C.c_void_p(C.addressof(config)), _dptr(uniforms), _dptr(out["tokens"]), _dptr(out["log_probs"]),
                _dptr(out["status"]), _dptr(out["diag"]))
        fn = self._lib.psx_b200_sample_rows
        keep = (logits, history_ids, history_offsets, config, uniforms, out)  # the buffers live as long as the call

        def call(fn=fn, args=args, out=out, keep=keep):
            status = fn(*args)
            if status:
                _check(status)
            return out
        return call

    def bind_row_pass_only(self, logits, history_ids, history_offsets, config, stream=None, vocab=None):
        """row_pass_only with its arguments converted once (see bind_sample_rows)."""
        rows = logits.shape[0]
        vocab = logits.shape[1] if vocab is None else vocab
        if stream is None:
            import torch
            stream = torch.cuda.current_stream(logits.device).cuda_stream
        args = (self._ctx, C.c_void_p(stream), _dptr(logits), C.c_int64(rows), C.c_int64(vocab),
                C.c_int64(logits.stride(0) if rows else vocab), _dptr(history_ids), _dptr(history_offsets),
                C.c_void_p(C.addressof(config)))
        fn = self._lib.psx_b200_row_pass_only
        keep = (logits, history_ids, history_offsets, config)

        def call(fn=fn, args=args, keep=keep):
            status = fn(*args)
            if status:
                _check(status)
        return call

    def process_logits_host(self, logits, history_ids, history_offsets, config):
        """ProcessLogits on host rows (numpy float32 (rows, vocab), modified in place).  Returns the
        per-row status array; raises when the device path declines a row."""
        rows, vocab = logits.shape
        status = np.zeros(rows, dtype=np.int32)

        def hptr(a):
            return None if a is None else C.c_void_p(a.ctypes.data)

        _check(self._lib.psx_b200_process_logits_host(self._ctx, hptr(logits), rows, vocab, logits.strides[0] // 4,
                                                      hptr(history_ids), hptr(history_offsets), C.addressof(config),
                                                      hptr(status)))
        return status

    def row_pass_only(self, logits, history_ids, history_offsets, config, stream=None, vocab=None):
        """Launches only the kernel that reads the logits (for timing and profiling)."""
        rows = logits.shape[0]
        vocab = logits.shape[1] if vocab is None else vocab
        if stream is None:
            import torch
            stream = torch.cuda.current_stream(logits.device).cuda_stream
        _check(self._lib.psx_b200_row_pass_only(self._ctx, C.c_void_p(stream), _dptr(logits), rows, vocab,
                                                logits.stride(0) if rows else vocab, _dptr(history_ids),
                                                _dptr(history_offsets), C.addressof(config)))

    @staticmethod
    def diag_to_numpy(diag_tensor):
        return diag_tensor.cpu().numpy().view(ROW_DIAG_DTYPE)

    # ---- host-resident sampling (the reference-facing call) ---------------------------------------
    def sample_rows_host(self, logits, history_ids, history_offsets, config, uniforms, row_stride=None, vocab=None,
                         raise_on_row_failure=True):
        """numpy (or pinned torch CPU) inputs; returns (tokens, log_probs, status, diag) as numpy."""
        rows = logits.shape[0]
        vocab = logits.shape[1] if vocab is None else vocab
        row_stride = (logits.strides[0] // 4 if hasattr(logits, "strides") else logits.stride(0)) \
            if row_stride is None else row_stride
        tokens = np.zeros(rows, dtype=np.int64)
        logp = np.zeros(rows, dtype=np.float32)
        status = np.zeros(rows, dtype=np.int32)
        diag = np.zeros(rows, dtype=ROW_DIAG_DTYPE)

        def hptr(a):
            if a is None:
                return None
            return C.c_void_p(a.ctypes.data if hasattr(a, "ctypes") else a.data_ptr())

        rc = self._lib.psx_b200_sample_rows_host(self._ctx, hptr(logits), rows, vocab, row_stride, hptr(history_ids),
                                                 hptr(history_offsets), C.addressof(config), hptr(uniforms),
                                                 hptr(tokens), hptr(logp), hptr(status), hptr(diag))
        if rc != OK and (rc != ERR_ROW_FAILED or raise_on_row_failure):
            _check(rc)
        return tokens, logp, status, diag

    # ---- top-k ---------------------------------------------------------------------------------------
    def top_k_rows(self, x, k, largest=True, stream=None):
        """x: cuda float32 contiguous (rows, cols).  Returns (values, indices) cuda float32 (rows, k)."""
        import torch
        rows, cols = x.shape
        values = torch.empty((rows, max(k, 0)), dtype=torch.float32, device=x.device)
        indices = torch.empty((rows, max(k, 0)), dtype=torch.float32, device=x.device)
        if stream is None:
            stream = torch.cuda.current_stream(x.device).cuda_stream
        _check(self._lib.psx_b200_top_k_rows(self._ctx, C.c_void_p(stream), _dptr(x), _dptr(values), _dptr(indices),
                                             rows, cols, k if k >= 0 else 0, int(largest)))
        return values, indices

    # ---- the language-model head -------------------------------------------------------------------------
    def lm_head_logits(self, hidden, weight, vocab_by_d=True, out=None, stream=None):
        """hidden: cuda float32 (rows, d); weight: (vocab, d) when vocab_by_d else (d, vocab).  Returns (rows, vocab)."""
        import torch
        rows, d = hidden.shape
        vocab = weight.shape[0] if vocab_by_d else weight.shape[1]
        out = torch.empty((rows, vocab), dtype=torch.float32, device=hidden.device) if out is None else out
        if stream is None:
            stream = torch.cuda.current_stream(hidden.device).cuda_stream
        _check(self._lib.psx_b200_lm_head_logits(self._ctx, C.c_void_p(stream), _dptr(hidden), rows, d, _dptr(weight), vocab,
                                                 0 if vocab_by_d else 1, _dptr(out), out.stride(0)))
        return out

    def lm_head_sample_rows(self, hidden, weight, history_ids, history_offsets, config, uniforms, vocab_by_d=True, out=None,
                            stream=None):
        """The head and the sampling step in one call: the logits stay in the context's scratch."""
        import torch
        rows, d = hidden.shape
        vocab = weight.shape[0] if vocab_by_d else weight.shape[1]
        out = out or self.alloc_outputs(rows)
        if stream is None:
            stream = torch.cuda.current_stream(hidden.device).cuda_stream
        _check(self._lib.psx_b200_lm_head_sample_rows(
            self._ctx, C.c_void_p(stream), _dptr(hidden), rows, d, _dptr(weight), vocab, 0 if vocab_by_d else 1,
            _dptr(history_ids), _dptr(history_offsets), C.addressof(config), _dptr(uniforms), _dptr(out["tokens"]),
            _dptr(out["log_probs"]), _dptr(out["status"]), _dptr(out["diag"])))
        return out

    # ---- row primitives ---------------------------------------------------------------------------------
    def softmax_rows(self, x, out=None, stream=None):
        """x: cuda float32 contiguous (rows, cols); out may be x itself."""
        import torch
        out = torch.empty_like(x) if out is None else out
        if stream is None:
            stream = torch.cuda.current_stream(x.device).cuda_stream
        _check(self._lib.psx_b200_softmax_rows(self._ctx, C.c_void_p(stream), _dptr(x), _dptr(out), x.shape[0], x.shape[1]))
        return out

    def logsumexp_rows(self, x, stream=None):
        import torch
        out = torch.empty(x.shape[0], dtype=torch.float32, device=x.device)
        if stream is None:
            stream = torch.cuda.current_stream(x.device).cuda_stream
        _check(self._lib.psx_b200_logsumexp_rows(self._ctx, C.c_void_p(stream), _dptr(x), _dptr(out), x.shape[0], x.shape[1]))
        return out

    def gather_rows(self, table, indices, stream=None):
        """table: cuda float32 (n, dim); indices: cuda float32 whole numbers (count,)."""
        import torch
        out = torch.empty((indices.shape[0], table.shape[1]), dtype=torch.float32, device=table.device)
        if stream is None:
            stream = torch.cuda.current_stream(table.device).cuda_stream
        _check(self._lib.psx_b200_gather_rows(self._ctx, C.c_void_p(stream), _dptr(table), _dptr(indices), _dptr(out),
                                              indices.shape[0], table.shape[1]))
        return out

    def decode_attention(self, q, keys, values, cached, scale=None, causal=True, window=0, key_keep=None, stream=None):
        """Attention of the new positions over the KV cache (psx_b200_decode_attention).  q: cuda float32
        (batch, heads, q_len, head_dim); keys / values: the cache, (batch, kv_heads, max_len, head_dim), with
        positions 0 .. cached + q_len - 1 filled; key_keep: (batch, cached + q_len) or None.  Returns the
        context, (batch, heads, q_len, head_dim), and a one-element int32 status tensor."""
        import torch
        batch, heads, q_len, head_dim = q.shape
        kv_heads, max_len = keys.shape[1], keys.shape[2]
        if scale is None:
            scale = 1.0 / float(np.sqrt(np.float32(head_dim)))
        context = torch.empty_like(q)
        status = torch.zeros(1, dtype=torch.int32, device=q.device)
        if stream is None:
            stream = torch.cuda.current_stream(q.device).cuda_stream
        _check(self._lib.psx_b200_decode_attention(self._ctx, C.c_void_p(stream), _dptr(q), _dptr(keys), _dptr(values),
                                                   _dptr(key_keep) if key_keep is not None else None, _dptr(context), batch, heads,
                                                   kv_heads, q_len, head_dim, cached, max_len, C.c_float(scale), int(bool(causal)),
                                                   window, _dptr(status)))
        return context, status

    # ---- vocabulary-sharded -----------------------------------------------------------------------------
    def shard_record_bytes(self, config) -> int:
        return int(self._lib.psx_b200_shard_record_bytes(C.addressof(config)))

    def shard_scan(self, shard_logits, shard_begin, vocab, history_ids, history_offsets, config, records, stream=None):
        import torch
        rows, cols = shard_logits.shape
        if stream is None:
            stream = torch.cuda.current_stream(shard_logits.device).cuda_stream
        _check(self._lib.psx_b200_shard_scan(self._ctx, C.c_void_p(stream), _dptr(shard_logits), rows, cols,
                                             shard_logits.stride(0), shard_begin, vocab, _dptr(history_ids),
                                             _dptr(history_offsets), C.addressof(config), _dptr(records)))

    def shard_merge(self, gathered, num_shards, rows, vocab, config, uniforms, out=None, stream=None, row_begin=0,
                    row_count=None):
        """Merges rows row_begin .. row_begin + row_count - 1 (all of them by default); `out` holds
        the merged rows only, the first of them at index 0."""
        import torch
        row_count = rows - row_begin if row_count is None else row_count
        out = out or self.alloc_outputs(row_count)
        if stream is None:
            stream = torch.cuda.current_stream(gathered.device).cuda_stream
        _check(self._lib.psx_b200_shard_merge_rows(self._ctx, C.c_void_p(stream), _dptr(gathered), num_shards, rows,
                                                   row_begin, row_count, vocab, C.addressof(config), _dptr(uniforms),
                                                   _dptr(out["tokens"]), _dptr(out["log_probs"]), _dptr(out["status"]),
                                                   _dptr(out.get("diag"))))
        return out

    def exchange(self, world, rank, rows, config):
        """This rank's end of a vocabulary-sharded exchange over peer memory (psx_b200_exchange_*)."""
        return Exchange(self, world, rank, rows, config)


class _DeviceBytes:
    """Device memory that the library owns, as something torch.as_tensor can wrap without a copy."""

    def __init__(self, address, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (address, False), "version": 2}


class Exchange:
    """One rank's end of the vocabulary-sharded step over peer memory (include/psx_b200.h:
    psx_b200_exchange_*).  `handle` (bytes) goes to every rank; open() takes all ranks' handles in
    rank order; sample() is one step; results() are views of the library's own buffer:
    {"tokens", "log_probs", "status"} of shape (world, rows_per_rank), rank r's rows in row r."""

    def __init__(self, ctx, world, rank, rows, config):
        self._lib, self._context = ctx._lib, ctx
        self.world, self.rank, self.rows = world, rank, rows
        self._ex = C.c_void_p()
        handle = C.create_string_buffer(int(self._lib.psx_b200_exchange_handle_bytes()))
        _check(self._lib.psx_b200_exchange_create(ctx._ctx, world, rank, rows, C.addressof(config), C.byref(self._ex), handle))
        self.handle = handle.raw
        self._views = None

    def open(self, handles: bytes):
        if len(handles) != self.world * len(self.handle):
            raise ValueError("open() takes the handles of all ranks, back to back in rank order")
        _check(self._lib.psx_b200_exchange_open(self._ex, handles))

    def sample(self, shard_logits, shard_begin, vocab, history_ids, history_offsets, config, uniforms, stream=None):
        import torch
        rows, cols = shard_logits.shape
        if rows != self.rows:
            raise ValueError(f"the exchange was created for {self.rows} rows, got {rows}")
        if stream is None:
            stream = torch.cuda.current_stream(shard_logits.device).cuda_stream
        _check(self._lib.psx_b200_exchange_sample(self._ex, C.c_void_p(stream), _dptr(shard_logits), cols,
                                                  shard_logits.stride(0), shard_begin, vocab, _dptr(history_ids),
                                                  _dptr(history_offsets), C.addressof(config), _dptr(uniforms)))
        return self.results(shard_logits.device)

    def results(self, device):
        """Views of the last step's results (the library keeps two sets and alternates: a step's results
        stay in place until the step after the next one)."""
        import torch
        address, per = C.c_void_p(), C.c_int64()
        _check(self._lib.psx_b200_exchange_results(self._ex, C.byref(address), C.byref(per)))
        if self._views is None:
            self._views = {}
        if address.value not in self._views:
            per = per.value
            raw = torch.as_tensor(_DeviceBytes(address.value, self.world * 16 * per), device=device)
            by_rank = raw.view(self.world, 16 * per)
            self._views[address.value] = {"tokens": by_rank[:, : 8 * per].view(torch.int64),
                                          "log_probs": by_rank[:, 8 * per: 12 * per].view(torch.float32),
                                          "status": by_rank[:, 12 * per:].view(torch.int32)}
        return self._views[address.value]

    def test_wait(self, wait_limit_ns, extra_arrivals):
        _check(self._lib.psx_b200_exchange_test_wait(self._ex, wait_limit_ns, extra_arrivals))

    def close(self):
        """Unmaps and frees.  Across ranks: only after a barrier, so that no rank is still inside a step."""
        if self._ex:
            self._views = None
            self._lib.psx_b200_exchange_destroy(self._ex)
            self._ex = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
