"""ctypes wrapper of the CPU oracle (TEST INFRASTRUCTURE - see oracle.cpp's header).

Only the test suite, the smoke check and the benchmark's CPU-baseline leg import this module.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB = HERE / "liboracle.so"
MODELGEN = HERE / "libmodelgen.so"

T_F32, T_F16, T_Q8_0, T_Q4_K, T_BF16, T_MXFP4 = 0, 1, 8, 12, 30, 39


def build(force: bool = False) -> Path:
    """Compiles the oracle and the host-only model writer when a source is newer than its library."""
    src = HERE / "oracle.cpp"
    if force or not LIB.exists() or LIB.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), "-B", "liboracle.so"], check=True, capture_output=True)
    _build_modelgen(force)
    return LIB


def _build_modelgen(force: bool = False) -> Path:
    sources = [HERE / "modelgen.cpp", HERE.parent / "retrograd_b200" / "csrc" / "synth.cpp", HERE.parent / "retrograd_b200" / "csrc" / "blocks.hpp"]
    if force or not MODELGEN.exists() or MODELGEN.stat().st_mtime < max(s.stat().st_mtime for s in sources):
        subprocess.run(["make", "-C", str(HERE), "-B", "libmodelgen.so"], check=True, capture_output=True)
    return MODELGEN


def synth_gguf(path, **spec) -> int:
    """Writes the seeded synthetic model `spec` describes (the keys of the GPU library's retro_b200_synth_gguf)
    without loading the GPU library: the same writer, compiled into a host-only helper."""
    gen = C.CDLL(str(_build_modelgen()))
    gen.ora_modelgen_last_error.restype = C.c_char_p
    gen.ora_synth_gguf.argtypes = [C.c_char_p, C.c_char_p, C.POINTER(C.c_uint64)]
    n = C.c_uint64()
    text = " ".join(f"{k}={v}" for k, v in spec.items())
    if gen.ora_synth_gguf(str(path).encode(), text.encode(), C.byref(n)) != 0:
        raise RuntimeError(gen.ora_modelgen_last_error().decode())
    return n.value


def threads(n: int = 0) -> int:
    """Sets (n > 0) and returns the OpenMP thread count of the forward pass."""
    return lib().ora_threads(n)


_lib = None
_P = C.POINTER


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        l = C.CDLL(str(LIB))
        l.ora_last_error.restype = C.c_char_p
        l.ora_threads.restype = C.c_int
        l.ora_threads.argtypes = [C.c_int]
        l.ora_model_load.restype = C.c_void_p
        l.ora_model_load.argtypes = [C.c_char_p]
        l.ora_model_free.argtypes = [C.c_void_p]
        l.ora_model_set_fast.argtypes = [C.c_void_p, C.c_int]
        l.ora_model_set_act_q8.argtypes = [C.c_void_p, C.c_int]
        l.ora_model_info.argtypes = [C.c_void_p, _P(C.c_uint32)]
        l.ora_lora_load.restype = C.c_int32
        l.ora_lora_load.argtypes = [C.c_void_p, C.c_char_p, C.c_float]
        l.ora_ctx_new.restype = C.c_void_p
        l.ora_ctx_new.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_int]
        l.ora_ctx_free.argtypes = [C.c_void_p]
        l.ora_kv_round.restype = None
        l.ora_kv_round.argtypes = [C.c_int, _P(C.c_float), _P(C.c_float), C.c_uint64]
        l.ora_step.argtypes = [C.c_void_p, C.c_size_t, _P(C.c_int32), _P(C.c_uint32), _P(C.c_int32), _P(C.c_uint8), _P(C.c_int32), _P(C.c_int32), _P(C.c_float)]
        l.ora_pack.restype = C.c_size_t
        l.ora_pack.argtypes = [C.c_size_t, _P(C.c_int32), _P(C.c_uint32), _P(C.c_int32), _P(C.c_uint8)] + [_P(C.c_int32)] * 5 + [_P(C.c_size_t)]
        l.ora_last_route_margins.restype = C.c_size_t
        l.ora_last_route_margins.argtypes = [C.c_void_p, _P(C.c_float), C.c_size_t]
        l.ora_last_routes.restype = C.c_size_t
        l.ora_last_routes.argtypes = [C.c_void_p, _P(C.c_int32), C.c_size_t]
        l.ora_seq_pos.argtypes = [C.c_void_p, C.c_int32, _P(C.c_int32), _P(C.c_int32)]
        l.ora_seq_rm.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_int32]
        l.ora_seq_cp.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32]
        l.ora_dequantize_row.argtypes = [C.c_uint32, C.c_void_p, C.c_size_t, _P(C.c_float)]
        l.ora_mul_mat_vec.argtypes = [C.c_uint32, C.c_size_t, C.c_size_t, C.c_void_p, _P(C.c_float), _P(C.c_float)]
        l.ora_mul_mat_vec_act_q8.argtypes = [C.c_uint32, C.c_size_t, C.c_size_t, C.c_void_p, _P(C.c_float), _P(C.c_float)]
        l.ora_rms_norm.argtypes = [_P(C.c_float), _P(C.c_float), C.c_size_t, C.c_float, _P(C.c_float)]
        l.ora_half_to_f32.restype = C.c_float
        l.ora_half_to_f32.argtypes = [C.c_uint16]
        l.ora_round_to_half.restype = C.c_float
        l.ora_round_to_half.argtypes = [C.c_float]
        l.ora_e8m0_half.restype = C.c_float
        l.ora_e8m0_half.argtypes = [C.c_uint8]
        l.ora_rng_new.restype = C.c_void_p
        l.ora_rng_new.argtypes = [C.c_uint32]
        l.ora_rng_free.argtypes = [C.c_void_p]
        l.ora_log_softmax_terms.argtypes = [_P(C.c_float), C.c_size_t, _P(C.c_float), _P(C.c_double)]
        l.ora_sample_token.restype = C.c_int32
        l.ora_sample_token.argtypes = [_P(C.c_float), C.c_size_t, C.c_float, C.c_float, C.c_void_p, _P(C.c_float)]
        l.ora_top_token_logprobs.argtypes = [_P(C.c_float), C.c_size_t, C.c_size_t, _P(C.c_int32), _P(C.c_float)]
        l.ora_sample_token_v2.restype = C.c_int32
        l.ora_sample_token_v2.argtypes = [
            _P(C.c_float), C.c_size_t, C.c_float, C.c_float, C.c_int32, C.c_float, C.c_float, C.c_float, C.c_float, C.c_uint32,
            C.c_uint32, _P(C.c_int32), _P(C.c_float), C.c_void_p, _P(C.c_int32), C.c_size_t, _P(C.c_float), _P(C.c_float),
            _P(C.c_int32), _P(C.c_float), C.c_size_t,
        ]
        l.ora_philox_uniform.restype = C.c_double
        l.ora_philox_uniform.argtypes = [C.c_uint32, C.c_uint64]
        l.ora_sample_philox.restype = C.c_int32
        l.ora_sample_philox.argtypes = [_P(C.c_float), C.c_size_t, C.c_float, C.c_float, C.c_uint32, C.c_uint64, _P(C.c_double)]
        _lib = l
    return _lib


def _f32(a):
    return a.ctypes.data_as(_P(C.c_float))


def _i32(a):
    return a.ctypes.data_as(_P(C.c_int32))


def dequantize_row(ggml_type: int, raw: bytes | np.ndarray, n: int) -> np.ndarray:
    buf = np.frombuffer(raw, dtype=np.uint8) if not isinstance(raw, np.ndarray) else raw
    buf = np.ascontiguousarray(buf)
    out = np.zeros(n, dtype=np.float32)
    if lib().ora_dequantize_row(ggml_type, buf.ctypes.data, n, _f32(out)) != 0:
        raise ValueError("dequantize_row refused the input (unknown type or partial block)")
    return out


def mul_mat_vec(ggml_type: int, a: np.ndarray, n_row: int, n_col: int, b: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b, dtype=np.float32)
    out = np.zeros(n_row, dtype=np.float32)
    if lib().ora_mul_mat_vec(ggml_type, n_row, n_col, a.ctypes.data, _f32(b), _f32(out)) != 0:
        raise ValueError("mul_mat_vec refused the input")
    return out


def mul_mat_vec_act_q8(ggml_type: int, a: np.ndarray, n_row: int, n_col: int, b: np.ndarray) -> np.ndarray:
    """The GEMV with b re-quantised to the weight type's 8-bit dot format (integer products, per-block scales)."""
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b, dtype=np.float32)
    out = np.zeros(n_row, dtype=np.float32)
    if lib().ora_mul_mat_vec_act_q8(ggml_type, n_row, n_col, a.ctypes.data, _f32(b), _f32(out)) != 0:
        raise ValueError("mul_mat_vec_act_q8 refused the input")
    return out


def rms_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    y = np.zeros_like(x)
    lib().ora_rms_norm(_f32(x), _f32(w), x.size, eps, _f32(y))
    return y


def pack(rows):
    """rows: iterable of (slot, n, pos0, sample). Returns the reference-order batch maps."""
    rows = list(rows)
    R = len(rows)
    slot = np.array([r[0] for r in rows], dtype=np.int32)
    n = np.array([r[1] for r in rows], dtype=np.uint32)
    pos0 = np.array([r[2] for r in rows], dtype=np.int32)
    sample = np.array([1 if r[3] else 0 for r in rows], dtype=np.uint8)
    T = int(n.sum())
    ts, tp, tr = (np.zeros(max(T, 1), dtype=np.int32) for _ in range(3))
    oi = np.zeros(max(R, 1), dtype=np.int32)
    cu = np.zeros(R + 1, dtype=np.int32)
    n_out = C.c_size_t()
    got = lib().ora_pack(R, _i32(slot), n.ctypes.data_as(_P(C.c_uint32)), _i32(pos0), sample.ctypes.data_as(_P(C.c_uint8)),
                         _i32(ts), _i32(tp), _i32(tr), _i32(oi), _i32(cu), C.byref(n_out))
    assert got == T
    return dict(tok_slot=ts[:T], tok_pos=tp[:T], tok_row=tr[:T], out_index=oi[: n_out.value], cu_rows=cu)


class Model:
    def __init__(self, path: str, fast: bool = False, act_q8: bool = False) -> None:
        """act_q8: the weight matmuls re-quantise activations to 8 bits and multiply integers, as the reference's CPU
        backend does (parity unpinned; reported beside the default act = f32, which every parity claim is made against)."""
        self._h = lib().ora_model_load(str(path).encode())
        if not self._h:
            raise RuntimeError(lib().ora_last_error().decode())
        info = (C.c_uint32 * 10)()
        lib().ora_model_info(self._h, info)
        (self.n_layer, self.d, self.n_head, self.n_head_kv, self.head_dim, self.ff, self.vocab, self.n_expert,
         self.n_expert_used, self.neox) = list(info)
        if fast:
            lib().ora_model_set_fast(self._h, 1)
        if act_q8:
            lib().ora_model_set_act_q8(self._h, 1)

    def lora_load(self, path: str, scale: float = 1.0) -> int:
        i = lib().ora_lora_load(self._h, str(path).encode(), scale)
        if i < 0:
            raise RuntimeError(lib().ora_last_error().decode())
        return i

    def close(self) -> None:
        if self._h:
            lib().ora_model_free(self._h)
            self._h = None


class Context:
    """Per-slot contiguous KV (deep copies on seq_cp): the independent check of the paged cache."""

    def __init__(self, model: Model, n_slots: int, n_ctx_seq: int, kv_f16: bool = True, kv_dtype: int | None = None) -> None:
        """kv_dtype: a retro_engine_kv_dtype value (0 F32, 1 F16, 2 Q8_0, 3 Q4_0); default F16 (or F32 with kv_f16=False)."""
        self.model = model
        if kv_dtype is None:
            kv_dtype = 1 if kv_f16 else 0
        self._h = lib().ora_ctx_new(model._h, n_slots, n_ctx_seq, int(kv_dtype))

    def step(self, rows) -> np.ndarray:
        """rows: iterable of (slot, tokens, pos0, sample[, adapter]). Returns logits [S, vocab]."""
        rows = list(rows)
        R = len(rows)
        slot = np.array([r[0] for r in rows], dtype=np.int32)
        n = np.array([len(r[1]) for r in rows], dtype=np.uint32)
        pos0 = np.array([r[2] for r in rows], dtype=np.int32)
        sample = np.array([1 if r[3] else 0 for r in rows], dtype=np.uint8)
        adapter = np.array([r[4] if len(r) > 4 else 0 for r in rows], dtype=np.int32)
        tokens = np.concatenate([np.asarray(r[1], dtype=np.int32) for r in rows])
        S = int(sample.sum())
        logits = np.zeros((max(S, 1), self.model.vocab), dtype=np.float32)
        status = lib().ora_step(self._h, R, _i32(slot), n.ctypes.data_as(_P(C.c_uint32)), _i32(pos0),
                                sample.ctypes.data_as(_P(C.c_uint8)), _i32(tokens), _i32(adapter), _f32(logits))
        if status != 0:
            raise RuntimeError(lib().ora_last_error().decode())
        return logits[:S]

    def last_route_margins(self) -> np.ndarray:
        """Per (layer, token) of the last step: the smallest gap between the routing probabilities that decided
        which experts were chosen and in which order (a gap near zero is a tie a float reordering may flip)."""
        n = lib().ora_last_route_margins(self._h, None, 0)
        out = np.zeros(n, dtype=np.float32)
        lib().ora_last_route_margins(self._h, out.ctypes.data_as(_P(C.c_float)), n)
        return out

    def last_routes(self) -> np.ndarray:
        n = lib().ora_last_routes(self._h, None, 0)
        out = np.zeros(max(n, 1), dtype=np.int32)
        lib().ora_last_routes(self._h, _i32(out), n)
        return out[:n]

    def seq_pos(self, slot: int):
        a, b = C.c_int32(), C.c_int32()
        lib().ora_seq_pos(self._h, slot, C.byref(a), C.byref(b))
        return a.value, b.value

    def seq_rm(self, slot: int, p0: int = -1, p1: int = -1) -> int:
        return lib().ora_seq_rm(self._h, slot, p0, p1)

    def seq_cp(self, src: int, dst: int, p0: int = -1, p1: int = -1) -> int:
        return lib().ora_seq_cp(self._h, src, dst, p0, p1)

    def close(self) -> None:
        if self._h:
            lib().ora_ctx_free(self._h)
            self._h = None


class Rng:
    """std::mt19937 seeded once per request, as the reference's step keeps it."""

    def __init__(self, seed: int) -> None:
        self._h = lib().ora_rng_new(seed)

    def __del__(self) -> None:
        if getattr(self, "_h", None):
            lib().ora_rng_free(self._h)
            self._h = None


def log_softmax_terms(logits: np.ndarray):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    mx, ls = C.c_float(), C.c_double()
    lib().ora_log_softmax_terms(_f32(logits), logits.size, C.byref(mx), C.byref(ls))
    return mx.value, ls.value


def kv_round(kv_dtype: int, row: np.ndarray) -> np.ndarray:
    """What a cache of `kv_dtype` (retro_engine_kv_dtype: 0 F32, 1 F16, 2 Q8_0, 3 Q4_0) returns for a stored row."""
    row = np.ascontiguousarray(row, dtype=np.float32)
    out = np.empty_like(row)
    lib().ora_kv_round(int(kv_dtype), _f32(row), _f32(out), row.size)
    return out


def token_logprob(logits: np.ndarray, token: int) -> np.float32:
    mx, ls = log_softmax_terms(logits)
    return np.float32(float(logits[token]) - mx - ls)


def sample_token(logits: np.ndarray, temperature: float, top_p: float, rng: Rng):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    lp = C.c_float()
    tok = lib().ora_sample_token(_f32(logits), logits.size, temperature, top_p, rng._h, C.byref(lp))
    return tok, lp.value


def top_token_logprobs(logits: np.ndarray, k: int):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    ids = np.zeros(k, dtype=np.int32)
    lps = np.zeros(k, dtype=np.float32)
    lib().ora_top_token_logprobs(_f32(logits), logits.size, k, _i32(ids), _f32(lps))
    return ids, lps


def sample_token_v2(logits, rng: Rng, temperature=1.0, top_p=1.0, top_k=0, min_p=0.0, repeat_penalty=1.0, frequency_penalty=0.0,
                    presence_penalty=0.0, penalty_window=0, logit_bias=(), history=(), k=0):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    bias_ids = np.array([b[0] for b in logit_bias], dtype=np.int32) if logit_bias else np.zeros(1, dtype=np.int32)
    bias_vals = np.array([b[1] for b in logit_bias], dtype=np.float32) if logit_bias else np.zeros(1, dtype=np.float32)
    hist = np.array(list(history), dtype=np.int32) if len(history) else np.zeros(1, dtype=np.int32)
    ids = np.zeros(max(k, 1), dtype=np.int32)
    lps = np.zeros(max(k, 1), dtype=np.float32)
    lp, slp = C.c_float(), C.c_float()
    tok = lib().ora_sample_token_v2(_f32(logits), logits.size, temperature, top_p, top_k, min_p, repeat_penalty, frequency_penalty,
                                    presence_penalty, penalty_window, len(logit_bias), _i32(bias_ids), _f32(bias_vals), rng._h,
                                    _i32(hist), len(history), C.byref(lp), C.byref(slp), _i32(ids), _f32(lps), k)
    return tok, lp.value, slp.value, ids[:k], lps[:k]


def philox_uniform(seed: int, draw: int) -> float:
    return lib().ora_philox_uniform(seed, draw)


def sample_philox(logits: np.ndarray, temperature: float, top_p: float, seed: int, draw: int):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    margin = C.c_double()
    tok = lib().ora_sample_philox(_f32(logits), logits.size, temperature, top_p, seed, draw, C.byref(margin))
    return tok, margin.value
