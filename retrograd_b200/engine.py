"""Host-side mirror of the reference's safe engine handle over libretro_b200's C ABI.

Names and semantics follow `retrograd_engine` (crates/retrograd-engine/src/step.rs:93-301,
412-505; crates/retrograd-engine/src/engine/step.rs:19-38; engine/mod.rs:57-102,151-208):
`StepRow.prefill / StepRow.decode`, `StepOutput` reused across steps and exposing no rows after a
failed call, status -3 mapped to `InvalidArgument`, every other failure to `EngineError`.
"""
from __future__ import annotations

import ctypes as C
import time
from dataclasses import dataclass, field
from typing import Iterable, Sequence

import numpy as np

from . import _ffi

ADAPTER_BASE = -1
KV_DTYPE_F32, KV_DTYPE_F16, KV_DTYPE_Q8_0, KV_DTYPE_Q4_0 = 0, 1, 2, 3
STATE_SEQ_FLAGS_NONE, STATE_SEQ_FLAGS_PARTIAL_ONLY, STATE_SEQ_FLAGS_ON_DEVICE = 0, 1, 2


class EngineError(RuntimeError):
    """A runtime failure reported by the library (status -1 or -2)."""


class InvalidArgument(EngineError):
    """A caller error reported before anything was decoded (status -3)."""


def _last_error() -> str:
    message = _ffi.load_library().retro_last_error()
    return message.decode("utf-8", "replace") if message else ""


def _check(status: int) -> None:
    if status == 0:
        return
    if status == -3:
        raise InvalidArgument(_last_error())
    raise EngineError(_last_error())


@dataclass
class SamplingParams:
    temperature: float = 1.0
    top_p: float = 1.0
    max_new_tokens: int = 1
    seed: int = 0


@dataclass
class SamplingParamsV2:
    temperature: float = 1.0
    top_p: float = 1.0
    max_new_tokens: int = 1
    seed: int = 0
    top_k: int = 0
    min_p: float = 0.0
    repeat_penalty: float = 1.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    penalty_window: int = 0
    logit_bias: Sequence[tuple[int, float]] = ()
    grammar: "Grammar | None" = None

    @classmethod
    def greedy(cls) -> "SamplingParamsV2":
        """Greedy decoding as the reference spells it: top_k = 1."""
        return cls(top_k=1)

    @classmethod
    def from_v1(cls, p: SamplingParams) -> "SamplingParamsV2":
        return cls(temperature=p.temperature, top_p=p.top_p, max_new_tokens=p.max_new_tokens, seed=p.seed)


class Grammar:
    """An owned GBNF text (`retro_grammar_from_gbnf`); rows that carry it sample only tokens the grammar can
    continue with. The handle may be dropped as soon as the step that carried it has returned."""

    def __init__(self, gbnf: str) -> None:
        self._lib = _ffi.load_library()
        self._h = self._lib.retro_grammar_from_gbnf(gbnf.encode())
        if not self._h:
            raise EngineError(_last_error())

    @classmethod
    def json_object(cls) -> "Grammar":
        g = cls.__new__(cls)
        g._lib = _ffi.load_library()
        g._h = g._lib.retro_grammar_json_object()
        return g

    def gbnf(self) -> str:
        return self._lib.retro_grammar_gbnf(self._h).decode()

    def __del__(self) -> None:  # pragma: no cover
        try:
            if self._h:
                self._lib.retro_grammar_free(self._h)
                self._h = None
        except Exception:
            pass


def grammar_check(gbnf: str, text: str) -> int:
    """0 = the grammar rejects `text`, 1 = a valid prefix, 2 = a complete match (host only)."""
    state = C.c_int()
    _check(_ffi.load_library().retro_b200_grammar_check(gbnf.encode(), text.encode(), C.byref(state)))
    return state.value


@dataclass
class StepRow:
    request: int
    slot: int
    tokens: Sequence[int]
    pos0: int
    sample: bool = False
    sampling: SamplingParamsV2 = field(default_factory=SamplingParamsV2)
    n_top_logprobs: int = 0
    want_logprob: bool = False
    adapter: int = 0  # 0 = the context's own adapter set, ADAPTER_BASE, or a loaded adapter id

    @classmethod
    def prefill(cls, request: int, slot: int, tokens: Sequence[int], pos0: int) -> "StepRow":
        return cls(request, slot, tokens, pos0, False)

    @classmethod
    def decode(cls, request: int, slot: int, token: int, pos0: int, sampling: SamplingParamsV2 | SamplingParams) -> "StepRow":
        if isinstance(sampling, SamplingParams):
            sampling = SamplingParamsV2.from_v1(sampling)
        return cls(request, slot, [token], pos0, True, sampling)


@dataclass
class StepOutRow:
    token: int = 0
    logprob: float = 0.0
    forced: bool = False
    sampled: bool = False
    n_top: int = 0
    sampled_logprob: float = 0.0


class StepOutput:
    """Reused output buffers of `Engine.step`; grown only when a call needs more."""

    def __init__(self, n_rows: int = 0, n_top_stride: int = 0) -> None:
        self._rows = (_ffi.StepOutRowV2C * max(n_rows, 1))()
        self._cap = max(n_rows, 1)
        self.n_top_stride = n_top_stride
        self._top_ids = np.zeros(self._cap * max(n_top_stride, 1), dtype=np.int32)
        self._top_logprobs = np.zeros(self._cap * max(n_top_stride, 1), dtype=np.float32)
        self.n_rows = 0

    def ensure(self, n_rows: int, n_top_stride: int) -> None:
        if n_rows > self._cap:
            self._rows = (_ffi.StepOutRowV2C * n_rows)()
            self._cap = n_rows
        self.n_top_stride = max(self.n_top_stride, n_top_stride)
        need = self._cap * max(self.n_top_stride, 1)
        if need > self._top_ids.size:
            self._top_ids = np.zeros(need, dtype=np.int32)
            self._top_logprobs = np.zeros(need, dtype=np.float32)

    def row(self, r: int) -> StepOutRow:
        if r >= self.n_rows:
            raise IndexError(r)
        o = self._rows[r]
        return StepOutRow(o.token, o.logprob, bool(o.forced), bool(o.sampled), o.n_top, o.sampled_logprob)

    def rows(self) -> list[StepOutRow]:
        return [self.row(r) for r in range(self.n_rows)]

    def top(self, r: int) -> tuple[np.ndarray, np.ndarray]:
        n = self._rows[r].n_top
        base = r * self.n_top_stride
        return self._top_ids[base : base + n].copy(), self._top_logprobs[base : base + n].copy()


@dataclass
class EngineConfig:
    n_ctx: int = 4096
    n_seq_max: int = 8
    n_batch: int = 512
    n_ubatch: int = 512
    kv_dtype: int = KV_DTYPE_F16
    flash_attn: bool = True
    device: int = 0
    threads: int = 0
    verbose: bool = False
    kv_unified: int = 1

    def to_c(self) -> _ffi.EngineConfigC:
        c = _ffi.EngineConfigC()
        c.struct_size = C.sizeof(_ffi.EngineConfigC)
        c.n_ctx, c.n_seq_max, c.n_batch, c.n_ubatch = self.n_ctx, self.n_seq_max, self.n_batch, self.n_ubatch
        c.kv_dtype, c.flash_attn, c.device, c.threads = self.kv_dtype, self.flash_attn, self.device, self.threads
        c.verbose, c.kv_unified = self.verbose, self.kv_unified
        c.expert_placement, c.expert_host_layers, c.expert_device_cache_bytes = 0, 0, 0
        return c


@dataclass
class EngineMemory:
    n_slots: int
    cells_total: int
    cells_used: int
    kv_bytes: int
    recurrent_bytes: int


def synth_gguf(path: str, **spec) -> int:
    """Writes a seeded random model as GGUF (see retro_b200_synth_gguf). Returns the file size."""
    lib = _ffi.load_library()
    text = " ".join(f"{k}={v}" for k, v in spec.items())
    n = C.c_uint64(0)
    _check(lib.retro_b200_synth_gguf(str(path).encode(), text.encode(), C.byref(n)))
    return n.value


def quantize_row(ggml_type: int, values) -> bytes:
    """One stored row of `ggml_type` from float values (the synthesiser's encoders)."""
    lib = _ffi.load_library()
    v = np.ascontiguousarray(values, dtype=np.float32)
    out = np.zeros(v.size * 4 + 64, dtype=np.uint8)
    n = C.c_size_t()
    _check(lib.retro_b200_quantize_row(ggml_type, v.ctypes.data_as(C.POINTER(C.c_float)), v.size, out.ctypes.data_as(C.POINTER(C.c_uint8)), out.size, C.byref(n)))
    return out[: n.value].tobytes()


def op_gemm(ggml_type: int, w_bytes, n_out: int, n_in: int, x, path: int = 0, iters: int = 0):
    """One dequant-fused GEMM through retro_b200_op_gemm. Returns (y [T, n_out], ms per launch)."""
    lib = _ffi.load_library()
    w = np.ascontiguousarray(np.frombuffer(w_bytes, dtype=np.uint8) if not isinstance(w_bytes, np.ndarray) else w_bytes)
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, n_in)
    y = np.zeros((x.shape[0], n_out), dtype=np.float32)
    ms = C.c_float()
    _check(lib.retro_b200_op_gemm(ggml_type, w.ctypes.data_as(C.POINTER(C.c_uint8)), n_out, n_in, x.ctypes.data_as(C.POINTER(C.c_float)),
                                  x.shape[0], y.ctypes.data_as(C.POINTER(C.c_float)), path, iters, C.byref(ms)))
    return y, ms.value


def op_gemm_mxfp4_grouped(banks, n_expert: int, n_out: int, n_in: int, x, offsets, iters: int = 0):
    """The grouped MXFP4 expert GEMM through retro_b200_op_gemm_mxfp4_grouped. Returns y [n_rows, n_out], or
    (y, ms per launch) when `iters` timed launches are asked for."""
    lib = _ffi.load_library()
    w = np.ascontiguousarray(np.frombuffer(banks, dtype=np.uint8) if not isinstance(banks, np.ndarray) else banks)
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, n_in)
    off = np.ascontiguousarray(offsets, dtype=np.int32)
    assert off.shape == (n_expert + 1,) and off[-1] == x.shape[0]
    y = np.zeros((x.shape[0], n_out), dtype=np.float32)
    ms = C.c_float()
    _check(lib.retro_b200_op_gemm_mxfp4_grouped(w.ctypes.data_as(C.POINTER(C.c_uint8)), n_expert, n_out, n_in, x.ctypes.data_as(C.POINTER(C.c_float)),
                                                off.ctypes.data_as(C.POINTER(C.c_int32)), y.ctypes.data_as(C.POINTER(C.c_float)), iters, C.byref(ms)))
    return (y, ms.value) if iters else y


def reasoning_check(start, ends, budget: int, n_prompt_tail: int, prompt, sampled, incomplete=()):
    """One request's reasoning-budget machine on the host (retro_b200_reasoning_check): returns (emitted tokens,
    forced flags) for the tokens a sampler drew after `prompt`."""
    lib = _ffi.load_library()
    arr = lambda v: (C.c_int32 * max(len(v), 1))(*v)
    tags = [arr(t) for t in ends]
    ptrs = (C.POINTER(C.c_int32) * max(len(tags), 1))(*[C.cast(t, C.POINTER(C.c_int32)) for t in tags])
    lens = (C.c_size_t * max(len(tags), 1))(*[len(t) for t in ends])
    out_t = (C.c_int32 * max(len(sampled), 1))()
    out_f = (C.c_uint8 * max(len(sampled), 1))()
    _check(lib.retro_b200_reasoning_check(arr(start), len(start), ptrs, lens, len(tags), budget, n_prompt_tail, arr(prompt), len(prompt),
                                          arr(incomplete), len(incomplete), arr(sampled), len(sampled), out_t, out_f))
    return list(out_t[: len(sampled)]), [bool(f) for f in out_f[: len(sampled)]]


def recode_mxfp4_as_q8_0(blocks: bytes) -> bytes | None:
    """MXFP4 blocks (17 B each) as Q8_0 blocks (34 B each) of the same values, as the engine does with expert
    banks at load; None when a block's scale is outside what an f16 holds. Host arithmetic only."""
    n = len(blocks) // 17
    src = C.create_string_buffer(bytes(blocks), len(blocks))
    dst = C.create_string_buffer(max(n * 34, 1))
    ok = C.c_int()
    _check(_ffi.load_library().retro_b200_recode_mxfp4_as_q8_0(src, n, dst, C.byref(ok)))
    return dst.raw[: n * 34] if ok.value else None


def nccl_unique_id() -> bytes:
    """The 128-byte NCCL id one rank creates and every rank passes to Engine.ep_init."""
    buf = C.create_string_buffer(128)
    _check(_ffi.load_library().retro_b200_nccl_unique_id(buf))
    return buf.raw


def ep_plan(all_offsets, rank: int):
    """The exchange plan of one MoE layer for `rank`, from every rank's per-expert pair offsets
    ([world, n_expert + 1], pairs sorted by expert). Host arithmetic only (no GPU needed). Returns a dict
    of int32 arrays: send_begin, send_count, recv_begin, recv_count (per peer), offsets [n_expert + 1]
    and sorted [n_recv] (rows of the receive buffer grouped by expert)."""
    lib = _ffi.load_library()
    off = np.ascontiguousarray(all_offsets, dtype=np.int32)
    world, n_expert = off.shape[0], off.shape[1] - 1
    per_peer = [np.zeros(world, dtype=np.int32) for _ in range(4)]
    offsets = np.zeros(n_expert + 1, dtype=np.int32)
    cap = int(off[:, -1].sum())
    sorted_rows = np.zeros(max(cap, 1), dtype=np.int32)
    n_recv = C.c_int32()
    ptr = lambda a: a.ctypes.data_as(C.POINTER(C.c_int32))
    _check(lib.retro_b200_ep_plan(ptr(off), world, rank, n_expert, *(ptr(a) for a in per_peer), ptr(offsets), ptr(sorted_rows), cap, C.byref(n_recv)))
    return dict(send_begin=per_peer[0], send_count=per_peer[1], recv_begin=per_peer[2], recv_count=per_peer[3], offsets=offsets,
                sorted=sorted_rows[: n_recv.value])


class Engine:
    def __init__(self, model_path: str, config: EngineConfig | None = None) -> None:
        self._lib = _ffi.load_library()
        self.config = config or EngineConfig()
        c = self.config.to_c()
        self._h = self._lib.retro_engine_new(str(model_path).encode(), C.byref(c))
        if not self._h:
            raise EngineError(_last_error())
        self._keep: list = []

    # entry points that exist for both handles: retro_engine_<name> here, retro_trainer_generation_<name> in TrainerGeneration
    _twin_prefix = "retro_engine_"

    def _twin(self, name: str):
        return getattr(self._lib, self._twin_prefix + name)

    def close(self) -> None:
        if self._h:
            self._lib.retro_engine_free(self._h)
            self._h = None

    def __del__(self) -> None:  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self) -> "Engine":
        return self

    def __exit__(self, *exc) -> None:
        self.close()

    # ---- introspection
    def vocab_size(self) -> int:
        v = C.c_uint32()
        _check(self._lib.retro_engine_vocab_size(self._h, C.byref(v)))
        return v.value

    def context_size(self) -> int:
        v = C.c_uint32()
        _check(self._lib.retro_engine_context_size(self._h, C.byref(v)))
        return v.value

    def eos_token(self) -> int:
        v = C.c_int32()
        _check(self._lib.retro_engine_eos_token(self._h, C.byref(v)))
        return v.value

    def is_eog_token(self, token: int) -> bool:
        v = C.c_bool()
        _check(self._lib.retro_engine_is_eog_token(self._h, token, C.byref(v)))
        return v.value

    def set_reasoning_tags(self, start: Sequence[int], ends: Sequence[Sequence[int]], n_prompt_tail: int) -> None:
        """The reasoning block's tags as token ids (from the caller's chat-template layer): the opening tag, the
        closing tags (the first is what a spent budget forces) and how much of a prompt's end primes a request."""
        s_arr = (C.c_int32 * max(len(start), 1))(*start)
        tags = [(C.c_int32 * max(len(t), 1))(*t) for t in ends]
        ptrs = (C.POINTER(C.c_int32) * max(len(tags), 1))(*[C.cast(t, C.POINTER(C.c_int32)) for t in tags])
        lens = (C.c_size_t * max(len(tags), 1))(*[len(t) for t in ends])
        name = "retro_b200_engine_set_reasoning_tags" if self._twin_prefix == "retro_engine_" else "retro_b200_trainer_set_reasoning_tags"
        _check(getattr(self._lib, name)(self._h, s_arr, len(start), ptrs, lens, len(tags), n_prompt_tail))

    def set_reasoning_budget(self, budget: int) -> None:
        name = "retro_engine_set_reasoning_budget" if self._twin_prefix == "retro_engine_" else "retro_trainer_set_reasoning_budget"
        _check(getattr(self._lib, name)(self._h, budget))

    def kv_unified(self) -> bool:
        v = C.c_bool()
        _check(self._twin("kv_unified")(self._h, C.byref(v)))
        return v.value

    def weights_version(self) -> int:
        v = C.c_uint64()
        _check(self._twin("weights_version")(self._h, C.byref(v)))
        return v.value

    def model_fingerprint(self) -> int:
        v = C.c_uint64()
        _check(self._lib.retro_engine_model_fingerprint(self._h, C.byref(v)))
        return v.value

    def is_hybrid(self) -> bool:
        v = C.c_bool()
        _check(self._lib.retro_engine_is_hybrid(self._h, C.byref(v)))
        return v.value

    def detokenize(self, tokens: Sequence[int], unparse_special: bool = False) -> bytes:
        arr = (C.c_int32 * len(tokens))(*tokens)
        n = C.c_size_t()
        _check(self._lib.retro_engine_detokenize(self._h, arr, len(tokens), unparse_special, None, 0, C.byref(n)))
        buf = C.create_string_buffer(max(n.value, 1))
        _check(self._lib.retro_engine_detokenize(self._h, arr, len(tokens), unparse_special, buf, n.value, C.byref(n)))
        return buf.raw[: n.value]

    def tokenize_text(self, text: str) -> list[int]:
        n = C.c_size_t()
        _check(self._lib.retro_engine_tokenize_text(self._h, text.encode(), None, 0, C.byref(n)))
        arr = (C.c_int32 * max(n.value, 1))()
        _check(self._lib.retro_engine_tokenize_text(self._h, text.encode(), arr, n.value, C.byref(n)))
        return list(arr[: n.value])

    # ---- the step
    def step(self, rows: Sequence[StepRow], out: StepOutput) -> None:
        out.n_rows = 0  # a failed call exposes nothing
        stride = max((r.n_top_logprobs for r in rows), default=0)
        out.ensure(len(rows), stride)
        n = len(rows)
        c_rows = (_ffi.StepRowV2C * max(n, 1))()
        keep = []
        for i, r in enumerate(rows):
            tokens = np.ascontiguousarray(r.tokens, dtype=np.int32)
            keep.append(tokens)
            if tokens.size < 1:
                raise InvalidArgument("a step row requires at least one token")
            if r.pos0 < 0:
                raise InvalidArgument("step row pos0 must be non-negative")
            if r.sample and r.request < 0:
                raise InvalidArgument("a sampling step row requires a request id")
            c = c_rows[i]
            c.struct_size = C.sizeof(_ffi.StepRowV2C)
            c.request, c.slot = r.request, r.slot
            c.tokens = tokens.ctypes.data_as(C.POINTER(C.c_int32))
            c.n, c.pos0, c.sample = tokens.size, r.pos0, r.sample
            s = r.sampling
            c.sampling.struct_size = C.sizeof(_ffi.SamplingParamsV2C)
            c.sampling.temperature, c.sampling.top_p = s.temperature, s.top_p
            c.sampling.max_new_tokens, c.sampling.seed = s.max_new_tokens, s.seed
            c.sampling.top_k, c.sampling.min_p = s.top_k, s.min_p
            c.sampling.repeat_penalty = s.repeat_penalty
            c.sampling.frequency_penalty, c.sampling.presence_penalty = s.frequency_penalty, s.presence_penalty
            c.sampling.penalty_window = s.penalty_window
            if len(s.logit_bias) > 4096:
                raise InvalidArgument("sampling n_logit_bias must not exceed 4096")
            if s.logit_bias:
                ids = np.ascontiguousarray([b[0] for b in s.logit_bias], dtype=np.int32)
                vals = np.ascontiguousarray([b[1] for b in s.logit_bias], dtype=np.float32)
                keep += [ids, vals]
                c.sampling.n_logit_bias = ids.size
                c.sampling.logit_bias_ids = ids.ctypes.data_as(C.POINTER(C.c_int32))
                c.sampling.logit_bias_values = vals.ctypes.data_as(C.POINTER(C.c_float))
            if s.grammar is not None:
                c.sampling.grammar = s.grammar._h
            c.n_top_logprobs, c.want_logprob, c.adapter = r.n_top_logprobs, int(r.want_logprob), r.adapter
        requests = [r.request for r in rows if r.request >= 0]
        if len(requests) != len(set(requests)):
            raise InvalidArgument("a request id appears twice in one step")
        any_top = out.n_top_stride > 0
        t0 = time.perf_counter()
        status = self._twin("step_v2")(
            self._h,
            c_rows,
            n,
            out._rows,
            out._top_ids.ctypes.data_as(C.POINTER(C.c_int32)) if any_top else None,
            out._top_logprobs.ctypes.data_as(C.POINTER(C.c_float)) if any_top else None,
            out.n_top_stride,
        )
        self.last_call_s = time.perf_counter() - t0   # wall time of the C call alone
        _check(status)
        out.n_rows = n

    def step_v1(self, rows: Sequence[StepRow], out_stride: int = 0):
        """The v1 entry point (retro_engine_step); returns (out rows, top ids, top logprobs)."""
        n = len(rows)
        c_rows = (_ffi.StepRowC * max(n, 1))()
        keep = []
        for i, r in enumerate(rows):
            tokens = np.ascontiguousarray(r.tokens, dtype=np.int32)
            keep.append(tokens)
            c = c_rows[i]
            c.struct_size = C.sizeof(_ffi.StepRowC)
            c.request, c.slot = r.request, r.slot
            c.tokens = tokens.ctypes.data_as(C.POINTER(C.c_int32))
            c.n, c.pos0, c.sample = tokens.size, r.pos0, r.sample
            c.sampling.temperature, c.sampling.top_p = r.sampling.temperature, r.sampling.top_p
            c.sampling.max_new_tokens, c.sampling.seed = r.sampling.max_new_tokens, r.sampling.seed
            c.n_top_logprobs, c.adapter = r.n_top_logprobs, r.adapter
        outs = (_ffi.StepOutRowC * max(n, 1))()
        ids = np.zeros(max(n * out_stride, 1), dtype=np.int32)
        lps = np.zeros(max(n * out_stride, 1), dtype=np.float32)
        _check(
            self._twin("step")(
                self._h,
                c_rows,
                n,
                outs,
                ids.ctypes.data_as(C.POINTER(C.c_int32)) if out_stride else None,
                lps.ctypes.data_as(C.POINTER(C.c_float)) if out_stride else None,
                out_stride,
            )
        )
        rows_out = [StepOutRow(o.token, o.logprob, bool(o.forced), bool(o.sampled), o.n_top, 0.0) for o in outs[:n]]
        return rows_out, ids.reshape(-1)[: n * out_stride].reshape(n, out_stride) if out_stride else ids[:0], (
            lps.reshape(-1)[: n * out_stride].reshape(n, out_stride) if out_stride else lps[:0]
        )

    # ---- sequence memory
    def seq_rm(self, slot: int, p0: int = -1, p1: int = -1) -> None:
        _check(self._twin("seq_rm")(self._h, slot, p0, p1))

    def seq_cp(self, src: int, dst: int, p0: int = -1, p1: int = -1) -> None:
        _check(self._twin("seq_cp")(self._h, src, dst, p0, p1))

    def seq_pos(self, slot: int) -> tuple[int, int]:
        a, b = C.c_int32(), C.c_int32()
        _check(self._twin("seq_pos")(self._h, slot, C.byref(a), C.byref(b)))
        return a.value, b.value

    def seq_save(self, slot: int, flags: int = 0) -> bytes:
        n = C.c_size_t()
        _check(self._twin("seq_save")(self._h, slot, flags, None, 0, C.byref(n)))
        buf = (C.c_uint8 * n.value)()
        _check(self._twin("seq_save")(self._h, slot, flags, buf, n.value, C.byref(n)))
        return bytes(buf[: n.value])

    def seq_load(self, slot: int, data: bytes, flags: int = 0) -> int:
        buf = (C.c_uint8 * max(len(data), 1)).from_buffer_copy(data if data else b"\0")
        n = C.c_size_t()
        _check(self._twin("seq_load")(self._h, slot, flags, buf, len(data), C.byref(n)))
        return n.value

    def memory(self) -> EngineMemory:
        m = _ffi.MemoryInfoC()
        _check(self._twin("memory")(self._h, C.byref(m)))
        return EngineMemory(m.n_slots, m.cells_total, m.cells_used, m.kv_bytes, m.recurrent_bytes)

    # ---- batched generators (retro_engine_generate_batch / _generate_continuous_batch)
    def _generation_outputs(self, n: int, n_out_max: int):
        tokens = np.zeros((n, n_out_max), dtype=np.int32)
        logprobs = np.zeros((n, n_out_max), dtype=np.float32)
        counts = (C.c_size_t * n)()
        forced = np.zeros((n, n_out_max), dtype=np.uint8)
        return tokens, logprobs, counts, forced

    @staticmethod
    def _v1(p: "SamplingParams"):
        return _ffi.SamplingParamsC(p.temperature, p.top_p, p.max_new_tokens, p.seed)

    def generate_batch(self, prompt: Sequence[int], samplings: Sequence["SamplingParams"], n_out_max: int):
        """One prompt, len(samplings) samples. Returns (token lists, logprob lists)."""
        n = len(samplings)
        ptoks = np.ascontiguousarray(prompt, dtype=np.int32)
        arr = (_ffi.SamplingParamsC * max(n, 1))(*[self._v1(p) for p in samplings])
        tokens, logprobs, counts, forced = self._generation_outputs(max(n, 1), max(n_out_max, 1))
        _check(self._lib.retro_engine_generate_batch(
            self._h, ptoks.ctypes.data_as(C.POINTER(C.c_int32)) if ptoks.size else None, ptoks.size, arr if n else None, n,
            tokens.ctypes.data_as(C.POINTER(C.c_int32)), logprobs.ctypes.data_as(C.POINTER(C.c_float)), n_out_max, counts,
            forced.ctypes.data_as(C.POINTER(C.c_uint8))))
        return [tokens[i, : counts[i]].tolist() for i in range(n)], [logprobs[i, : counts[i]].tolist() for i in range(n)]

    def generate_continuous(self, sequences: Sequence[tuple[Sequence[int], "SamplingParams"]], n_out_max: int):
        """One completion per (prompt, sampling) pair. Returns (token lists, logprob lists)."""
        n = len(sequences)
        keep = [np.ascontiguousarray(p, dtype=np.int32) for p, _ in sequences]
        arr = (_ffi.GenerationSequence * max(n, 1))()
        for i, (_, sp) in enumerate(sequences):
            arr[i].prompt_tokens = keep[i].ctypes.data_as(C.POINTER(C.c_int32)) if keep[i].size else None
            arr[i].n_prompt = keep[i].size
            arr[i].sampling = self._v1(sp)
        tokens, logprobs, counts, forced = self._generation_outputs(max(n, 1), max(n_out_max, 1))
        _check(self._lib.retro_engine_generate_continuous_batch(
            self._h, arr if n else None, n, tokens.ctypes.data_as(C.POINTER(C.c_int32)), logprobs.ctypes.data_as(C.POINTER(C.c_float)),
            n_out_max, counts, forced.ctypes.data_as(C.POINTER(C.c_uint8))))
        return [tokens[i, : counts[i]].tolist() for i in range(n)], [logprobs[i, : counts[i]].tolist() for i in range(n)]

    def request_free(self, request: int) -> None:
        _check(self._twin("request_free")(self._h, request))

    # ---- per-row adapters
    def adapter_load(self, path: str, scale: float = 1.0) -> int:
        v = C.c_int32()
        _check(self._lib.retro_engine_adapter_load(self._h, str(path).encode(), scale, C.byref(v)))
        return v.value

    def adapter_unload(self, adapter: int) -> None:
        _check(self._twin("adapter_unload")(self._h, adapter))

    def adapter_rows_info(self) -> dict:
        info = _ffi.AdapterRowsInfoC()
        _check(self._twin("adapter_rows_info")(self._h, C.byref(info)))
        return dict(n_adapters=info.n_adapters, max_rank=info.max_rank, stacked_bytes=info.stacked_bytes, unpadded_bytes=info.unpadded_bytes)

    # ---- one active adapter at a time: rows with adapter == 0 decode under it
    def load_lora(self, path: str) -> None:
        _check(self._lib.retro_engine_load_lora(self._h, str(path).encode()))

    def load_lora_named(self, name: str, path: str) -> None:
        _check(self._lib.retro_engine_load_lora_named(self._h, name.encode(), str(path).encode()))

    def activate_lora(self, name: str | None) -> None:
        _check(self._lib.retro_engine_activate_lora(self._h, name.encode() if name is not None else None))

    def set_lora_enabled(self, enabled: bool) -> None:
        _check(self._lib.retro_engine_set_lora_enabled(self._h, enabled))

    def active_adapter(self) -> str:
        n = C.c_size_t()
        _check(self._lib.retro_engine_active_adapter(self._h, None, 0, C.byref(n)))
        buf = C.create_string_buffer(n.value + 1)
        _check(self._lib.retro_engine_active_adapter(self._h, buf, n.value + 1, C.byref(n)))
        return buf.value.decode()

    # ---- counters
    def memory_report(self) -> dict:
        r = _ffi.MemoryReportC()
        _check(self._lib.retro_engine_memory_report(self._h, C.byref(r)))
        return {name: getattr(r, name) for name, _ in _ffi.MemoryReportC._fields_}

    def generation_stats(self) -> dict:
        st = _ffi.GenerationStatsC()
        _check(self._twin("stats" if self._twin_prefix.startswith("retro_trainer") else "generation_stats")(self._h, C.byref(st)))
        return {name: getattr(st, name) for name, _ in _ffi.GenerationStatsC._fields_}

    # ---- MoE expert banks
    def expert_banks(self) -> list[dict]:
        n = C.c_size_t()
        _check(self._lib.retro_engine_expert_banks(self._h, None, 0, C.byref(n)))
        banks = (_ffi.ExpertBankDescC * max(n.value, 1))()
        _check(self._lib.retro_engine_expert_banks(self._h, banks, n.value, C.byref(n)))
        return [dict(layer=b.layer, role=b.role.decode(), name=b.tensor.name.decode(), ne=list(b.tensor.ne), n_elements=b.tensor.n_elements,
                     n_bytes=b.tensor.n_bytes, type_name=b.tensor.type_name.decode()) for b in banks[: n.value]]

    def expert_stats(self) -> "_ffi.ExpertCacheStatsC":
        st = _ffi.ExpertCacheStatsC()
        _check(self._lib.retro_engine_expert_stats(self._h, C.byref(st)))
        return st

    def expert_route_paths(self) -> tuple[int, int, int]:
        out = (C.c_uint64 * 3)()
        _check(self._lib.retro_engine_expert_route_paths(self._h, out))
        return out[0], out[1], out[2]

    # ---- MoE telemetry
    def expert_route_enable(self, sample_every: int = 1) -> None:
        _check(self._lib.retro_engine_expert_route_enable(self._h, sample_every))

    def expert_route_counts(self, layer: int, n_expert: int) -> np.ndarray:
        out = np.zeros(n_expert, dtype=np.uint32)
        _check(self._lib.retro_engine_expert_route_counts(self._h, layer, out.ctypes.data_as(C.POINTER(C.c_uint32)), n_expert))
        return out

    # ---- inspection hooks (no counterpart in the reference)
    def last_pack(self) -> dict:
        nt, no = C.c_size_t(), C.c_size_t()
        _check(self._lib.retro_b200_engine_last_pack(self._h, C.byref(nt), C.byref(no), None, None, None, None, None, None, 0))
        cap = max(nt.value, self.config.n_batch) + 1
        arrs = {k: np.zeros(cap, dtype=np.int32) for k in ("tok_slot", "tok_pos", "tok_row", "tok_cell", "out_index", "cu_rows")}
        ptr = lambda a: a.ctypes.data_as(C.POINTER(C.c_int32))
        _check(
            self._lib.retro_b200_engine_last_pack(
                self._h, C.byref(nt), C.byref(no), ptr(arrs["tok_slot"]), ptr(arrs["tok_pos"]), ptr(arrs["tok_row"]),
                ptr(arrs["tok_cell"]), ptr(arrs["out_index"]), ptr(arrs["cu_rows"]), cap,
            )
        )
        T, S = nt.value, no.value
        out = {k: arrs[k][:T] for k in ("tok_slot", "tok_pos", "tok_row", "tok_cell")}
        out["out_index"] = arrs["out_index"][:S]
        out["cu_rows"] = arrs["cu_rows"]
        out["n_tokens"], out["n_out"] = T, S
        return out

    def last_logits(self, index: int) -> np.ndarray:
        v = self.vocab_size()
        out = np.zeros(v, dtype=np.float32)
        _check(self._lib.retro_b200_engine_last_logits(self._h, index, out.ctypes.data_as(C.POINTER(C.c_float)), v))
        return out

    def last_routes(self) -> np.ndarray:
        n = C.c_size_t()
        _check(self._lib.retro_b200_engine_last_routes(self._h, None, 0, C.byref(n)))
        out = np.zeros(max(n.value, 1), dtype=np.int32)
        _check(self._lib.retro_b200_engine_last_routes(self._h, out.ctypes.data_as(C.POINTER(C.c_int32)), out.size, C.byref(n)))
        return out[: n.value]

    def block_table(self, slot: int) -> tuple[np.ndarray, int]:
        n, b = C.c_size_t(), C.c_uint32()
        _check(self._lib.retro_b200_engine_block_table(self._h, slot, None, 0, C.byref(n), C.byref(b)))
        out = np.zeros(max(n.value, 1), dtype=np.int32)
        _check(self._lib.retro_b200_engine_block_table(self._h, slot, out.ctypes.data_as(C.POINTER(C.c_int32)), out.size, C.byref(n), C.byref(b)))
        return out[: n.value], b.value

    def blocks(self) -> tuple[int, int]:
        a, b = C.c_uint64(), C.c_uint64()
        _check(self._lib.retro_b200_engine_blocks(self._h, C.byref(a), C.byref(b)))
        return a.value, b.value

    def last_step_stats(self) -> tuple[float, int]:
        ms, n = C.c_float(), C.c_uint64()
        _check(self._lib.retro_b200_engine_last_step_stats(self._h, C.byref(ms), C.byref(n)))
        return ms.value, n.value

    def last_step_io(self) -> tuple[int, int]:
        a, b = C.c_uint64(), C.c_uint64()
        _check(self._lib.retro_b200_engine_last_step_io(self._h, C.byref(a), C.byref(b)))
        return a.value, b.value

    def expert_storage(self, layer: int) -> tuple[int, int, int]:
        """GGML type codes of the layer's gate / up / down expert banks as held on the device."""
        t = (C.c_uint32 * 3)()
        _check(self._lib.retro_b200_engine_expert_storage(self._h, layer, t))
        return t[0], t[1], t[2]

    def ep_init(self, rank: int, world: int, unique_id: bytes) -> None:
        """Joins the expert-parallel group (collective over all `world` engines, one per GPU)."""
        if len(unique_id) != 128:
            raise ValueError("the NCCL id is 128 bytes")
        _check(self._lib.retro_b200_engine_ep_init(self._h, rank, world, C.create_string_buffer(unique_id, 128)))

    def ep_idle_step(self) -> None:
        """The step of a rank that has no rows of its own while other ranks of the group step."""
        _check(self._lib.retro_b200_engine_ep_idle_step(self._h))

    def graph_stats(self) -> tuple[int, int]:
        """(steps replayed from a captured CUDA graph, graphs cached)."""
        a, b = C.c_uint64(), C.c_uint64()
        _check(self._lib.retro_b200_engine_graph_stats(self._h, C.byref(a), C.byref(b)))
        return a.value, b.value

    PROFILE_CLASSES = ("gemm", "attention", "sample", "pack", "moe", "lora", "other")

    def profile(self, enabled: bool, reset: bool = False) -> None:
        _check(self._lib.retro_b200_engine_profile(self._h, int(enabled), int(reset)))

    def profile_read(self) -> dict:
        ms = (C.c_double * 7)()
        n = (C.c_uint64 * 7)()
        _check(self._lib.retro_b200_engine_profile_read(self._h, ms, n, 7))
        return {name: {"ms": ms[i], "launches": n[i]} for i, name in enumerate(self.PROFILE_CLASSES)}


class TrainerGeneration(Engine):
    """The generation context an RL trainer owns, driven through the `retro_trainer_generation_*` twins of the
    engine's step and sequence entry points (crates/retrograd-infer/src/backend.rs:376-461 is the reference's
    caller). `weights_updated` is the trainer's notice after an optimizer step: with a path the trained adapter
    is read again; either way the KV is forgotten and the weights version moves on."""

    _twin_prefix = "retro_trainer_generation_"

    def __init__(self, model_path: str, config: EngineConfig | None = None, adapter_path: str | None = None) -> None:
        self._lib = _ffi.load_library()
        self.config = config or EngineConfig()
        c = self.config.to_c()
        self._h = self._lib.retro_b200_trainer_generation_new(str(model_path).encode(), C.byref(c), str(adapter_path).encode() if adapter_path else None)
        if not self._h:
            raise EngineError(_last_error())
        self._keep = []

    def close(self) -> None:
        if self._h:
            self._lib.retro_b200_trainer_generation_free(self._h)
            self._h = None

    def weights_updated(self, adapter_path: str | None = None) -> None:
        _check(self._lib.retro_b200_trainer_weights_updated(self._h, str(adapter_path).encode() if adapter_path else None))

    def adapter_snapshot(self, replace: int = 0, scale: float = 1.0) -> int:
        v = C.c_int32()
        _check(self._lib.retro_trainer_generation_adapter_snapshot(self._h, replace, scale, C.byref(v)))
        return v.value
