"""B200-native batched decode step behind the reference's `retro_engine_*` C ABI.

The product is `libretro_b200.so` (CUDA kernels for sm_100a plus the C-ABI runtime). This package
is the thin host-side mirror of the reference's `retrograd_engine::Engine` / `StepRow` /
`StepOutput` (crates/retrograd-engine/src/step.rs:93-301,412-505) over that library, used by the
parity tests and the benchmark. There is no CPU fallback: loading fails loudly when the library
has not been built, and creating an engine fails loudly without a CUDA device.
"""
from ._ffi import LIB_PATH, load_library
from .engine import (
    ADAPTER_BASE,
    Engine,
    EngineConfig,
    EngineError,
    Grammar,
    InvalidArgument,
    KV_DTYPE_F16,
    KV_DTYPE_F32,
    KV_DTYPE_Q4_0,
    KV_DTYPE_Q8_0,
    SamplingParams,
    SamplingParamsV2,
    StepOutput,
    StepRow,
    TrainerGeneration,
    ep_plan,
    grammar_check,
    nccl_unique_id,
    op_gemm,
    reasoning_check,
    op_gemm_mxfp4_grouped,
    quantize_row,
    recode_mxfp4_as_q8_0,
    synth_gguf,
)

__all__ = [
    "ADAPTER_BASE",
    "Engine",
    "EngineConfig",
    "EngineError",
    "Grammar",
    "InvalidArgument",
    "KV_DTYPE_F16",
    "KV_DTYPE_F32",
    "KV_DTYPE_Q4_0",
    "KV_DTYPE_Q8_0",
    "LIB_PATH",
    "SamplingParams",
    "SamplingParamsV2",
    "StepOutput",
    "StepRow",
    "TrainerGeneration",
    "ep_plan",
    "grammar_check",
    "load_library",
    "nccl_unique_id",
    "op_gemm",
    "reasoning_check",
    "op_gemm_mxfp4_grouped",
    "quantize_row",
    "recode_mxfp4_as_q8_0",
    "synth_gguf",
]
