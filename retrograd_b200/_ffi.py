"""ctypes declarations of libretro_b200's C ABI (include/retro_b200.h)."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import os

# RB200_CHECKED=1 selects the bounds-checked build of the same sources (see retro_b200_checked_build in the header)
LIB_PATH = Path(__file__).resolve().parent / ("libretro_b200_checked.so" if os.environ.get("RB200_CHECKED") == "1" else "libretro_b200.so")


class SamplingParamsC(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_p", C.c_float), ("max_new_tokens", C.c_uint32), ("seed", C.c_uint32)]


class GenerationSequence(C.Structure):
    _fields_ = [("prompt_tokens", C.POINTER(C.c_int32)), ("n_prompt", C.c_size_t), ("sampling", SamplingParamsC)]


class StepRowC(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32),
        ("request", C.c_int32),
        ("slot", C.c_int32),
        ("tokens", C.POINTER(C.c_int32)),
        ("n", C.c_uint32),
        ("pos0", C.c_int32),
        ("sample", C.c_bool),
        ("sampling", SamplingParamsC),
        ("n_top_logprobs", C.c_uint32),
        ("adapter", C.c_int32),
    ]


class StepOutRowC(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32),
        ("token", C.c_int32),
        ("logprob", C.c_float),
        ("n_top", C.c_uint32),
        ("forced", C.c_uint8),
        ("sampled", C.c_uint8),
    ]


class SamplingParamsV2C(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32),
        ("temperature", C.c_float),
        ("top_p", C.c_float),
        ("max_new_tokens", C.c_uint32),
        ("seed", C.c_uint32),
        ("top_k", C.c_int32),
        ("min_p", C.c_float),
        ("repeat_penalty", C.c_float),
        ("frequency_penalty", C.c_float),
        ("presence_penalty", C.c_float),
        ("penalty_window", C.c_uint32),
        ("n_logit_bias", C.c_uint32),
        ("logit_bias_ids", C.POINTER(C.c_int32)),
        ("logit_bias_values", C.POINTER(C.c_float)),
        ("grammar", C.c_void_p),
    ]


class StepRowV2C(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32),
        ("request", C.c_int32),
        ("slot", C.c_int32),
        ("tokens", C.POINTER(C.c_int32)),
        ("n", C.c_uint32),
        ("pos0", C.c_int32),
        ("sample", C.c_bool),
        ("sampling", SamplingParamsV2C),
        ("n_top_logprobs", C.c_uint32),
        ("want_logprob", C.c_uint8),
        ("adapter", C.c_int32),
    ]


class StepOutRowV2C(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32),
        ("token", C.c_int32),
        ("logprob", C.c_float),
        ("n_top", C.c_uint32),
        ("forced", C.c_uint8),
        ("sampled", C.c_uint8),
        ("sampled_logprob", C.c_float),
    ]


class EngineConfigC(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32),
        ("n_ctx", C.c_uint32),
        ("n_seq_max", C.c_uint32),
        ("n_batch", C.c_uint32),
        ("n_ubatch", C.c_uint32),
        ("kv_dtype", C.c_int32),
        ("flash_attn", C.c_bool),
        ("device", C.c_int32),
        ("threads", C.c_uint32),
        ("verbose", C.c_bool),
        ("kv_unified", C.c_uint32),
        ("expert_placement", C.c_int32),
        ("expert_host_layers", C.c_uint32),
        ("expert_device_cache_bytes", C.c_uint64),
    ]


class MemoryInfoC(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32),
        ("n_slots", C.c_uint32),
        ("cells_total", C.c_uint64),
        ("cells_used", C.c_uint64),
        ("kv_bytes", C.c_uint64),
        ("recurrent_bytes", C.c_uint64),
    ]


class AdapterRowsInfoC(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32),
        ("n_adapters", C.c_uint32),
        ("max_rank", C.c_uint32),
        ("stacked_bytes", C.c_uint64),
        ("unpadded_bytes", C.c_uint64),
    ]


class MemoryReportC(C.Structure):
    _fields_ = [
        ("model_weight_bytes", C.c_uint64), ("optimizer_kv_bytes", C.c_uint64), ("optimizer_compute_bytes", C.c_uint64),
        ("generation_kv_bytes", C.c_uint64), ("generation_compute_bytes", C.c_uint64), ("has_generation_context", C.c_bool),
        ("trainable_parameter_bytes", C.c_uint64), ("trainable_gradient_bytes", C.c_uint64), ("optimizer_state_bytes", C.c_uint64),
        ("trainable_parameters_are_model_subset", C.c_bool), ("adapter_on_host", C.c_bool), ("base_trainable_on_host", C.c_bool),
        ("device_bytes", C.c_uint64), ("host_bytes", C.c_uint64), ("device_total_bytes", C.c_uint64), ("device_used_bytes", C.c_uint64),
        ("device_peak_used_bytes", C.c_uint64), ("backend_scratch_bytes", C.c_uint64), ("backend_scratch_peak_bytes", C.c_uint64),
        ("device_memory_samples", C.c_uint64), ("checkpoint_count", C.c_uint64), ("checkpoint_retained_bytes", C.c_uint64),
        ("checkpoint_live_peak_bytes", C.c_uint64), ("checkpoint_live_peak_count", C.c_uint64), ("checkpoint_long_lived_bytes", C.c_uint64),
        ("checkpoint_long_lived_count", C.c_uint64), ("checkpoint_graph_nodes", C.c_uint64), ("checkpoint_max_span_nodes", C.c_uint64),
        ("checkpoint_total_span_nodes", C.c_uint64),
    ]


class GenerationStatsC(C.Structure):
    _fields_ = [(name, C.c_uint64) for name in ("calls", "sequences", "prompt_tokens", "prefilled_tokens", "reused_tokens", "hits", "evictions")]


class TensorDescC(C.Structure):
    _fields_ = [("name", C.c_char * 128), ("ne", C.c_int64 * 4), ("n_elements", C.c_uint64), ("n_bytes", C.c_uint64), ("storage_id", C.c_uint64),
                ("type_name", C.c_char * 64)]


class ExpertBankDescC(C.Structure):
    _fields_ = [("layer", C.c_uint32), ("role", C.c_char * 16), ("tensor", TensorDescC)]


class _CacheCounters(C.Structure):
    _fields_ = [("hits", C.c_uint64), ("misses", C.c_uint64), ("bytes", C.c_uint64)]


class ExpertCacheGroupC(C.Structure):
    _fields_ = [("n_slots", C.c_int32), ("n_layers", C.c_int32), ("n_expert", C.c_int32), ("device_bytes", C.c_uint64)]


class ExpertCacheStatsC(C.Structure):
    _fields_ = [("small", _CacheCounters), ("large", _CacheCounters), ("copy", _CacheCounters), ("n_groups", C.c_int32),
                ("groups", ExpertCacheGroupC * 16)]


# Every symbol include/retro_b200.h declares: name -> (restype, argtypes).
_P = C.POINTER
SYMBOLS = {
    "retro_last_error": (C.c_char_p, []),
    "retro_engine_new": (C.c_void_p, [C.c_char_p, _P(EngineConfigC)]),
    "retro_engine_new_checked": (C.c_void_p, [C.c_char_p, _P(EngineConfigC), _P(C.c_bool)]),
    "retro_engine_free": (None, [C.c_void_p]),
    "retro_engine_eos_token": (C.c_int, [C.c_void_p, _P(C.c_int32)]),
    "retro_engine_vocab_size": (C.c_int, [C.c_void_p, _P(C.c_uint32)]),
    "retro_engine_is_eog_token": (C.c_int, [C.c_void_p, C.c_int32, _P(C.c_bool)]),
    "retro_engine_set_reasoning_budget": (C.c_int, [C.c_void_p, C.c_int32]),
    "retro_b200_reasoning_check": (C.c_int, [_P(C.c_int32), C.c_size_t, _P(_P(C.c_int32)), _P(C.c_size_t), C.c_size_t, C.c_int32, C.c_size_t, _P(C.c_int32),
                                             C.c_size_t, _P(C.c_int32), C.c_size_t, _P(C.c_int32), C.c_size_t, _P(C.c_int32), _P(C.c_uint8)]),
    "retro_trainer_set_reasoning_budget": (C.c_int, [C.c_void_p, C.c_int32]),
    "retro_b200_engine_set_reasoning_tags": (C.c_int, [C.c_void_p, _P(C.c_int32), C.c_size_t, _P(_P(C.c_int32)), _P(C.c_size_t), C.c_size_t, C.c_size_t]),
    "retro_b200_trainer_set_reasoning_tags": (C.c_int, [C.c_void_p, _P(C.c_int32), C.c_size_t, _P(_P(C.c_int32)), _P(C.c_size_t), C.c_size_t, C.c_size_t]),
    "retro_engine_context_size": (C.c_int, [C.c_void_p, _P(C.c_uint32)]),
    "retro_engine_detokenize": (C.c_int, [C.c_void_p, _P(C.c_int32), C.c_size_t, C.c_bool, C.c_char_p, C.c_size_t, _P(C.c_size_t)]),
    "retro_engine_tokenize_text": (C.c_int, [C.c_void_p, C.c_char_p, _P(C.c_int32), C.c_size_t, _P(C.c_size_t)]),
    "retro_engine_tokenize_fragment": (C.c_int, [C.c_void_p, C.c_char_p, _P(C.c_int32), C.c_size_t, _P(C.c_size_t)]),
    "retro_engine_adapter_load": (C.c_int, [C.c_void_p, C.c_char_p, C.c_float, _P(C.c_int32)]),
    "retro_engine_adapter_unload": (C.c_int, [C.c_void_p, C.c_int32]),
    "retro_engine_adapter_rows_info": (C.c_int, [C.c_void_p, _P(AdapterRowsInfoC)]),
    "retro_engine_graphs_reused": (C.c_int, [C.c_void_p, _P(C.c_uint64)]),
    "retro_engine_step": (C.c_int, [C.c_void_p, _P(StepRowC), C.c_size_t, _P(StepOutRowC), _P(C.c_int32), _P(C.c_float), C.c_size_t]),
    "retro_engine_step_v2": (C.c_int, [C.c_void_p, _P(StepRowV2C), C.c_size_t, _P(StepOutRowV2C), _P(C.c_int32), _P(C.c_float), C.c_size_t]),
    "retro_engine_seq_rm": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32]),
    "retro_engine_seq_cp": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32]),
    "retro_engine_seq_save": (C.c_int, [C.c_void_p, C.c_int32, C.c_uint32, _P(C.c_uint8), C.c_size_t, _P(C.c_size_t)]),
    "retro_engine_seq_load": (C.c_int, [C.c_void_p, C.c_int32, C.c_uint32, _P(C.c_uint8), C.c_size_t, _P(C.c_size_t)]),
    "retro_engine_seq_pos": (C.c_int, [C.c_void_p, C.c_int32, _P(C.c_int32), _P(C.c_int32)]),
    "retro_engine_memory": (C.c_int, [C.c_void_p, _P(MemoryInfoC)]),
    "retro_engine_request_free": (C.c_int, [C.c_void_p, C.c_int32]),
    "retro_engine_generate_batch": (C.c_int, [C.c_void_p, _P(C.c_int32), C.c_size_t, _P(SamplingParamsC), C.c_size_t, _P(C.c_int32), _P(C.c_float),
                                              C.c_size_t, _P(C.c_size_t), _P(C.c_uint8)]),
    "retro_engine_generate_continuous_batch": (C.c_int, [C.c_void_p, _P(GenerationSequence), C.c_size_t, _P(C.c_int32), _P(C.c_float),
                                                         C.c_size_t, _P(C.c_size_t), _P(C.c_uint8)]),
    "retro_engine_kv_unified": (C.c_int, [C.c_void_p, _P(C.c_bool)]),
    "retro_engine_weights_version": (C.c_int, [C.c_void_p, _P(C.c_uint64)]),
    "retro_engine_model_fingerprint": (C.c_int, [C.c_void_p, _P(C.c_uint64)]),
    "retro_engine_is_hybrid": (C.c_int, [C.c_void_p, _P(C.c_bool)]),
    "retro_engine_expert_route_enable": (C.c_int, [C.c_void_p, C.c_uint32]),
    "retro_engine_expert_route_counts": (C.c_int, [C.c_void_p, C.c_uint32, _P(C.c_uint32), C.c_size_t]),
    "retro_engine_expert_route_reset": (C.c_int, [C.c_void_p]),
    "retro_engine_load_lora": (C.c_int, [C.c_void_p, C.c_char_p]),
    "retro_engine_set_lora_enabled": (C.c_int, [C.c_void_p, C.c_bool]),
    "retro_engine_load_lora_named": (C.c_int, [C.c_void_p, C.c_char_p, C.c_char_p]),
    "retro_engine_activate_lora": (C.c_int, [C.c_void_p, C.c_char_p]),
    "retro_engine_active_adapter": (C.c_int, [C.c_void_p, C.c_char_p, C.c_size_t, _P(C.c_size_t)]),
    "retro_engine_memory_report": (C.c_int, [C.c_void_p, _P(MemoryReportC)]),
    "retro_engine_generation_stats": (C.c_int, [C.c_void_p, _P(GenerationStatsC)]),
    "retro_engine_expert_banks": (C.c_int, [C.c_void_p, _P(ExpertBankDescC), C.c_size_t, _P(C.c_size_t)]),
    "retro_engine_expert_stats": (C.c_int, [C.c_void_p, _P(ExpertCacheStatsC)]),
    "retro_engine_expert_route_paths": (C.c_int, [C.c_void_p, _P(C.c_uint64)]),
    "retro_grammar_from_json_schema": (C.c_void_p, [C.c_char_p]),
    "retro_grammar_from_gbnf": (C.c_void_p, [C.c_char_p]),
    "retro_grammar_json_object": (C.c_void_p, []),
    "retro_grammar_gbnf": (C.c_char_p, [C.c_void_p]),
    "retro_grammar_free": (None, [C.c_void_p]),
    "retro_trainer_generation_step": (C.c_int, [C.c_void_p, _P(StepRowC), C.c_size_t, _P(StepOutRowC), _P(C.c_int32), _P(C.c_float), C.c_size_t]),
    "retro_trainer_generation_step_v2": (C.c_int, [C.c_void_p, _P(StepRowV2C), C.c_size_t, _P(StepOutRowV2C), _P(C.c_int32), _P(C.c_float), C.c_size_t]),
    "retro_trainer_generation_seq_rm": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32]),
    "retro_trainer_generation_seq_cp": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32]),
    "retro_trainer_generation_seq_save": (C.c_int, [C.c_void_p, C.c_int32, C.c_uint32, _P(C.c_uint8), C.c_size_t, _P(C.c_size_t)]),
    "retro_trainer_generation_seq_load": (C.c_int, [C.c_void_p, C.c_int32, C.c_uint32, _P(C.c_uint8), C.c_size_t, _P(C.c_size_t)]),
    "retro_trainer_generation_seq_pos": (C.c_int, [C.c_void_p, C.c_int32, _P(C.c_int32), _P(C.c_int32)]),
    "retro_trainer_generation_memory": (C.c_int, [C.c_void_p, _P(MemoryInfoC)]),
    "retro_trainer_generation_request_free": (C.c_int, [C.c_void_p, C.c_int32]),
    "retro_trainer_generation_kv_unified": (C.c_int, [C.c_void_p, _P(C.c_bool)]),
    "retro_trainer_generation_weights_version": (C.c_int, [C.c_void_p, _P(C.c_uint64)]),
    "retro_trainer_generation_stats": (C.c_int, [C.c_void_p, _P(GenerationStatsC)]),
    "retro_trainer_generation_adapter_snapshot": (C.c_int, [C.c_void_p, C.c_int32, C.c_float, _P(C.c_int32)]),
    "retro_trainer_generation_adapter_unload": (C.c_int, [C.c_void_p, C.c_int32]),
    "retro_trainer_generation_adapter_rows_info": (C.c_int, [C.c_void_p, _P(AdapterRowsInfoC)]),
    "retro_b200_trainer_generation_new": (C.c_void_p, [C.c_char_p, _P(EngineConfigC), C.c_char_p]),
    "retro_b200_trainer_generation_free": (None, [C.c_void_p]),
    "retro_b200_trainer_weights_updated": (C.c_int, [C.c_void_p, C.c_char_p]),
    "retro_b200_synth_gguf": (C.c_int, [C.c_char_p, C.c_char_p, _P(C.c_uint64)]),
    "retro_b200_quantize_row": (C.c_int, [C.c_uint32, _P(C.c_float), C.c_size_t, _P(C.c_uint8), C.c_size_t, _P(C.c_size_t)]),
    "retro_b200_engine_last_pack": (
        C.c_int,
        [C.c_void_p, _P(C.c_size_t), _P(C.c_size_t), _P(C.c_int32), _P(C.c_int32), _P(C.c_int32), _P(C.c_int32), _P(C.c_int32), _P(C.c_int32), C.c_size_t],
    ),
    "retro_b200_engine_last_logits": (C.c_int, [C.c_void_p, C.c_size_t, _P(C.c_float), C.c_size_t]),
    "retro_b200_engine_last_routes": (C.c_int, [C.c_void_p, _P(C.c_int32), C.c_size_t, _P(C.c_size_t)]),
    "retro_b200_engine_block_table": (C.c_int, [C.c_void_p, C.c_int32, _P(C.c_int32), C.c_size_t, _P(C.c_size_t), _P(C.c_uint32)]),
    "retro_b200_engine_blocks": (C.c_int, [C.c_void_p, _P(C.c_uint64), _P(C.c_uint64)]),
    "retro_b200_engine_last_step_stats": (C.c_int, [C.c_void_p, _P(C.c_float), _P(C.c_uint64)]),
    "retro_b200_op_gemm": (C.c_int, [C.c_uint32, _P(C.c_uint8), C.c_uint32, C.c_uint32, _P(C.c_float), C.c_uint32, _P(C.c_float), C.c_int, C.c_uint32, _P(C.c_float)]),
    "retro_b200_op_gemm_mxfp4_grouped": (C.c_int, [_P(C.c_uint8), C.c_uint32, C.c_uint32, C.c_uint32, _P(C.c_float), _P(C.c_int32), _P(C.c_float), C.c_uint32,
                                                   _P(C.c_float)]),
    "retro_b200_gemm_q4k_noalloc": (C.c_int, [C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p]),
    "retro_b200_engine_last_step_io": (C.c_int, [C.c_void_p, _P(C.c_uint64), _P(C.c_uint64)]),
    "retro_b200_grammar_check": (C.c_int, [C.c_char_p, C.c_char_p, _P(C.c_int)]),
    "retro_b200_checked_build": (C.c_int, []),
    "retro_b200_engine_check_word": (C.c_int, [C.c_void_p, _P(C.c_int32)]),
    "retro_b200_engine_graph_stats": (C.c_int, [C.c_void_p, _P(C.c_uint64), _P(C.c_uint64)]),
    "retro_b200_nccl_unique_id": (C.c_int, [C.c_void_p]),
    "retro_b200_engine_expert_storage": (C.c_int, [C.c_void_p, C.c_int, _P(C.c_uint32)]),
    "retro_b200_recode_mxfp4_as_q8_0": (C.c_int, [C.c_void_p, C.c_size_t, C.c_void_p, _P(C.c_int)]),
    "retro_b200_engine_ep_init": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "retro_b200_engine_ep_idle_step": (C.c_int, [C.c_void_p]),
    "retro_b200_ep_plan": (C.c_int, [_P(C.c_int32), C.c_int, C.c_int, C.c_int, _P(C.c_int32), _P(C.c_int32), _P(C.c_int32), _P(C.c_int32),
                                     _P(C.c_int32), _P(C.c_int32), C.c_int32, _P(C.c_int32)]),
    "retro_b200_engine_profile": (C.c_int, [C.c_void_p, C.c_int, C.c_int]),
    "retro_b200_engine_profile_read": (C.c_int, [C.c_void_p, _P(C.c_double), _P(C.c_uint64), C.c_size_t]),
}

_lib = None


def load_library() -> C.CDLL:
    """Loads libretro_b200.so and binds every declared symbol; raises if it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} has not been built: run `python -m retrograd_b200.build` (there is no fallback implementation)"
        )
    lib = C.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SYMBOLS.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib
