"""ctypes binding of libxinfer_b200.so.  Fails loudly when the library is missing."""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libxinfer_b200.so")
_lib = None

OK = 0
NOOP_INVALID_SHAPE = 1
ERR_CUDA = -1
ERR_INVALID_ARGUMENT = -2
ERR_OUT_OF_MEMORY = -3
ERR_CONTRACT = -4
ERR_DEVICE_TIMEOUT = -5
ERR_NO_DEVICE = -6


class XInferError(RuntimeError):
    def __init__(self, code: int, what: str):
        super().__init__(f"{what}: status {code}")
        self.code = code


class FusedDesc(C.Structure):
    """xinfer_fused_desc (FusedProjectionDesc of the reference, src/ops/linear.h:66-81)."""
    _fields_ = [("Y", C.c_void_p), ("W_int4", C.c_void_p), ("scales", C.c_void_p), ("bias", C.c_void_p),
                ("N", C.c_int64)]


class AcceptResult(C.Structure):
    """xinfer_accept_result (SpeculativeAcceptanceResult, src/ops/sampling.h:27-36)."""
    _fields_ = [("accepted_tokens", C.c_int64 * 64), ("bonus_or_resampled_token", C.c_int64),
                ("rejected_token", C.c_int64), ("num_accepted", C.c_int64), ("num_rejected", C.c_int64),
                ("num_resampled", C.c_int64), ("num_remaining", C.c_int64), ("has_rejected_token", C.c_int32),
                ("reserved", C.c_int32)]


class ModelConfig(C.Structure):
    """xinfer_model_config: the shape fields of the reference's ModelConfig (src/targets/qwen3_8_27b/weights.h:58-107)."""
    _fields_ = [("hidden_size", C.c_int64), ("intermediate_size", C.c_int64), ("num_hidden_layers", C.c_int64),
                ("num_attention_heads", C.c_int64), ("num_key_value_heads", C.c_int64), ("vocab_size", C.c_int64),
                ("linear_num_v_heads", C.c_int64), ("linear_num_k_heads", C.c_int64),
                ("full_attention_interval", C.c_int32), ("rope_dim", C.c_int32), ("rms_norm_eps", C.c_float),
                ("rope_theta", C.c_float)]


class AcceptRecord(C.Structure):
    _fields_ = [("bonus_or_resampled_token", C.c_int64), ("rejected_token", C.c_int64), ("num_accepted", C.c_int32),
                ("num_rejected", C.c_int32), ("num_resampled", C.c_int32), ("num_remaining", C.c_int32),
                ("has_rejected_token", C.c_int32), ("reserved", C.c_int32)]


_vp, _i64, _i32, _f32, _u64, _sz = C.c_void_p, C.c_int64, C.c_int, C.c_float, C.c_uint64, C.c_size_t

# name -> (restype, argtypes); the list is also what the symbol-export test checks.
SIGNATURES = {
    "xinfer_b200_init": (_i32, [_i32]),
    "xinfer_b200_init_current": (_i32, []),
    "xinfer_device_status": (_i32, [_i32]),
    "xinfer_last_cuda_error": (C.c_char_p, []),
    "xinfer_b200_version": (C.c_char_p, []),
    "xinfer_last_linear_path": (_i32, []),
    "xinfer_set_linear_path": (None, [_i32]),
    "xinfer_debug_set_wait_hooks": (None, [_i64, _i32]),
    "xinfer_linear_plan_record_begin": (None, []),
    "xinfer_linear_plan_record_end": (None, []),
    "xinfer_linear_plan_rewind": (None, []),
    "xinfer_linear_plan_clear": (None, []),
    "xinfer_linear_int4_f16f16": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32]),
    "xinfer_linear_int4_f16f32": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32]),
    "xinfer_linear_int4_f32f32": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32]),
    "xinfer_linear_int4_f16f16_ld": (_i32, [_vp, _vp, _i64, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32]),
    "xinfer_linear_int4_f16f16_noalloc": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32]),
    "xinfer_linear_int4_fused_f16": (_i32, [_vp, _vp, C.POINTER(FusedDesc), _i32, _i64, _i64, _i32]),
    "xinfer_linear_int4_fused_f32": (_i32, [_vp, _vp, C.POINTER(FusedDesc), _i32, _i64, _i64, _i32]),
    "xinfer_mlp_gate_up_swiglu_int4_f16": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32]),
    "xinfer_mlp_gate_up_swiglu_int4_f32": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32]),
    "xinfer_argmax_scratch_size": (_sz, [_i64]),
    "xinfer_argmax": (_i64, [_vp, _vp, _i64, _vp, _vp]),
    "xinfer_argmax_rows": (_i32, [_vp, _vp, _i64, _i64, _i64, _vp]),
    "xinfer_speculative_accept_reject": (_i32, [_vp, _vp, _sz, _vp, _i64, _vp, _vp, C.POINTER(AcceptResult)]),
    "xinfer_speculative_accept_reject_batched": (_i32, [_vp, _vp, _vp, _i64, _i64, _vp, _vp, _f32, _i32, _i32, _i32,
                                                        _i32, _vp]),
    "xinfer_philox_uniform": (_i32, [_vp, _vp, _i64, _u64, _u64]),
    "xinfer_spec_decoder_create": (_i32, [_vp, _i32, _i32, _i64, _u64, C.POINTER(_vp)]),
    "xinfer_spec_decoder_destroy": (None, [_vp]),
    "xinfer_spec_decoder_reset": (_i32, [_vp, _i64, _u64]),
    "xinfer_spec_decoder_set_tokens": (_i32, [_vp, _vp]),
    "xinfer_spec_decoder_step": (_i32, [_vp, _vp]),
    "xinfer_spec_decoder_capture": (_i32, [_vp, _vp]),
    "xinfer_spec_decoder_results": (_i32, [_vp, _vp, _vp, _vp]),
    "xinfer_spec_decoder_override_drafts": (_i32, [_vp, _vp]),
    "xinfer_spec_decoder_enqueue_linears": (_i32, [_vp, _vp]),
    "xinfer_spec_decoder_info": (_i64, [_vp, _i32]),
    "xinfer_spec_decoder_tensor": (_vp, [_vp, _i32, C.c_char_p, C.POINTER(_i64)]),
    "xinfer_spec_decoder_error": (C.c_char_p, [_vp]),
    "xinfer_rmsnorm_f16": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _f32]),
    "xinfer_rmsnorm_residual_f16": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _f32]),
    "xinfer_rope_f16": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _f32, _i64]),
    "xinfer_attention_write_kv_cache_f16": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64]),
    "xinfer_sdpa_causal_cached_f16": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _f32, _i64]),
    "xinfer_causal_conv1d_silu_f16": (_i32, [_vp, _vp, _vp, _vp, _i64, _vp, _i64]),
    "xinfer_recurrent_gated_delta_net_f16": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i32, _i64, _i64]),
    "xinfer_tp_create": (_i32, [_i32, _i32, _sz, C.POINTER(_vp)]),
    "xinfer_tp_destroy": (None, [_vp]),
    "xinfer_tp_handle_bytes": (_sz, []),
    "xinfer_tp_handle": (_i32, [_vp, _vp]),
    "xinfer_tp_connect": (_i32, [_vp, _vp]),
    "xinfer_tp_rank": (_i32, [_vp]),
    "xinfer_tp_world": (_i32, [_vp]),
    "xinfer_tp_alloc": (_i32, [_vp, _sz, C.POINTER(_sz)]),
    "xinfer_tp_ptr": (_vp, [_vp, _sz]),
    "xinfer_tp_linear_int4_f16f16": (_i32, [_vp, _vp, _sz, _i64, _i64, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _i32]),
    "xinfer_tp_push": (_i32, [_vp, _vp, _sz, _sz]),
    "xinfer_tp_barrier": (_i32, [_vp, _vp]),
    "xinfer_tp_set_wait_limit": (None, [_vp, _i64]),
    "xinfer_tp_status": (_i32, [_vp]),
    "xinfer_spec_decoder_exchange_bytes": (_sz, [_vp, _i32, _i32, _i32]),
    "xinfer_spec_decoder_load_artifact": (_i32, [_vp, _vp, _i32]),
    "xinfer_spec_decoder_prefill": (_i32, [_vp, _vp, _vp, _i64]),
    "xinfer_spec_decoder_set_sampling": (_i32, [_vp, _f32, _u64]),
    "xinfer_spec_decoder_generate": (_i32, [_vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _vp]),
    "xinfer_sample_tokens_top_p": (_i32, [_vp, _vp, _i64, _i64, _i32, _f32, _f32, _vp, _vp, _vp]),
    "xinfer_spec_decoder_set_top_p": (_i32, [_vp, _f32]),
    "xinfer_sample_tokens": (_i32, [_vp, _vp, _i64, _i64, _i32, _f32, _vp, _vp, _vp]),
    "xinfer_spec_decoder_create_tp": (_i32, [_vp, _i32, _i32, _i64, _u64, _vp, C.POINTER(_vp)]),
    "xinfer_arena_create": (_i32, [_sz, _sz, C.POINTER(_vp)]),
    "xinfer_arena_destroy": (None, [_vp]),
    "xinfer_arena_allocate": (_i32, [_vp, _sz, _sz, C.POINTER(_vp)]),
    "xinfer_arena_allocate_persistent": (_i32, [_vp, _sz, _sz, C.POINTER(_vp)]),
    "xinfer_arena_persistent_buffer": (_i32, [_vp, _sz, _sz, C.POINTER(_vp)]),
    "xinfer_arena_reset": (None, [_vp]),
    "xinfer_arena_capacity": (_sz, [_vp]),
    "xinfer_arena_allocated_bytes": (_sz, [_vp]),
    "xinfer_arena_remaining_bytes": (_sz, [_vp]),
    "xinfer_arena_peak_allocated_bytes": (_sz, [_vp]),
    "xinfer_arena_base_ptr": (_vp, [_vp]),
    "xinfer_device_alloc": (_i32, [_sz, C.POINTER(_vp)]),
    "xinfer_device_free": (None, [_vp]),
    "xinfer_stream_create": (_i32, [C.POINTER(_vp)]),
    "xinfer_stream_destroy": (None, [_vp]),
    "xinfer_stream_synchronize": (_i32, [_vp]),
    "xinfer_copy_device_to_host": (_i32, [_vp, _vp, _sz]),
    "xinfer_copy_host_to_device": (_i32, [_vp, _vp, _sz]),
    "xinfer_crc64": (_u64, [_vp, _sz]),
    "xinfer_crc64_file": (_u64, [C.c_char_p, _u64]),
    "xinfer_crc64_update": (_u64, [_u64, _vp, _sz]),
    "xinfer_artifact_open": (_i32, [C.c_char_p, _i32, C.POINTER(_vp)]),
    "xinfer_artifact_close": (None, [_vp]),
    "xinfer_artifact_section_count": (_i32, [_vp]),
    "xinfer_artifact_find": (_i32, [_vp, C.c_char_p]),
    "xinfer_artifact_section_info": (_i32, [_vp, _i32, C.POINTER(C.c_char_p), C.POINTER(C.c_uint32), C.POINTER(_u64),
                                            C.POINTER(_u64), C.POINTER(_u64)]),
    "xinfer_artifact_metadata": (C.c_char_p, [_vp, C.POINTER(_u64)]),
    "xinfer_artifact_error": (C.c_char_p, [_vp]),
    "xinfer_artifact_read_section": (_i32, [_vp, C.c_char_p, _vp, _u64]),
    "xinfer_artifact_load_section": (_i32, [_vp, C.c_char_p, _u64, _u64, _vp, _i32]),
    "xinfer_artifact_load_linear": (_i32, [_vp, C.c_char_p, _i64, _i64, _i32, _i64, _i64, _vp, _vp, _i32]),
    "xinfer_artifact_load_bf16_as_f32": (_i32, [_vp, C.c_char_p, _i64, _i32, _vp]),
}


def library_path() -> str:
    return _LIB_PATH


def lib():
    """The loaded C-ABI library.  Raises if it has not been built: there is no fallback path."""
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise ImportError(
                f"{_LIB_PATH} is missing. Build it with `python -m xinfer_b200.build` "
                "(nvcc, sm_100a). xinfer_b200 has no CPU or PyTorch fallback.")
        handle = C.CDLL(_LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError here means a declared symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(code: int, what: str) -> int:
    if code < 0:
        detail = lib().xinfer_last_cuda_error()
        raise XInferError(code, what + (f" ({detail.decode()})" if detail else ""))
    return code
