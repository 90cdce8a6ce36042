"""ctypes loader of ``libdecidra_b200.so``. There is no fallback: if the CUDA library is missing or
cannot be loaded, importing the engine fails with an explicit error."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

from .config import ModelConfig, Options

LIB_PATH = Path(__file__).resolve().parent / "libdecidra_b200.so"

OK, E_INVALID, E_OOM, E_UNSUPPORTED, E_CUDA, E_TIMEOUT, E_OVERLOADED, E_FAILED = 0, 1, 2, 3, 4, 5, 6, 7
PROF_NAMES = ("gemm", "attn", "gdn", "elementwise", "readout")


class Info(C.Structure):
    _fields_ = [
        ("device", C.c_int32), ("sm_count", C.c_int32), ("cc_major", C.c_int32), ("cc_minor", C.c_int32),
        ("device_name", C.c_char * 128), ("hidden", C.c_int32), ("num_layers", C.c_int32), ("readout_rows", C.c_int32),
        ("supports_vision", C.c_int32), ("weight_bytes", C.c_uint64), ("workspace_bytes", C.c_uint64),
    ]


class TensorInfo(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("rank", C.c_int32), ("shape", C.c_uint64 * 8), ("bytes", C.c_uint64), ("data", C.c_void_p)]


class SchedOptions(C.Structure):
    """Mirrors ``dcd_sched_options``."""
    _fields_ = [
        ("max_queue", C.c_int32), ("batch_requests", C.c_int32), ("batch_rows", C.c_int32), ("batch_window_us", C.c_int64),
        ("state_cache_entries", C.c_int32), ("pin_cache", C.c_int32), ("state_cache_bytes", C.c_int64),
        ("host_state_cache_bytes", C.c_int64), ("sched_priority", C.c_int32), ("cross_state_pass", C.c_int32),
        ("submit_timeout_us", C.c_int64), ("cold_one_pass", C.c_int64), ("reserved", C.c_int64 * 3),
    ]


OP_INT_CTX = C.CFUNCTYPE(C.c_int, C.c_void_p)
OP_CAPTURE = C.CFUNCTYPE(C.c_int, C.c_void_p, C.POINTER(C.c_uint32), C.c_size_t, C.POINTER(C.c_void_p))
OP_READOUT = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.POINTER(C.POINTER(C.c_uint32)), C.POINTER(C.c_size_t), C.c_size_t,
                         C.POINTER(C.c_float))
OP_MOVE = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p))
OP_FREE = C.CFUNCTYPE(None, C.c_void_p, C.c_void_p)
OP_MEM = C.CFUNCTYPE(C.c_int, C.c_void_p, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t))
OP_ERR = C.CFUNCTYPE(C.c_void_p, C.c_void_p)  # returns the address of a NUL-terminated buffer the callee keeps alive
OP_SIZE = C.CFUNCTYPE(C.c_size_t, C.c_void_p, C.c_size_t)
OP_CAPTURE_READOUT = C.CFUNCTYPE(C.c_int, C.c_void_p, C.POINTER(C.c_uint32), C.c_size_t, C.POINTER(C.POINTER(C.c_uint32)), C.POINTER(C.c_size_t),
                                 C.c_size_t, C.POINTER(C.c_void_p), C.POINTER(C.c_float))
OP_READOUT_MULTI = C.CFUNCTYPE(C.c_int, C.c_void_p, C.POINTER(C.c_void_p), C.c_size_t, C.POINTER(C.POINTER(C.c_uint32)), C.POINTER(C.c_size_t),
                               C.POINTER(C.c_uint32), C.c_size_t, C.POINTER(C.c_float))


class SchedEngineOps(C.Structure):
    """Mirrors ``dcd_sched_engine_ops``: the engine operations the scheduler's worker calls."""
    _fields_ = [
        ("ctx", C.c_void_p), ("readout_rows", C.c_int32), ("reserved0", C.c_int32),
        ("rebind_blas", OP_INT_CTX), ("capture_state", OP_CAPTURE), ("readout", OP_READOUT), ("offload", OP_MOVE), ("restore", OP_MOVE),
        ("state_free", OP_FREE), ("host_free", OP_FREE), ("trim_pools", OP_INT_CTX), ("mem_info", OP_MEM), ("last_error", OP_ERR),
        ("state_bytes_for", OP_SIZE), ("pass_reserve", OP_SIZE), ("readout_multi", OP_READOUT_MULTI), ("capture_readout", OP_CAPTURE_READOUT),
    ]


SCHED_STAT_NAMES = (
    "submitted", "waiting", "running", "channel", "worker_alive", "requests_gpu_hit", "requests_host_hit", "requests_miss",
    "reused_tokens", "captures", "state_tokens", "question_tokens", "questions_answered", "questions_failed", "questions_cancelled",
    "groups_success", "groups_failed", "group_requests", "group_questions", "cancelled_queued", "cancelled_at_reply", "offloads",
    "offload_bytes", "restores", "restore_bytes", "evict_gpu_entry_limit", "evict_gpu_byte_limit", "evict_gpu_offload_failed",
    "evict_host_budget", "oom_retry_capture", "oom_retry_question", "fail_headroom", "fail_state_restore", "fail_state_capture",
    "fail_state_offload", "fail_question_pass", "reject_queue_full", "reject_worker_stopped", "gpu_entries", "host_entries",
    "gpu_bytes", "host_bytes", "gpu_free_bytes", "cross_state_passes", "requests_fallback")


class SchedStats(C.Structure):
    """Mirrors ``dcd_sched_stats`` (all uint64)."""
    _fields_ = [(n, C.c_uint64) for n in SCHED_STAT_NAMES]


class ProfEntry(C.Structure):
    _fields_ = [("ms", C.c_double), ("work", C.c_double), ("launches", C.c_int64)]


# name -> (restype, argtypes); every symbol declared in include/decidra_b200.h
P, I, F, SZ = C.c_void_p, C.c_int, C.c_float, C.c_size_t
I32P, U32P, FP = C.POINTER(C.c_int32), C.POINTER(C.c_uint32), C.POINTER(C.c_float)
SIGNATURES = {
    "dcd_engine_create": (I, [C.POINTER(ModelConfig), C.POINTER(Options), I, C.POINTER(P)]),
    "dcd_engine_destroy": (None, [P]),
    "dcd_last_error": (C.c_char_p, [P]),
    "dcd_engine_info": (I, [P, C.POINTER(Info)]),
    "dcd_engine_init_random": (I, [P, C.c_uint64]),
    "dcd_engine_load_tensor": (I, [P, I, I, FP, SZ]),
    "dcd_engine_read_tensor": (I, [P, I, I, FP, SZ]),
    "dcd_engine_load_tensor_typed": (I, [P, I, I, P, I, SZ]),
    "dcd_checkpoint_open": (I, [C.c_char_p, C.POINTER(P)]),
    "dcd_checkpoint_close": (None, [P]),
    "dcd_checkpoint_count": (SZ, [P]),
    "dcd_checkpoint_name": (C.c_char_p, [P, SZ]),
    "dcd_checkpoint_tensor": (I, [P, C.c_char_p, C.POINTER(TensorInfo)]),
    "dcd_config_from_dir": (I, [C.c_char_p, C.POINTER(ModelConfig)]),
    "dcd_engine_load_checkpoint": (I, [P, P, C.c_char_p]),
    "dcd_sched_default_options": (None, [C.POINTER(SchedOptions)]),
    "dcd_scheduler_create": (I, [P, C.POINTER(SchedOptions), C.POINTER(P)]),
    "dcd_scheduler_create_with_ops": (I, [C.POINTER(SchedEngineOps), C.POINTER(SchedOptions), C.POINTER(P)]),
    "dcd_scheduler_destroy": (None, [P]),
    "dcd_scheduler_last_error": (C.c_char_p, []),
    "dcd_scheduler_submit": (I, [P, U32P, SZ, C.POINTER(U32P), C.POINTER(SZ), SZ, C.c_char_p, C.POINTER(P)]),
    "dcd_ticket_wait": (I, [P, FP, SZ]),
    "dcd_ticket_done": (I, [P]),
    "dcd_ticket_error": (C.c_char_p, [P]),
    "dcd_ticket_cancel": (None, [P]),
    "dcd_ticket_free": (None, [P]),
    "dcd_scheduler_stats": (I, [P, C.POINTER(SchedStats)]),
    "dcd_prompt_last_error": (C.c_char_p, []),
    "dcd_format_float": (I, [C.c_double, P, SZ, C.POINTER(SZ)]),
    "dcd_pyjson_dumps": (I, [C.c_char_p, SZ, P, SZ, C.POINTER(SZ)]),
    "dcd_pyjson_repr": (I, [C.c_char_p, SZ, I, P, SZ, C.POINTER(SZ)]),
    "dcd_pyjson_truthy": (I, [C.c_char_p, SZ, C.POINTER(C.c_int)]),
    "dcd_d3_parse_question": (I, [C.c_char_p, SZ, P, SZ, C.POINTER(SZ)]),
    "dcd_d3_render": (I, [C.c_char_p, SZ, C.c_char_p, SZ, C.POINTER(C.c_char_p), SZ, P, SZ, C.POINTER(SZ)]),
    "dcd_d3_state_end_char": (I, [C.c_char_p, SZ, C.c_char_p, SZ, C.POINTER(SZ)]),
    "dcd_d3_state_token_count": (I, [C.POINTER(SZ), SZ, SZ, C.POINTER(SZ)]),
    "dcd_d3_contains_media": (I, [C.c_char_p, SZ, C.POINTER(C.c_int)]),
    "dcd_rebind_blas": (I, [P]),
    "dcd_capture_state": (I, [P, U32P, SZ, P, C.POINTER(P)]),
    "dcd_readout_state_once_batch": (I, [P, P, C.POINTER(U32P), C.POINTER(SZ), SZ, FP]),
    "dcd_readout_state_once_flat": (I, [P, P, U32P, U32P, SZ, FP]),
    "dcd_readout_state_once_device": (I, [P, P, P, P, SZ, SZ, SZ, P]),
    "dcd_readout_multi_state_batch": (I, [P, C.POINTER(P), SZ, C.POINTER(U32P), C.POINTER(SZ), U32P, SZ, FP]),
    "dcd_capture_state_device": (I, [P, P, SZ, C.POINTER(P)]),
    "dcd_capture_and_readout": (I, [P, U32P, SZ, C.POINTER(U32P), C.POINTER(SZ), SZ, C.POINTER(P), FP]),
    "dcd_capture_and_readout_device": (I, [P, P, P, SZ, SZ, SZ, SZ, C.POINTER(P), P]),
    "dcd_decision_logits_split": (I, [P, U32P, SZ, SZ, FP]),
    "dcd_state_free": (None, [P, P]),
    "dcd_state_tokens": (SZ, [P]),
    "dcd_state_pos_end": (SZ, [P]),
    "dcd_state_bytes": (SZ, [P]),
    "dcd_state_bytes_for": (SZ, [P, SZ]),
    "dcd_pass_reserve_bytes": (SZ, [P, SZ]),
    "dcd_state_offload": (I, [P, P, C.POINTER(P)]),
    "dcd_state_restore": (I, [P, P, C.POINTER(P)]),
    "dcd_host_state_free": (None, [P]),
    "dcd_state_zero_gdn_state": (I, [P, P, I]),
    "dcd_state_zero_gdn_hist": (I, [P, P, I]),
    "dcd_state_read_tensor": (I, [P, P, I, I, FP, C.POINTER(SZ)]),
    "dcd_trim_pools": (I, [P]),
    "dcd_mem_info": (I, [P, C.POINTER(SZ), C.POINTER(SZ)]),
    "dcd_timer_begin": (I, [P]),
    "dcd_timer_end": (I, [P]),
    "dcd_timer_seconds": (C.c_double, [P]),
    "dcd_vision_encode": (I, [P, P, SZ]),
    "dcd_engine_sync": (I, [P]),
    "dcd_profile_enable": (I, [P, I]),
    "dcd_profile_read": (I, [P, C.POINTER(ProfEntry)]),
    "dcd_launch_count": (C.c_int64, [P]),
    "dcd_debug_bounded_wait_probe": (C.c_int, [P, C.c_int]),
    "dcd_debug_set_gemm_group_m": (None, [I]),
    "dcd_debug_layer_outputs": (I, [P, FP, SZ]),
    "dcd_block_cascade_mask": (I, [SZ, SZ, C.POINTER(C.c_uint8)]),
    "dcd_plan_chunks": (I, [C.POINTER(SZ), SZ, SZ, SZ, SZ, SZ, I32P, I32P, I32P]),
    "dcd_decode_answer": (I, [FP, I, F, I, FP, FP]),
    "dcd_pack": (I, [P, I32P, SZ, C.c_int32, I32P, I32P, I32P, I32P]),
    "dcd_k_gemm_bf16_tc": (I, [P, P, P, I, I, I, I, I, I, P, P]),
    "dcd_k_gemm_bf16_tc_resid": (I, [P, P, P, P, I, I, I, I, I, P, P]),
    "dcd_k_gemm_fp8_tc": (I, [P, P, P, I, I, I, I, I, P, P, I, P, P]),
    "dcd_k_quant_fp8_rows": (I, [P, SZ, P, P, I, I, F, I, P]),
    "dcd_k_quant_w4_g128": (I, [P, P, P, I, I, P]),
    "dcd_k_dequant_w4_g128": (I, [P, P, P, I, I, P]),
    "dcd_k_w4_repack": (I, [P, P, P, P, I, I, P]),
    "dcd_k_gemm_w4a16_tc": (I, [P, P, P, P, P, I, I, I, I, I, I, P, P]),
    "dcd_k_nvfp4_quant_rows": (I, [P, SZ, F, P, P, I, I, P]),
    "dcd_k_nvfp4_dequant_rows": (I, [P, P, P, I, I, P]),
    "dcd_k_nvfp4_fakequant_rows": (I, [P, SZ, F, P, I, I, P]),
    "dcd_k_nvfp4_tile_scales": (I, [P, P, I, I, P]),
    "dcd_k_nvfp4_quant_act_tiled": (I, [P, SZ, P, P, I, I, P]),
    "dcd_k_nvfp4_swiglu_quant_tiled": (I, [P, I, P, P, I, I, P]),
    "dcd_k_gemm_nvfp4_tc": (I, [P, P, P, P, P, I, I, I, I, P, I, P, I, P]),
    "dcd_k_gemm_nvfp4_tc_tiled": (I, [P, P, P, P, P, I, I, I, I, P, I, P, I, P, P, P, P]),
    "dcd_k_gemm_fma": (I, [P, P, P, I, I, I, I, P]),
    "dcd_k_rmsnorm": (I, [P, P, P, I, I, F, I, I, P]),
    "dcd_k_add_rmsnorm": (I, [P, P, P, P, P, I, I, F, I, P]),
    "dcd_k_rmsnorm_gated": (I, [P, P, I, P, P, I, I, I, F, I, P]),
    "dcd_k_silu_mul": (I, [P, P, P, SZ, I, P]),
    "dcd_k_add": (I, [P, P, P, SZ, I, P]),
    "dcd_k_conv1d_silu": (I, [P, I, P, P, P, P, P, I, I, I, P]),
    "dcd_k_gdn_prepare": (I, [P, I, P, P, I, P, P, P, P, P, P, I, I, I, I, I, P]),
    "dcd_k_gdn_recurrent": (I, [P, P, P, I, P, P, P, P, P, P, I, I, I, I, I, I, I, P]),
    "dcd_k_gdn_chunked": (I, [P, P, P, I, P, P, P, P, P, P, I, I, I, I, I, I, I, P]),
    "dcd_k_gdn_chunked_tc": (I, [P, P, P, I, P, P, P, P, P, P, I, I, I, I, I, I, P, I, P]),
    "dcd_k_gdn_wy_tc": (I, [P, P, P, I, P, P, P, P, P, P, I, I, I, I, I, I, P, I, P]),
    "dcd_k_gdn_wy_tc_phases": (I, [P, P, P, I, P, P, P, P, P, P, I, I, I, I, I, I, P, I, P, P]),
    "dcd_k_qk_norm_rope": (I, [P, I, P, I, P, P, P, P, P, I, P, P, I, I, I, I, I, F, P, I, P]),
    "dcd_k_attention": (I, [P, P, I, P, I, P, P, I, P, I, P, P, P, I, I, I, I, I, I, P]),
    "dcd_k_attention_tc": (I, [P, P, I, P, I, P, P, I, P, I, P, P, P, I, I, I, I, I, P, P]),
    "dcd_k_attention_tc_split": (I, [P, P, I, P, I, P, P, I, P, I, P, P, P, I, I, I, I, I, P, I, P, C.c_size_t, P]),
    "dcd_k_attention_tc_noalloc": (I, [P, P, I, P, I, P, P, I, P, I, P, P, I, I, I, I, I, P, P, C.c_char_p, SZ]),
    "dcd_k_readout": (I, [P, P, P, I, I, I, P]),
}

_lib = None


def load() -> C.CDLL:
    """Load the CUDA library; raise if it is absent (build it with ``python -m decidra_b200.build``)."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m decidra_b200.build`. "
                "decidra_b200 has no CPU or PyTorch fallback.")
        lib = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the library does not export a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib
