"""ctypes view of include/leafcutter_b200.h (the C ABI of libleafcutter_b200.so)."""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libleafcutter_b200.so")

LC_OK = 0
LC_ERR_INVALID, LC_ERR_UNSUPPORTED, LC_ERR_CUDA, LC_ERR_OOM, LC_ERR_KV_FULL, LC_ERR_MISSING, LC_ERR_STATE = -1, -2, -3, -4, -5, -6, -7
STATUS_NAMES = {0: "LC_OK", -1: "LC_ERR_INVALID", -2: "LC_ERR_UNSUPPORTED", -3: "LC_ERR_CUDA", -4: "LC_ERR_OOM",
                -5: "LC_ERR_KV_FULL", -6: "LC_ERR_MISSING", -7: "LC_ERR_STATE"}

TYPE_F32, TYPE_F16, TYPE_Q4_0, TYPE_Q8_0, TYPE_Q4_K, TYPE_Q5_K, TYPE_Q6_K, TYPE_IQ4_NL = 0, 1, 2, 8, 12, 13, 14, 20
# (elements per block, bytes per block): rust/src/model/quant.rs:186-262
QUANT_GEOMETRY = {TYPE_F32: (1, 4), TYPE_F16: (1, 2), TYPE_Q4_0: (32, 18), TYPE_Q8_0: (32, 34), TYPE_Q4_K: (256, 144),
                  TYPE_Q5_K: (256, 176), TYPE_Q6_K: (256, 210), TYPE_IQ4_NL: (32, 18)}


class ModelConfig(C.Structure):
    _fields_ = [("hidden_size", C.c_int32), ("num_layers", C.c_int32), ("num_heads", C.c_int32),
                ("num_kv_heads", C.c_int32), ("intermediate_size", C.c_int32), ("max_seq_len", C.c_int32),
                ("vocab_size", C.c_int32), ("rope_theta", C.c_float), ("rms_eps", C.c_float),
                ("kv_dtype", C.c_int32), ("rope_mode", C.c_int32), ("n_experts", C.c_int32), ("top_k", C.c_int32),
                ("max_seqs", C.c_int32), ("kv_page_tokens", C.c_int32), ("kv_pool_tokens", C.c_int64),
                ("device", C.c_int32), ("tp_size", C.c_int32), ("tp_rank", C.c_int32), ("reserved", C.c_int32 * 5)]


class Counters(C.Structure):
    _fields_ = [("tokens_prefilled", C.c_uint64), ("tokens_decoded", C.c_uint64), ("forward_calls", C.c_uint64),
                ("kernel_launches", C.c_uint64), ("weight_bytes", C.c_uint64), ("kv_pages_in_use", C.c_uint64),
                ("kv_pages_total", C.c_uint64), ("sanitize_hits", C.c_uint64), ("algo_bytes_last_step", C.c_uint64),
                ("reserved", C.c_uint64 * 7)]


class CorruptTensor(C.Structure):
    _fields_ = [("name", C.c_char * 112), ("ggml_type", C.c_uint32), ("reserved", C.c_uint32), ("blocks_total", C.c_uint64),
                ("blocks_bad", C.c_uint64)]


class GgufReport(C.Structure):
    _fields_ = [("architecture", C.c_char * 16), ("arch_supported", C.c_int32), ("total_tensors", C.c_int32),
                ("tensors_by_type", C.c_int32 * 32), ("unsupported_types", C.c_uint32), ("n_missing", C.c_int32),
                ("n_extra", C.c_int32), ("can_run", C.c_int32), ("n_corrupt_tensors", C.c_int32),
                ("total_blocks_checked", C.c_uint64), ("total_bad_blocks", C.c_uint64), ("config", ModelConfig)]


TOKEN_CB = C.CFUNCTYPE(None, C.c_int64, C.c_void_p)

_f = C.POINTER(C.c_float)
_sz = C.c_size_t
_vp = C.c_void_p
_i32 = C.c_int32
_u32 = C.c_uint32
_u64 = C.c_uint64

# name -> (restype, argtypes); every name here is declared in include/leafcutter_b200.h
SIGNATURES = {
    "lc_last_error": (C.c_char_p, []),
    "lc_version": (C.c_char_p, []),
    "lc_device_count": (_i32, []),
    "lc_set_device": (_i32, [_i32]),
    "lc_tensor_bytes": (_sz, [_u32, _sz]),
    "lc_matmul_f32": (_i32, [_vp, _vp, _sz, _sz, _sz, _vp]),
    "lc_vec_add": (_i32, [_vp, _vp, _sz, _vp]),
    "lc_vec_mul": (_i32, [_vp, _vp, _sz, _vp]),
    "lc_vec_scale": (_i32, [_vp, C.c_float, _sz, _vp]),
    "lc_vec_scale_mul": (_i32, [_vp, C.c_float, _vp, _sz, _vp]),
    "lc_rms_norm": (_i32, [_vp, _vp, C.c_float, _sz, _sz, _vp]),
    "lc_silu": (_i32, [_vp, _sz, _vp]),
    "lc_softmax": (_i32, [_vp, _sz, _sz, _vp]),
    "lc_sum_sq": (_i32, [_vp, _sz, _vp]),
    "lc_dequantize": (_i32, [_u32, _vp, _sz, _vp]),
    "lc_qmatmul": (_i32, [_u32, _vp, _vp, _sz, _sz, _sz, _vp]),
    "lc_q8_0_matmul_shard": (_i32, [_vp, _vp, _vp, _sz, _sz, _sz, _vp]),
    "lc_q4_0_matmul_shard": (_i32, [_vp, _vp, _vp, _sz, _sz, _sz, _vp]),
    "lc_rope": (_i32, [_vp, _sz, _sz, _sz, C.c_float, _sz]),
    "lc_argmax": (_i32, [_vp, _sz, _vp]),
    "lc_dev_alloc": (_i32, [_sz, C.POINTER(_vp)]),
    "lc_dev_free": (_i32, [_vp]),
    "lc_dev_upload": (_i32, [_vp, _vp, _sz]),
    "lc_dev_download": (_i32, [_vp, _vp, _sz]),
    "lc_dev_sync": (_i32, []),
    "lc_qmatmul_dev": (_i32, [_u32, _vp, _vp, _sz, _sz, _sz, _vp]),
    "lc_dequantize_dev": (_i32, [_u32, _vp, _sz, _vp]),
    "lc_attention_decode_dev": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _vp]),
    "lc_attention_decode_static": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _vp]),
    "lc_timer_begin": (_i32, []),
    "lc_timer_end": (_i32, [_f]),
    "lc_flush_l2": (_i32, []),
    "lc_synth_tensor_host": (_i32, [_u32, _u64, C.c_char_p, C.c_float, _sz, _vp]),
    "lc_synth_tensor_dev": (_i32, [_u32, _u64, C.c_char_p, C.c_float, _sz, _vp]),
    "lc_synth_tokens": (_i32, [_u64, _sz, C.c_int64, _vp]),
    "lc_model_create": (_i32, [C.POINTER(ModelConfig), C.POINTER(_vp)]),
    "lc_model_set_tensor": (_i32, [_vp, C.c_char_p, _u32, C.POINTER(_u64), _i32, _vp, _sz]),
    "lc_model_synth_tensor": (_i32, [_vp, C.c_char_p, _u32, C.POINTER(_u64), _i32, _u64, C.c_float]),
    "lc_model_get_tensor": (_i32, [_vp, C.c_char_p, _vp, _sz]),
    "lc_model_finalize": (_i32, [_vp]),
    "lc_model_destroy": (_i32, [_vp]),
    "lc_model_load_gguf": (_i32, [C.c_char_p, C.POINTER(ModelConfig), C.POINTER(_vp)]),
    "lc_model_get_config": (_i32, [_vp, C.POINTER(ModelConfig)]),
    "lc_sample_top_p": (_i32, [_vp, _sz, C.c_float, C.c_float, C.c_float, C.POINTER(C.c_int64)]),
    "lc_model_set_seed": (_i32, [_vp, _u64]),
    "lc_seeded_uniform": (C.c_float, [_u64, _u64]),
    "lc_scan_blocks": (_i32, [_u32, _vp, _sz, C.POINTER(_u64), C.POINTER(_u64)]),
    "lc_scan_blocks_dev": (_i32, [_u32, _vp, _sz, C.POINTER(_u64), C.POINTER(_u64)]),
    "lc_gguf_inspect": (_i32, [C.c_char_p, _i32, C.POINTER(GgufReport), C.POINTER(CorruptTensor), _i32, C.c_char_p, _sz]),
    "lc_shard_engine_load": (_i32, [C.c_char_p, _i32, _i32, C.POINTER(_vp)]),
    "lc_shard_engine_forward": (_i32, [_vp, _vp, _i32, _vp, _vp]),
    "lc_shard_engine_generate": (_i32, [_vp, _vp, _i32, _i32, C.c_float, C.c_float, _vp, C.POINTER(_i32)]),
    "lc_shard_engine_set_seed": (_i32, [_vp, _u64]),
    "lc_shard_engine_reset_kv_cache": (_i32, [_vp]),
    "lc_shard_engine_kv_cache_memory_bytes": (_i32, [_vp, C.POINTER(_u64)]),
    "lc_shard_engine_destroy": (_i32, [_vp]),
    "lc_kv_clear": (_i32, [_vp, _i32]),
    "lc_kv_memory_bytes": (_i32, [_vp, C.POINTER(_u64)]),
    "lc_kv_length": (_i32, [_vp, _i32, C.POINTER(_i32)]),
    "lc_forward": (_i32, [_vp, _vp, _i32, _vp]),
    "lc_forward_batch": (_i32, [_vp, _i32, _vp, _vp, _vp, _vp, _vp]),
    "lc_generate": (_i32, [_vp, _vp, _i32, _i32, C.c_float, C.c_float, _i32, _vp, C.POINTER(_i32), TOKEN_CB, _vp]),
    "lc_decode_loop": (_i32, [_vp, _i32, _vp, _vp, _i32, _vp, _f]),
    "lc_get_counters": (_i32, [_vp, C.POINTER(Counters)]),
    "lc_reset_counters": (_i32, [_vp]),
    "lc_probe_attention": (_i32, [_vp, _i32, _vp, _i32, _vp]),
    "lc_probe_ffn": (_i32, [_vp, _i32, _vp, _i32, _vp]),
    "lc_dist_unique_id": (_i32, [_vp]),
    "lc_dist_init": (_i32, [_i32, _i32, _vp]),
    "lc_dist_set_backend": (_i32, [_i32]),
    "lc_dist_finalize": (_i32, []),
    "lc_dist_debug": (_i32, [_vp]),
    "lc_dist_info": (_i32, [C.POINTER(_i32), C.POINTER(_i32), C.POINTER(_i32)]),
    "lc_dist_time_allreduce": (_i32, [_sz, _i32, C.POINTER(C.c_float)]),
    "lc_tcgen05_probe": (_i32, [C.POINTER(C.c_double)]),
    "lc_model_group": (_i32, [C.POINTER(_vp), _i32]),
    "lc_shard_plan": (_i32, [C.POINTER(ModelConfig), C.c_char_p, _vp, _i32, C.POINTER(_i32), C.POINTER(_u64), C.POINTER(_u64)]),
}


class LeafcutterError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(status, status)}: {message}")
        self.status = status


_lib = None


def load() -> C.CDLL:
    """Loads the shared library.  There is no fallback: a missing library is an error."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing; build it with `python -m leafcutterllm_b200.build` "
                          "(needs nvcc).  leafcutterllm_b200 has no CPU or PyTorch fallback.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means the .so does not match the header
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(status: int) -> None:
    if status != LC_OK:
        raise LeafcutterError(status, load().lc_last_error().decode("utf-8", "replace"))
