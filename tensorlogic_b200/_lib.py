"""ctypes view of libtlcuda.so (the C ABI declared in include/tlcuda.h).

The library is built in-tree by ``tensorlogic_b200.build``.  There is no
fallback: if the shared object is missing, or no CUDA device is present, the
calls fail loudly.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtlcuda.so")

OK = 0
ERR_SHAPE_MISMATCH, ERR_INVALID_OPERATION, ERR_DEVICE, ERR_CUDA = -1, -2, -3, -4
ERR_ALLOCATION, ERR_LOAD, ERR_BUFFER_EXHAUSTED, ERR_INDEX = -5, -6, -7, -8
ERR_INVALID_DIMENSION, ERR_TIMEOUT, ERR_COMM = -9, -10, -11

TYPE_F32, TYPE_F16, TYPE_Q4_0, TYPE_Q8_0 = 0, 1, 2, 8
SPLIT_NONE, SPLIT_ROWS, SPLIT_COLS = 0, 1, 2

_ERROR_NAMES = {
    -1: "ShapeMismatch", -2: "InvalidOperation", -3: "DeviceConversionError", -4: "CudaError",
    -5: "AllocationError", -6: "LoadError", -7: "BufferExhausted", -8: "IndexOutOfBounds",
    -9: "InvalidDimension", -10: "Timeout", -11: "CommError",
}


class TensorError(RuntimeError):
    """Mirror of TensorLogic's TensorError (src/error.rs:9-49): ``kind`` names the variant."""

    def __init__(self, code: int, message: str):
        self.code = code
        self.kind = _ERROR_NAMES.get(code, f"Error{code}")
        super().__init__(f"{self.kind}: {message}")


class PoolStats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("total_pooled", "size_classes", "total_memory", "reuse_count",
                                          "allocation_count", "eviction_count", "live_bytes")]


class LlamaConfig(C.Structure):
    """tlc_llama_config of include/tlcuda.h."""
    _fields_ = [("n_layers", C.c_int32), ("d_model", C.c_int32), ("n_heads", C.c_int32), ("n_kv_heads", C.c_int32),
                ("head_dim", C.c_int32), ("ffn_dim", C.c_int32), ("vocab", C.c_int32), ("rms_eps", C.c_float),
                ("rope_base", C.c_uint32), ("max_seq", C.c_int32), ("max_batch", C.c_int32),
                ("max_prefill", C.c_int32), ("tp_rank", C.c_int32), ("tp_size", C.c_int32),
                ("logits_all_rows", C.c_int32), ("no_graph", C.c_int32)]


vp, i32, i64, u32, u64, sz, f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_uint32, C.c_uint64, C.c_size_t, C.c_float
P = C.POINTER

# name -> (restype, argtypes).  Every function declared in include/tlcuda.h.
PROTOTYPES = {
    "tlc_last_error": (C.c_char_p, []),
    "tlc_version": (C.c_char_p, []),
    "tlc_init": (i32, [i32, P(vp)]),
    "tlc_destroy": (i32, [vp]),
    "tlc_set_option": (i32, [vp, C.c_char_p, i64]),
    "tlc_selftest_wait_timeout": (i32, [vp, i32]),
    "tlc_device_name": (i32, [vp, C.c_char_p, sz]),
    "tlc_mem_info": (i32, [vp, P(sz), P(sz)]),
    "tlc_sm_count": (i32, [vp, P(i32)]),
    "tlc_synchronize": (i32, [vp]),
    "tlc_stream": (vp, [vp]),
    "tlc_launch_count": (u64, [vp]),
    "tlc_perf_report": (i32, [vp, C.c_char_p, sz, i32, P(sz)]),
    "tlc_alloc": (i32, [vp, sz, P(vp)]),
    "tlc_free": (i32, [vp]),
    "tlc_buf_ptr": (vp, [vp]),
    "tlc_buf_size": (sz, [vp]),
    "tlc_pool_stats_get": (i32, [vp, P(PoolStats)]),
    "tlc_pool_trim": (i32, [vp, sz]),
    "tlc_upload": (i32, [vp, vp, vp, sz]),
    "tlc_download": (i32, [vp, vp, vp, sz]),
    "tlc_host_alloc": (i32, [sz, P(vp)]),
    "tlc_host_free": (i32, [vp]),
    "tlc_qtensor_create": (i32, [vp, i32, i64, i64, vp, sz, i32, i32, i32, P(vp)]),
    "tlc_qtensor_create_synthetic": (i32, [vp, i32, i64, i64, u64, u64, i32, i32, i32, i32, P(vp)]),
    "tlc_synth_blocks_host": (i32, [i32, u64, u64, i32, i64, i64, vp]),
    "tlc_fill_normal_f16": (i32, [vp, vp, sz, u64, u64, f32, f32]),
    "tlc_qtensor_create_normal_f16": (i32, [vp, i64, i64, u64, u64, f32, f32, P(vp)]),
    "tlc_qtensor_destroy": (i32, [vp]),
    "tlc_qtensor_info": (i32, [vp, P(i32), P(i64), P(i64), P(sz), P(vp)]),
    "tlc_qtensor_blocks": (i32, [vp, vp, vp]),
    "tlc_tiled_bytes": (sz, [i32, i64, i64]),
    "tlc_tile_blocks_host": (i32, [i32, i64, i64, vp, vp]),
    "tlc_dequant": (i32, [vp, vp, vp]),
    "tlc_linear": (i32, [vp, vp, vp, i32, i64, vp, vp]),
    "tlc_linear_host": (i32, [vp, vp, vp, i32, i64, vp, vp]),
    "tlc_rms_norm": (i32, [vp, vp, vp, vp, i32, i32, f32]),
    "tlc_rope": (i32, [vp, vp, vp, i32, i32, i32, i32, u32, vp]),
    "tlc_rope_table": (i32, [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32]),
    "tlc_matmul": (i32, [vp, vp, vp, vp, i32, i32, i32, i32]),
    "tlc_sigmoid": (i32, [vp, vp, vp, sz]),
    "tlc_mul": (i32, [vp, vp, vp, vp, sz]),
    "tlc_add": (i32, [vp, vp, vp, vp, sz]),
    "tlc_swiglu": (i32, [vp, vp, vp, vp, sz]),
    "tlc_softmax": (i32, [vp, vp, vp, i32, i32]),
    "tlc_embedding": (i32, [vp, vp, i32, i32, P(i32), i32, vp]),
    "tlc_norm_linear_multi": (i32, [vp, i32, P(vp), P(vp), P(i32), vp, i32, vp, f32, i32, u32, vp]),
    "tlc_swiglu_gate_up": (i32, [vp, vp, vp, vp, i32, vp, f32, vp]),
    "tlc_linear_residual": (i32, [vp, vp, vp, i32, vp, vp]),
    "tlc_kvcache_create": (i32, [vp, i32, i32, i32, i32, i32, P(vp)]),
    "tlc_kvcache_destroy": (i32, [vp]),
    "tlc_kvcache_layer_ptrs": (i32, [vp, i32, P(vp), P(vp)]),
    "tlc_kvcache_append": (i32, [vp, vp, i32, vp, vp, i32, i32, vp]),
    "tlc_attention": (i32, [vp, vp, i32, vp, vp, i32, i32, i32, i32, vp, i32, f32]),
    "tlc_attention_decode_static": (i32, [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp, i32, f32]),
    "tlc_attention_decode_static_status": (i32, [vp, vp]),
    "tlc_model_load_gguf": (i32, [vp, C.c_char_p, i32, i32, P(vp)]),
    "tlc_gguf_open": (i32, [C.c_char_p, P(vp)]),
    "tlc_gguf_close": (i32, [vp]),
    "tlc_gguf_tensor_count": (i32, [vp]),
    "tlc_gguf_tensor_info": (i32, [vp, i32, P(C.c_char_p), P(i32), P(i64), P(i64), P(u64), P(u64)]),
    "tlc_gguf_meta_num": (i32, [vp, C.c_char_p, P(C.c_double)]),
    "tlc_gguf_meta_str": (C.c_char_p, [vp, C.c_char_p]),
    "tlc_gguf_data_start": (u64, [vp]),
    "tlc_model_create": (i32, [vp, P(vp)]),
    "tlc_model_add": (i32, [vp, C.c_char_p, vp]),
    "tlc_model_destroy": (i32, [vp]),
    "tlc_model_get": (i32, [vp, C.c_char_p, P(vp)]),
    "tlc_model_tensor_count": (i32, [vp]),
    "tlc_model_tensor_name": (C.c_char_p, [vp, i32]),
    "tlc_model_meta_num": (i32, [vp, C.c_char_p, P(C.c_double)]),
    "tlc_model_meta_str": (C.c_char_p, [vp, C.c_char_p]),
    "tlc_llama_create": (i32, [vp, vp, P(LlamaConfig), P(vp)]),
    "tlc_llama_destroy": (i32, [vp]),
    "tlc_llama_prefill": (i32, [vp, P(i32), i32, i32, vp, i32, P(i32)]),
    "tlc_llama_set_state": (i32, [vp, i32, P(i32), P(i32)]),
    "tlc_llama_decode_host": (i32, [vp, i32, P(i32), P(i32), vp]),
    "tlc_llama_decode_enqueue": (i32, [vp, i32, i32]),
    "tlc_llama_read_state": (i32, [vp, i32, P(i32), P(i32)]),
    "tlc_llama_step_trace": (i32, [vp, i32, P(u64), sz]),
    "tlc_llama_decode_enqueue_parts": (i32, [vp, i32, i32, i32]),
    "tlc_llama_launches_per_step": (i32, [vp, i32]),
    "tlc_llama_cache": (vp, [vp]),
    "tlc_llama_set_sampling": (i32, [vp, f32, u64]),
    "tlc_sample_uniform_host": (f32, [u64, u32, u32]),
    "tlc_temperature_sample": (i32, [vp, vp, i32, i32, f32, P(f32), P(i32)]),
    "tlc_weight_cache_open": (i32, [vp, C.c_char_p, i64, P(vp)]),
    "tlc_weight_cache_close": (i32, [vp]),
    "tlc_weight_cache_get": (i32, [vp, C.c_char_p, P(vp)]),
    "tlc_weight_cache_contains": (i32, [vp, C.c_char_p]),
    "tlc_weight_cache_clear": (i32, [vp]),
    "tlc_weight_cache_stats": (i32, [vp, P(i64), P(i64), P(u64), P(u64), P(u64)]),
    "tlc_comm_unique_id": (i32, [vp]),
    "tlc_comm_init": (i32, [vp, vp, i32, i32, P(vp)]),
    "tlc_comm_destroy": (i32, [vp]),
    "tlc_comm_rank": (i32, [vp]),
    "tlc_comm_size": (i32, [vp]),
    "tlc_allreduce_f16": (i32, [vp, vp, vp, sz]),
    "tlc_allgather_f16": (i32, [vp, vp, vp, vp, sz]),
    "tlc_comm_p2p_export": (i32, [vp, sz, vp]),
    "tlc_comm_p2p_import": (i32, [vp, vp]),
    "tlc_comm_p2p_ready": (i32, [vp]),
    "tlc_allreduce_residual_f16": (i32, [vp, vp, vp, vp, vp, sz]),
    "tlc_llama_set_comm": (i32, [vp, vp]),
}

_lib = None


def load() -> C.CDLL:
    """dlopen libtlcuda.so and attach prototypes.  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m tensorlogic_b200.build` "
            "(needs nvcc); there is no fallback implementation")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(rc: int) -> None:
    if rc != OK:
        msg = load().tlc_last_error()
        raise TensorError(rc, msg.decode("utf-8", "replace") if msg else "")
