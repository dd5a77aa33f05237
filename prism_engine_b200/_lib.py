"""ctypes binding of ``libprism_cuda.so`` (the C ABI in ``include/prism_cuda.h``).

There is no CPU implementation behind this module: if the CUDA library is not
built, or no sm_100 device is present, loading or creating a context raises.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libprism_cuda.so")

OK = 0
E_NULL, E_ARG, E_NOTFOUND, E_CUDA, E_STATE, E_IO, E_COMM, E_TIMEOUT = -1, -2, -3, -4, -5, -6, -7, -8
NCCL_ID_BYTES = 128


class PrismCudaError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"prism_cuda error {code}: {msg}")
        self.code = code
        self.msg = msg


class ModelConfig(C.Structure):
    """Mirror of ``prism_model_config``."""

    _fields_ = [
        ("num_layers", C.c_uint32), ("hidden_size", C.c_uint32), ("num_heads", C.c_uint32),
        ("num_kv_heads", C.c_uint32), ("head_dim", C.c_uint32), ("intermediate_size", C.c_uint32),
        ("vocab_size", C.c_uint32), ("norm_eps", C.c_float), ("rope_theta", C.c_float),
        ("tie_word_embeddings", C.c_uint32), ("bits", C.c_uint32), ("max_seq", C.c_uint32),
        ("max_batch", C.c_uint32), ("rope_use_theta", C.c_uint32), ("rope_k", C.c_uint32),
        ("kv_int8", C.c_uint32), ("down_guard", C.c_uint32), ("kv_page_size", C.c_uint32), ("kv_pool_pages", C.c_uint32),
    ]


class CImagePlan(C.Structure):
    """Mirror of ``prism_cimage_plan``."""

    _fields_ = [("version", C.c_uint32), ("num_layers", C.c_uint32), ("n_nodes", C.c_uint32),
                ("n_gemm_nodes", C.c_uint32), ("kv_fp16", C.c_int32), ("architecture", C.c_char * 32),
                ("attention_strategy", C.c_char * 24), ("lm_head_backend", C.c_char * 16)]


# name -> (restype, argtypes); every symbol include/prism_cuda.h and include/prism_cuda_bench.h declare
_vp, _i32, _u32, _u64, _sz = C.c_void_p, C.c_int32, C.c_uint32, C.c_uint64, C.c_size_t
_cp = C.c_char_p
_pi32, _pu32 = C.POINTER(C.c_int32), C.POINTER(C.c_uint32)
SIGNATURES = {
    "prism_cuda_create": (C.c_int, [C.c_int, C.POINTER(_vp)]),
    "prism_cuda_destroy": (None, [_vp]),
    "prism_cuda_last_error": (_cp, [_vp]),
    "prism_cuda_stream": (_vp, [_vp]),
    "prism_cuda_synchronize": (C.c_int, [_vp]),
    "prism_cuda_set_option": (C.c_int, [_vp, _cp, C.c_int64]),
    "prism_cuda_launch_count": (_u64, [_vp]),
    "prism_cuda_upload_palettized": (C.c_int, [_vp, _cp, _vp, _sz, _u32, _u32, _u32, _pi32]),
    "prism_cuda_upload_palettized_shard": (C.c_int, [_vp, _cp, _vp, _sz, _u32, _u32, _u32, _u32, _u32, _u32, _u32, _pi32]),
    "prism_cuda_synth_palettized": (C.c_int, [_vp, _cp, _u32, _u32, _u32, _u64, C.c_float, _pi32]),
    "prism_cuda_find_tensor": (C.c_int, [_vp, _cp, _pi32]),
    "prism_cuda_tensor_dims": (C.c_int, [_vp, _i32, _pu32, _pu32, _pu32]),
    "prism_cuda_download_payload": (C.c_int, [_vp, _i32, _vp, _sz]),
    "prism_cuda_dequant": (C.c_int, [_vp, _i32, _vp]),
    "prism_cuda_dequant_dev": (C.c_int, [_vp, _i32, _vp]),
    "prism_cuda_free_tensor": (C.c_int, [_vp, _i32]),
    "prism_cuda_gemv": (C.c_int, [_vp, _i32, _vp, _vp]),
    "prism_cuda_gemv_key": (C.c_int, [_vp, _cp, _vp, _sz, _vp, _sz]),
    "prism_cuda_gemv_dev": (C.c_int, [_vp, _i32, _vp, _vp]),
    "prism_cuda_gemv_static_dev": (C.c_int, [_vp, _i32, _vp, _vp]),
    "prism_cuda_gemv_residual_dev": (C.c_int, [_vp, _i32, _vp, _vp, _vp]),
    "prism_cuda_fused_gate_up": (C.c_int, [_vp, _i32, _i32, _vp, _vp]),
    "prism_cuda_fused_gate_up_key": (C.c_int, [_vp, _cp, _cp, _vp, _sz, _vp, _sz]),
    "prism_cuda_fused_gate_up_dev": (C.c_int, [_vp, _i32, _i32, _vp, _vp]),
    "prism_cuda_mlp": (C.c_int, [_vp, _i32, _i32, _i32, _vp, _vp]),
    "prism_cuda_mlp_dev": (C.c_int, [_vp, _i32, _i32, _i32, _vp, _vp]),
    "prism_cuda_gemm": (C.c_int, [_vp, _i32, _vp, _u32, _vp]),
    "prism_cuda_gemm_dev": (C.c_int, [_vp, _i32, _vp, _u32, _vp]),
    "prism_cuda_rms_norm": (C.c_int, [_vp, _vp, _vp, _u32, C.c_float]),
    "prism_cuda_rope": (C.c_int, [_vp, _vp, _u32, C.c_int64, _u32, C.c_float]),
    "prism_cuda_softmax": (C.c_int, [_vp, _vp, _vp, _u32]),
    "prism_cuda_silu": (C.c_int, [_vp, _vp, _u32]),
    "prism_cuda_vec_add": (C.c_int, [_vp, _vp, _vp, _u32]),
    "prism_cuda_attention": (C.c_int, [_vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _vp]),
    "prism_cuda_argmax": (C.c_int, [_vp, _vp, _u32, _pu32]),
    "prism_cuda_engine_create": (C.c_int, [_vp, C.POINTER(ModelConfig), C.POINTER(_vp)]),
    "prism_cuda_engine_destroy": (None, [_vp]),
    "prism_cuda_engine_bind": (C.c_int, [_vp, _u32, _u32, _i32]),
    "prism_cuda_engine_bind_by_keys": (C.c_int, [_vp, _cp]),
    "prism_cuda_engine_load_cimage": (C.c_int, [_vp, _cp, _cp]),
    "prism_cuda_engine_synth_weights": (C.c_int, [_vp, _u64, C.c_float]),
    "prism_cuda_engine_generate": (C.c_int, [_vp, _vp, _u32, _u32, _u32, _vp, _vp]),
    "prism_cuda_engine_reset": (C.c_int, [_vp, _u32]),
    "prism_cuda_engine_step": (C.c_int, [_vp, _vp, _vp, _vp]),
    "prism_cuda_engine_decode": (C.c_int, [_vp, _vp, _u32, _vp]),
    "prism_cuda_engine_step_bytes": (_u64, [_vp]),
    "prism_cuda_engine_last_ms": (C.c_double, [_vp]),
    "prism_cuda_engine_position": (_u32, [_vp]),
    "prism_cuda_engine_last_device_ms": (C.c_double, [_vp]),
    "prism_cuda_engine_kernels_per_step": (_u32, [_vp]),
    "prism_cuda_engine_profile_gemv": (C.c_int, [_vp, _u32, C.POINTER(C.c_double), C.POINTER(_u64), _pu32]),
    "prism_cuda_bench_cycle": (C.c_int, [_vp, C.c_int, _pi32, _u32, _u32, _vp, C.POINTER(C.c_double)]),
    "prism_cuda_engine_profile_part": (C.c_int, [_vp, _u32, _u32, C.POINTER(C.c_double), _pu32]),
    "prism_cuda_load_cimage": (C.c_int, [_vp, _cp, _pu32]),
    "prism_cuda_bench_gemm": (C.c_int, [_vp, _i32, _vp, _u32, _u32, C.POINTER(C.c_double)]),
    "prism_cuda_tp_unique_id": (C.c_int, [_vp]),
    "prism_cuda_tp_init": (C.c_int, [_vp, C.c_int, C.c_int, _vp]),
    "prism_cuda_tp_world": (C.c_int, [_vp, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "prism_cuda_tp_peer_ready": (C.c_int, [_vp]),
    "prism_cuda_palettize": (C.c_int, [_vp, C.POINTER(C.c_float), C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
                                       C.POINTER(C.c_uint8), C.c_size_t]),
    "prism_cuda_palettize_dev": (C.c_int, [_vp, _vp, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, _vp]),
    "prism_cuda_gemv_partition": (C.c_int, [C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
                                            C.POINTER(C.c_uint32), C.POINTER(C.c_uint32), C.c_uint32]),
    "prism_cuda_gemv_partition_ctas": (C.c_uint32, [C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32]),
    "prism_cuda_tp_all_reduce_dev": (C.c_int, [_vp, _vp, _sz]),
    "prism_cuda_tp_peer_reason": (_cp, [_vp]),
    "prism_cuda_tp_all_reduce_resid_dev": (C.c_int, [_vp, _vp, _vp, _sz]),
    "prism_cuda_tp_init_loopback": (C.c_int, [_vp, C.c_int, C.c_int]),
    "prism_cuda_kv_init": (C.c_int, [_vp, _u32, _u32, _u32]),
    "prism_cuda_kv_append": (C.c_int, [_vp, _u32, _vp, _vp, _u64]),
    "prism_cuda_attention_kv": (C.c_int, [_vp, _u32, _vp, _u32, _u32, _u32, _u32, _vp]),
    "prism_cuda_attention_step_kv": (C.c_int, [_vp, _u32, _vp, _vp, _vp, _u64, _u32, _u32, _u32, _u32, C.c_float, _vp]),
    "prism_cuda_load_cimage_cached": (C.c_int, [_vp, _cp, _cp, _pu32, C.POINTER(C.c_int)]),
    "prism_cuda_cimage_plan": (C.c_int, [_vp, C.POINTER(CImagePlan)]),
}

_lib = None


def load() -> C.CDLL:
    """Loads the CUDA library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m prism_engine_b200.build` "
                "(there is no CPU implementation to fall back to)")
        L = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)  # AttributeError if the library does not export a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(ctx, rc: int) -> None:
    if rc != OK:
        msg = load().prism_cuda_last_error(ctx)
        raise PrismCudaError(rc, msg.decode("utf-8", "replace") if msg else "")
