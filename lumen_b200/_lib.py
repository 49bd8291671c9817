"""ctypes loader for liblumen_b200.so and the prototypes of include/lumen_b200.h.

There is no CPU fallback: if the shared library is missing this module raises, and every call
on a machine without a B200 returns LUMEN_ERR_CUDA, which `check` turns into an exception.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "liblumen_b200.so"

OK = 0
ERR_INVALID, ERR_SHAPE, ERR_KV_OVERFLOW, ERR_ROPE_RANGE, ERR_EMBED_RANGE, ERR_CACHE_COUNT = 1, 2, 3, 4, 5, 6
ERR_CUDA, ERR_NCCL, ERR_TIMEOUT, ERR_DTYPE, ERR_PARAM_NAME, ERR_UNSUPPORTED, ERR_MISSING_PARAM = 7, 8, 9, 10, 11, 12, 13
F32, BF16 = 0, 1
NCCL_ID_BYTES = 128


class SampleParamsC(C.Structure):
    """`lumen_sample_params` (arguments of sample_top_p, src/main.rs:74-80, plus the uniform draw)."""

    _fields_ = [("temperature", C.c_float), ("top_p", C.c_float), ("repetition_penalty", C.c_float),
                ("recent_tokens", C.POINTER(C.c_int32)), ("n_recent", C.c_size_t), ("uniform", C.c_float)]


class LlamaConfigC(C.Structure):
    """`lumen_llama_config` (LlamaConfig, src/models/llama.rs:11-21, + head_dim, qk_norm, weight_dtype)."""

    _fields_ = [
        ("vocab_size", C.c_size_t), ("hidden_size", C.c_size_t), ("intermediate_size", C.c_size_t),
        ("num_hidden_layers", C.c_size_t), ("num_attention_heads", C.c_size_t),
        ("num_key_value_heads", C.c_size_t), ("rms_norm_eps", C.c_float), ("max_seq_len", C.c_size_t),
        ("rope_theta", C.c_float), ("head_dim", C.c_size_t), ("qk_norm", C.c_int), ("weight_dtype", C.c_int),
    ]


_P = C.c_void_p
_PP = C.POINTER(C.c_void_p)
_SZ = C.c_size_t
_SZP = C.POINTER(C.c_size_t)
_I = C.c_int
_F = C.c_float
_FP = C.c_void_p  # float* passed as a raw address (numpy / torch / device pointers)

# name -> (restype, argtypes); one entry per declaration in include/lumen_b200.h
PROTOTYPES = {
    "lumen_nccl_unique_id": (_I, [_P]),
    "lumen_ctx_create": (_I, [_I, _I, _I, _P, _PP]),
    "lumen_ctx_destroy": (_I, [_P]),
    "lumen_ctx_synchronize": (_I, [_P]),
    "lumen_ctx_stream": (_P, [_P]),
    "lumen_ctx_launch_count": (C.c_uint64, [_P]),
    "lumen_last_error": (C.c_char_p, [_P]),
    "lumen_status_string": (C.c_char_p, [_I]),
    "lumen_version": (_I, []),
    "lumen_tensor_from_host": (_I, [_P, _FP, _SZP, _I, _PP]),
    "lumen_tensor_from_host_bf16": (_I, [_P, _P, _SZP, _I, _PP]),
    "lumen_tensor_empty": (_I, [_P, _SZP, _I, _I, _PP]),
    "lumen_tensor_ndim": (_I, [_P]),
    "lumen_tensor_shape": (_I, [_P, _SZP]),
    "lumen_tensor_numel": (_SZ, [_P]),
    "lumen_tensor_dtype": (_I, [_P]),
    "lumen_tensor_data": (_P, [_P]),
    "lumen_tensor_to_host": (_I, [_P, _FP]),
    "lumen_tensor_set": (_I, [_P, _FP]),
    "lumen_tensor_reshape": (_I, [_P, C.POINTER(C.c_int64), _I, _PP]),
    "lumen_tensor_free": (_I, [_P]),
    "lumen_matmul": (_I, [_P, _P, _P, _PP]),
    "lumen_linear_forward": (_I, [_P, _P, _P, _P, _PP]),
    "lumen_rmsnorm": (_I, [_P, _P, _P, _F, _PP]),
    "lumen_silu": (_I, [_P, _P, _PP]),
    "lumen_mul": (_I, [_P, _P, _P, _PP]),
    "lumen_add": (_I, [_P, _P, _P, _PP]),
    "lumen_embedding": (_I, [_P, _P, _P, _PP]),
    "lumen_fused_softmax": (_I, [_P, _P, _F, _I, _PP]),
    "lumen_gemv": (_I, [_P, _FP, _P, _I, _I, _SZ, _SZ, _FP]),
    "lumen_gemv_repeat": (_I, [_P, _FP, _P, _SZ, _I, _I, _SZ, _SZ, _FP, _SZ, C.POINTER(C.c_float)]),
    "lumen_attention_decode_repeat": (_I, [_P, _FP, _FP, _FP, _SZ, _P, _SZ, _P, _FP, _SZ, C.POINTER(C.c_float)]),
    "lumen_gemv_kn_static": (_I, [_P, _FP, _P, _I, _SZ, _SZ, _FP]),
    "lumen_rope_new": (_I, [_P, _SZ, _SZ, _F, _PP]),
    "lumen_rope_forward": (_I, [_P, _P, _SZ, _PP]),
    "lumen_rope_free": (_I, [_P]),
    "lumen_kv_new": (_I, [_P, _SZ, _SZ, _SZ, _SZ, _PP]),
    "lumen_kv_reset": (_I, [_P]),
    "lumen_kv_len": (_SZ, [_P]),
    "lumen_kv_free": (_I, [_P]),
    "lumen_kv_read": (_I, [_P, _FP, _FP]),
    "lumen_kv_write": (_I, [_P, _FP, _FP, _SZ]),
    "lumen_llama_kv_new": (_I, [_P, _SZ, _SZ, _SZ, _PP]),
    "lumen_llama_kv_update": (_I, [_P, _P, _P, _SZ]),
    "lumen_llama_kv_get_view": (_I, [_P, _SZ, _PP, _PP]),
    "lumen_llama_kv_free": (_I, [_P]),
    "lumen_self_attention_new": (_I, [_P, _SZ, _SZ, _SZ, _SZ, _F, _I, _PP]),
    "lumen_self_attention_set_weight": (_I, [_P, _I, _P]),
    "lumen_self_attention_forward": (_I, [_P, _P, _P, _PP, _PP]),
    "lumen_self_attention_free": (_I, [_P]),
    "lumen_attention_decode": (_I, [_P, _FP, _FP, _FP, _SZ, _P, _P, _I, _FP]),
    "lumen_llama_new": (_I, [_P, C.POINTER(LlamaConfigC), _PP]),
    "lumen_tp_param_slice": (_I, [C.POINTER(LlamaConfigC), _I, _I, C.c_char_p, _SZP]),
    "lumen_llama_set_param": (_I, [_P, C.c_char_p, _P, _SZP, _I, _I]),
    "lumen_llama_init_kv_caches": (_I, [_P, _SZ, _PP]),
    "lumen_llama_reset_kv_caches": (_I, [_P, _PP, _SZ]),
    "lumen_llama_forward": (_I, [_P, _FP, _SZ, _SZ, _PP, _SZ, _SZ, _FP]),
    "lumen_llama_forward_last": (_I, [_P, _FP, _SZ, _SZ, _PP, _SZ, _SZ, _FP]),
    "lumen_llama_forward_device": (_I, [_P, _FP, _SZ, _SZ, _PP, _SZ, _FP]),
    "lumen_sample_top_p": (_I, [_P, _FP, _SZ, C.POINTER(SampleParamsC), C.POINTER(C.c_int32)]),
    "lumen_llama_forward_sample": (_I, [_P, _FP, _SZ, _PP, _SZ, C.POINTER(SampleParamsC), C.POINTER(C.c_int32)]),
    "lumen_llama_free": (_I, [_P]),
    "lumen_llama_weight_bytes": (_SZ, [_P]),
    "lumen_llama_decode_trace": (_I, [_P, C.POINTER(C.c_uint64), _SZ, _SZP]),
}

_lib = None


def load() -> C.CDLL:
    """Load the shared library (built by `lumen_b200.build.build()`); raise if it is absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python lumen_b200/build.py` (needs nvcc). "
            "lumen_b200 has no CPU or PyTorch fallback.")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError here means the library does not export a declared symbol
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


class LumenError(RuntimeError):
    """A non-zero status from the C ABI.  `.code` is the LUMEN_ERR_* value."""

    def __init__(self, code: int, message: str):
        super().__init__(f"[lumen status {code}] {message}")
        self.code = code


def check(status: int, ctx_handle=None) -> None:
    """Turn a non-zero status into an exception, mirroring the reference's `panic!`s."""
    if status == OK:
        return
    lib = load()
    msg = lib.lumen_status_string(status).decode()
    if ctx_handle:
        detail = lib.lumen_last_error(ctx_handle).decode()
        if detail:
            msg = f"{msg}: {detail}"
    raise LumenError(status, msg)
