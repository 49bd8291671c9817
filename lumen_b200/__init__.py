"""lumen_b200 — B200 (sm_100a) implementation of the Llama inference hot path of chen-197/Lumen.

The package is a thin host-side mirror of the reference's Tensor / Module / LlamaModel / KV-cache
interface over a C-ABI CUDA library (include/lumen_b200.h).  Importing it loads that library and
fails if it has not been built: there is no CPU or PyTorch fallback.
"""
from . import _lib

_lib.load()

from ._lib import BF16, F32, LumenError  # noqa: E402
from .layers import (Embedding, KVCache, KVCacheInner, Linear, LlamaKVCache, Module, RMSNorm,  # noqa: E402
                     RotaryEmbedding, SelfAttention, SiLU, attention_decode, attention_decode_repeat, fused_softmax, gemv, gemv_kn_static,
                     gemv_repeat, matmul, reshape, sample_top_p)
from .llama import LlamaConfig, LlamaModel  # noqa: E402
from .loader import load_llama_weights  # noqa: E402
from .tokenizer import LlamaTokenizer  # noqa: E402
from .tensor import (Context, Tensor, default_context, is_inference_mode, is_no_grad, no_grad,  # noqa: E402
                     set_inference_mode)

__all__ = [
    "BF16", "F32", "LumenError", "Context", "Tensor", "default_context", "is_inference_mode", "is_no_grad",
    "no_grad", "set_inference_mode", "Module", "Linear", "Embedding", "RMSNorm", "SiLU", "RotaryEmbedding",
    "SelfAttention", "KVCache", "KVCacheInner", "LlamaKVCache", "LlamaConfig", "LlamaModel", "LlamaTokenizer", "load_llama_weights", "matmul", "reshape",
    "fused_softmax", "gemv", "gemv_kn_static", "gemv_repeat", "attention_decode", "attention_decode_repeat", "sample_top_p",
]
