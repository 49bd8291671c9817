"""Ops, Module and the layers on the Llama path — host-side mirror of the reference's
src/ops/{matmul,fused,shape}.rs, src/module.rs and src/layers/{basic,norm,attention,activation}.

Every function launches CUDA kernels through the C ABI; nothing here computes on the host.
"""
from __future__ import annotations

import ctypes as C
import weakref

import numpy as np

from . import _lib
from .tensor import Context, Tensor, default_context, require_no_grad, set_inference_mode


# ---- ops ---------------------------------------------------------------------------------------------
def _unary_out(ctx: Context, fn, *args) -> Tensor:
    h = C.c_void_p()
    ctx.check(fn(ctx.h, *args, C.byref(h)))
    return Tensor(h, ctx)


def matmul(a: Tensor, b: Tensor) -> Tensor:
    """ops::matmul::matmul (src/ops/matmul.rs:10): a[...,K] @ b[N,K]^T -> [...,N]."""
    return _unary_out(a.ctx, a.ctx._lib.lumen_matmul, a.h, b.h)


def reshape(t: Tensor, shape) -> Tensor:
    """ops::shape::reshape (src/ops/shape.rs:9)."""
    return t.reshape(shape)


def fused_softmax(x: Tensor, scale: float, is_causal: bool) -> Tensor:
    """ops::fused::fused_softmax forward (src/ops/fused.rs:17)."""
    return _unary_out(x.ctx, x.ctx._lib.lumen_fused_softmax, x.h, C.c_float(scale), int(is_causal))


def gemv_repeat(ctx, x_ptr: int, w_ptrs, w_dtype: int, layout_kn: bool, k: int, n: int, y_ptr: int, iters: int) -> float:
    """`lumen_gemv_repeat`: microseconds per call of `iters` back-to-back products rotating over the matrices `w_ptrs`."""
    arr = (C.c_void_p * len(w_ptrs))(*w_ptrs)
    us = C.c_float()
    ctx.check(ctx._lib.lumen_gemv_repeat(ctx.h, x_ptr, arr, len(w_ptrs), w_dtype, int(layout_kn), k, n, y_ptr, iters, C.byref(us)))
    return float(us.value)


def attention_decode_repeat(ctx, q_ptr: int, k_ptr: int, v_ptr: int, n_head: int, caches, rope, out_ptr: int, iters: int) -> float:
    """`lumen_attention_decode_repeat`: microseconds per call of `iters` back-to-back decode-attention steps rotating over
    `caches` (each call appends one row to the cache it uses)."""
    arr = (C.c_void_p * len(caches))(*[c.h for c in caches])
    us = C.c_float()
    ctx.check(ctx._lib.lumen_attention_decode_repeat(ctx.h, q_ptr, k_ptr, v_ptr, n_head, arr, len(caches), rope.h if rope else None,
                                                     out_ptr, iters, C.byref(us)))
    return float(us.value)


def gemv(ctx: Context, x_ptr: int, w_ptr: int, w_dtype: int, layout_kn: bool, k: int, n: int, y_ptr: int) -> None:
    """Vector-matrix product on raw device pointers (`lumen_gemv`)."""
    ctx.check(ctx._lib.lumen_gemv(ctx.h, x_ptr, w_ptr, w_dtype, int(layout_kn), k, n, y_ptr))


def gemv_kn_static(ctx: Context, x_ptr: int, w_ptr: int, w_dtype: int, k: int, n: int, y_ptr: int) -> None:
    """[K,N]-layout vector-matrix product that allocates nothing (`lumen_gemv_kn_static`)."""
    ctx.check(ctx._lib.lumen_gemv_kn_static(ctx.h, x_ptr, w_ptr, w_dtype, k, n, y_ptr))


# ---- Module (src/module.rs:12-24) ------------------------------------------------------------------------
class Module:
    def forward(self, input: Tensor) -> Tensor:  # noqa: A002 - the reference's argument name
        raise NotImplementedError

    def parameters(self) -> list:
        return []

    def train_mode(self) -> None:
        set_inference_mode(False)

    def eval_mode(self) -> None:
        set_inference_mode(True)

    def __call__(self, *a, **k):
        return self.forward(*a, **k)


# ---- layers ------------------------------------------------------------------------------------------------
class Linear(Module):
    """src/layers/basic/linear.rs:7-50.  weight is [out_features, in_features]; bias optional."""

    def __init__(self, weight: Tensor, bias: Tensor | None = None):
        self.weight, self.bias = weight, bias

    @classmethod
    def new_no_bias(cls, in_features: int, out_features: int, ctx: Context | None = None) -> "Linear":
        return cls(Tensor.from_array_no_grad(np.zeros((out_features, in_features), np.float32), ctx))

    def forward(self, input: Tensor) -> Tensor:  # noqa: A002
        ctx = input.ctx
        return _unary_out(ctx, ctx._lib.lumen_linear_forward, input.h, self.weight.h, self.bias.h if self.bias else None)

    def parameters(self):
        return [self.weight] + ([self.bias] if self.bias else [])


class Embedding(Module):
    """src/layers/basic/embedding.rs:9-57.  Token ids arrive as f32."""

    def __init__(self, weight: Tensor):
        self.weight = weight
        self.vocab_size, self.embed_dim = weight.shape

    def forward(self, indices: Tensor) -> Tensor:
        ctx = indices.ctx
        return _unary_out(ctx, ctx._lib.lumen_embedding, indices.h, self.weight.h)

    def parameters(self):
        return [self.weight]


class RMSNorm(Module):
    """src/layers/norm/rms_norm.rs:8-62."""

    def __init__(self, dim: int, eps: float, ctx: Context | None = None, weight: Tensor | None = None):
        self.weight = weight if weight is not None else Tensor.from_array_no_grad(np.ones(dim, np.float32), ctx)
        self.eps = eps

    def forward(self, input: Tensor) -> Tensor:  # noqa: A002
        ctx = input.ctx
        return _unary_out(ctx, ctx._lib.lumen_rmsnorm, input.h, self.weight.h, C.c_float(self.eps))

    def parameters(self):
        return [self.weight]


class SiLU(Module):
    """src/layers/activation.rs:131-147."""

    def forward(self, input: Tensor) -> Tensor:  # noqa: A002
        return _unary_out(input.ctx, input.ctx._lib.lumen_silu, input.h)


class RotaryEmbedding:
    """src/layers/attention/encoding.rs:6-123."""

    def __init__(self, dim: int, max_seq_len: int, theta: float, ctx: Context | None = None):
        self.ctx = ctx or default_context()
        self.dim, self.max_seq_len, self.theta = dim, max_seq_len, theta
        self.h = C.c_void_p()
        self.ctx.check(self.ctx._lib.lumen_rope_new(self.ctx.h, dim, max_seq_len, C.c_float(theta), C.byref(self.h)))
        self._finalizer = weakref.finalize(self, self.ctx._lib.lumen_rope_free, C.c_void_p(self.h.value))

    def forward(self, x: Tensor, offset: int) -> Tensor:
        h = C.c_void_p()
        self.ctx.check(self.ctx._lib.lumen_rope_forward(self.h, x.h, offset, C.byref(h)))
        return Tensor(h, self.ctx)


class KVCacheInner:
    """src/layers/attention/self_attention.rs:24-44: k,v [B,Hkv,max_seq,D] zero-initialised, `len`."""

    def __init__(self, b: int, h_kv: int, max_seq: int, d: int, ctx: Context | None = None, _handle=None):
        self.ctx = ctx or default_context()
        self.shape = (b, h_kv, max_seq, d)
        if _handle is None:
            _handle = C.c_void_p()
            self.ctx.check(self.ctx._lib.lumen_kv_new(self.ctx.h, b, h_kv, max_seq, d, C.byref(_handle)))
        self.h = _handle
        self._finalizer = weakref.finalize(self, self.ctx._lib.lumen_kv_free, C.c_void_p(self.h.value))

    def reset(self) -> None:
        self.ctx.check(self.ctx._lib.lumen_kv_reset(self.h))

    @property
    def len(self) -> int:
        return int(self.ctx._lib.lumen_kv_len(self.h))

    def read(self):
        """Host copies of the `k` and `v` slabs."""
        k = np.empty(self.shape, np.float32)
        v = np.empty(self.shape, np.float32)
        self.ctx.check(self.ctx._lib.lumen_kv_read(self.h, k.ctypes.data, v.ctypes.data))
        return k, v

    def write(self, k: np.ndarray, v: np.ndarray, length: int) -> None:
        """Overwrite the slabs and `len` from the host (the reference's fields are public)."""
        k = np.ascontiguousarray(k, np.float32)
        v = np.ascontiguousarray(v, np.float32)
        if k.shape != self.shape or v.shape != self.shape:
            raise _lib.LumenError(_lib.ERR_SHAPE, f"expected slabs of shape {self.shape}")
        self.ctx.check(self.ctx._lib.lumen_kv_write(self.h, k.ctypes.data, v.ctypes.data, length))


KVCache = KVCacheInner  # `pub type KVCache = Rc<RefCell<KVCacheInner>>` (self_attention.rs:30)


class SelfAttention:
    """src/layers/attention/self_attention.rs:46-127, :299-306 (no-grad paths)."""

    def __init__(self, embed_dim: int, n_head: int, n_kv_head: int, max_seq_len: int, rope_theta: float,
                 causal: bool, ctx: Context | None = None):
        self.ctx = ctx or default_context()
        self.n_head, self.n_kv_head, self.head_dim = n_head, n_kv_head, embed_dim // max(n_head, 1)
        self.max_seq, self.causal = max_seq_len, causal
        self.h = C.c_void_p()
        self.ctx.check(self.ctx._lib.lumen_self_attention_new(self.ctx.h, embed_dim, n_head, n_kv_head, max_seq_len,
                                                              C.c_float(rope_theta), int(causal), C.byref(self.h)))
        self._finalizer = weakref.finalize(self, self.ctx._lib.lumen_self_attention_free, C.c_void_p(self.h.value))
        self.w_q = self.w_k = self.w_v = self.w_o = None

    def set_weights(self, w_q: Tensor, w_k: Tensor, w_v: Tensor, w_o: Tensor) -> None:
        for which, w in enumerate((w_q, w_k, w_v, w_o)):
            self.ctx.check(self.ctx._lib.lumen_self_attention_set_weight(self.h, which, w.h))
        self.w_q, self.w_k, self.w_v, self.w_o = (Linear(w) for w in (w_q, w_k, w_v, w_o))

    def forward(self, x: Tensor, cache: KVCacheInner | None = None):
        """Returns (output, cache) like the reference's `(Tensor, Option<KVCache>)`."""
        require_no_grad("SelfAttention::forward")
        out, cache_out = C.c_void_p(), C.c_void_p()
        self.ctx.check(self.ctx._lib.lumen_self_attention_forward(self.h, x.h, cache.h if cache else None,
                                                                  C.byref(out), C.byref(cache_out)))
        if cache is None:
            b = x.shape[0]
            cache = KVCacheInner(b, self.n_kv_head, self.max_seq, self.head_dim, self.ctx, _handle=cache_out)
        return Tensor(out, self.ctx), cache


def sample_top_p(ctx: Context, logits_ptr: int, vocab: int, temperature: float, top_p: float, repetition_penalty: float,
                 recent_tokens, uniform: float) -> int:
    """`sample_top_p` (src/main.rs:74-137) on a device logits vector (`lumen_sample_top_p`)."""
    rec = np.ascontiguousarray(recent_tokens, dtype=np.int32)
    sp = _lib.SampleParamsC(temperature, top_p, repetition_penalty, rec.ctypes.data_as(C.POINTER(C.c_int32)), rec.size, uniform)
    tok = C.c_int32()
    ctx.check(ctx._lib.lumen_sample_top_p(ctx.h, logits_ptr, vocab, C.byref(sp), C.byref(tok)))
    return int(tok.value)


def attention_decode(ctx: Context, q_ptr: int, k_new_ptr: int, v_new_ptr: int, n_head: int, cache: KVCacheInner,
                     rope: RotaryEmbedding | None, out_ptr: int, causal: bool = True) -> None:
    """`lumen_attention_decode` on raw device pointers."""
    ctx.check(ctx._lib.lumen_attention_decode(ctx.h, q_ptr, k_new_ptr, v_new_ptr, n_head, cache.h,
                                              rope.h if rope else None, int(causal), out_ptr))


class LlamaKVCache:
    """src/kv_cache.rs:5-59."""

    def __init__(self, config, ctx: Context | None = None):
        self.ctx = ctx or default_context()
        self.max_seq_len = config.max_seq_len
        self.head_num = config.num_key_value_heads
        self.dim = config.hidden_size // config.num_attention_heads
        self.h = C.c_void_p()
        self.ctx.check(self.ctx._lib.lumen_llama_kv_new(self.ctx.h, self.head_num, self.max_seq_len, self.dim, C.byref(self.h)))
        self._finalizer = weakref.finalize(self, self.ctx._lib.lumen_llama_kv_free, C.c_void_p(self.h.value))

    def update(self, k: Tensor, v: Tensor, start_pos: int) -> None:
        self.ctx.check(self.ctx._lib.lumen_llama_kv_update(self.h, k.h, v.h, start_pos))

    def get_view(self, current_len: int):
        k, v = C.c_void_p(), C.c_void_p()
        self.ctx.check(self.ctx._lib.lumen_llama_kv_get_view(self.h, current_len, C.byref(k), C.byref(v)))
        return Tensor(k, self.ctx), Tensor(v, self.ctx)
