"""ctypes binding of the C oracle (oracle/lumen_oracle.c) — TEST INFRASTRUCTURE.

PARITY UNPINNED: the reference (chen-197/Lumen, Rust) has no golden vectors and cannot be
built in this environment; the C code restates its source (citations in lumen_oracle_impl.h).

Every function takes and returns numpy arrays.  `prec` selects the f32 restatement ("f32",
reference arithmetic) or the f64 shadow ("f64").
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

_DIR = Path(__file__).resolve().parent
_SO = _DIR / "_build" / "liblumen_oracle.so"


def build(force: bool = False) -> Path:
    """Compile the oracle with the Makefile beside it (gcc + OpenMP)."""
    src_m = max((_DIR / n).stat().st_mtime for n in ("lumen_oracle.c", "lumen_oracle_impl.h", "Makefile"))
    if force or not _SO.exists() or _SO.stat().st_mtime < src_m:
        subprocess.run(["make", "-C", str(_DIR)], check=True, capture_output=True)
    return _SO


class Config(C.Structure):
    """Mirror of `lo_config`: LlamaConfig (src/models/llama.rs:11-21) + head_dim + qk_norm."""

    _fields_ = [
        ("vocab", C.c_long), ("hidden", C.c_long), ("inter", C.c_long), ("layers", C.c_long),
        ("heads", C.c_long), ("kv_heads", C.c_long), ("eps", C.c_float), ("max_seq", C.c_long),
        ("theta", C.c_float), ("head_dim", C.c_long), ("qk_norm", C.c_int),
    ]


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not _SO.exists():
            build()
        _lib = C.CDLL(str(_SO))
        for name in ("lo_kv_new_f32", "lo_kv_new_f64", "lo_llama_new_f32", "lo_llama_new_f64",
                     "lo_llama_kv_new", "lo_kv_k_f32", "lo_kv_v_f32", "lo_kv_k_f64", "lo_kv_v_f64"):
            getattr(_lib, name).restype = C.c_void_p
        for name in ("lo_kv_len_f32", "lo_kv_len_f64"):
            getattr(_lib, name).restype = C.c_long
    return _lib


def _dt(prec):
    return np.float32 if prec == "f32" else np.float64


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _fn(name, prec):
    return getattr(lib(), f"{name}_{prec}")


def num_threads() -> int:
    return int(lib().lo_num_threads())


def host_cores() -> int:
    """Cores this process may run on (its affinity mask; the machine's count where that is unknown)."""
    try:
        return len(os.sched_getaffinity(0))
    except (AttributeError, OSError):
        return os.cpu_count() or 1


def set_num_threads(n: int | None = None) -> int:
    """Use `n` threads (default: every core of this process) whatever OMP_NUM_THREADS says; returns the count in use."""
    lib().lo_set_num_threads(C.c_int(int(n) if n else host_cores()))
    return num_threads()


def matmul(a, w, prec="f32"):
    """a[..., K] @ w[N, K]^T (src/ops/matmul.rs:10-103)."""
    a, w = _f32(a), _f32(w)
    k = a.shape[-1]
    n, k2 = w.shape
    if k != k2:
        raise ValueError(f"MatMul shape mismatch: K={k} vs K={k2}")
    m = a.size // k
    out = np.empty(a.shape[:-1] + (n,), dtype=_dt(prec))
    _fn("lo_matmul", prec)(_p(a), C.c_long(m), C.c_long(k), _p(w), C.c_long(n), _p(out))
    return out


def rmsnorm(x, w, eps, prec="f32"):
    x, w = _f32(x), _f32(w)
    dim = x.shape[-1]
    out = np.empty(x.shape, dtype=_dt(prec))
    _fn("lo_rmsnorm", prec)(_p(x), C.c_long(x.size // dim), C.c_long(dim), _p(w), C.c_float(eps), _p(out))
    return out


def rope_table(dim, max_seq, theta, prec="f32"):
    cos = np.empty((max_seq, dim), dtype=_dt(prec))
    sin = np.empty((max_seq, dim), dtype=_dt(prec))
    _fn("lo_rope_table", prec)(C.c_long(dim), C.c_long(max_seq), C.c_float(theta), _p(cos), _p(sin))
    return cos, sin


def rope_forward(x, offset, max_seq, theta, prec="f32"):
    """x[B,H,S,D] rotated at positions offset..offset+S (encoding.rs:56-123)."""
    x = _f32(x)
    b, h, s, d = x.shape
    out = np.empty(x.shape, dtype=_dt(prec))
    rc = _fn("lo_rope_forward", prec)(_p(x), C.c_long(b), C.c_long(h), C.c_long(s), C.c_long(d),
                                      C.c_long(offset), C.c_long(max_seq), C.c_float(theta), _p(out))
    if rc:
        raise IndexError("RoPE index out of range")
    return out


def silu(x, prec="f32"):
    x = _f32(x)
    out = np.empty(x.shape, dtype=_dt(prec))
    _fn("lo_silu", prec)(_p(x), C.c_long(x.size), _p(out))
    return out


def mul(a, b, prec="f32"):
    a, b = _f32(a), _f32(b)
    out = np.empty(a.shape, dtype=_dt(prec))
    _fn("lo_mul", prec)(_p(a), _p(b), C.c_long(a.size), _p(out))
    return out


def add(a, b, prec="f32"):
    a, b = _f32(a), _f32(b)
    out = np.empty(a.shape, dtype=_dt(prec))
    _fn("lo_add", prec)(_p(a), _p(b), C.c_long(a.size), _p(out))
    return out


def embedding(ids, table, prec="f32"):
    ids, table = _f32(ids), _f32(table)
    vocab, dim = table.shape
    out = np.empty(ids.shape + (dim,), dtype=_dt(prec))
    rc = _fn("lo_embedding", prec)(_p(ids), C.c_long(ids.size), _p(table), C.c_long(vocab), C.c_long(dim), _p(out))
    if rc:
        raise IndexError("Embedding index out of bounds")
    return out


def fused_softmax(x, scale, causal, prec="f32"):
    x = _f32(x)
    b, h, q, k = x.shape
    out = np.empty(x.shape, dtype=_dt(prec))
    _fn("lo_fused_softmax", prec)(_p(x), C.c_long(b), C.c_long(h), C.c_long(q), C.c_long(k),
                                  C.c_float(scale), C.c_int(int(causal)), _p(out))
    return out


def sample_top_p(logits, temperature, top_p, repetition_penalty, recent_tokens, r) -> int:
    """`sample_top_p` of src/main.rs:74-137 with the uniform draw `r` given."""
    x = _f32(logits).ravel()
    rec = np.ascontiguousarray(recent_tokens, dtype=np.int64)
    f = lib().lo_sample_top_p
    f.restype = C.c_long
    return int(f(_p(x), C.c_long(x.size), C.c_float(temperature), C.c_float(top_p), C.c_float(repetition_penalty),
                 rec.ctypes.data_as(C.c_void_p), C.c_long(rec.size), C.c_float(r)))


def round_bf16(x):
    x = _f32(x)
    out = np.empty_like(x)
    lib().lo_round_bf16(_p(x), C.c_long(x.size), _p(out))
    return out


class KVCache:
    """KVCacheInner (self_attention.rs:24-44): k,v [B,Hkv,max_seq,D], len."""

    def __init__(self, b, h_kv, max_seq, d, prec="f32"):
        self.prec, self.shape = prec, (b, h_kv, max_seq, d)
        self.h = C.c_void_p(_fn("lo_kv_new", prec)(C.c_long(b), C.c_long(h_kv), C.c_long(max_seq), C.c_long(d)))

    def __del__(self):
        if getattr(self, "h", None):
            _fn("lo_kv_free", self.prec)(self.h)
            self.h = None

    def reset(self):
        _fn("lo_kv_reset", self.prec)(self.h)

    @property
    def len(self):
        return int(_fn("lo_kv_len", self.prec)(self.h))

    @len.setter
    def len(self, n):
        _fn("lo_kv_set_len", self.prec)(self.h, C.c_long(int(n)))

    def _view(self, which):
        ptr = _fn(f"lo_kv_{which}", self.prec)(self.h)
        n = int(np.prod(self.shape))
        ct = C.c_float if self.prec == "f32" else C.c_double
        return np.ctypeslib.as_array(C.cast(ptr, C.POINTER(ct)), shape=(n,)).reshape(self.shape)

    @property
    def k(self):
        return self._view("k")

    @property
    def v(self):
        return self._view("v")


def attention(q, k, v, cache: KVCache, n_head, theta, rope_max, causal=True, q_norm=None, k_norm=None,
              norm_eps=1e-6):
    """Attention core of SelfAttention::forward after the q/k/v projections.

    q[B,S,Hq*D], k/v[B,S,Hkv*D]; S==1 takes the decode path (self_attention.rs:125-297), else
    the prefill path (:308-426).  Returns [B,S,Hq,D] and advances the cache.
    """
    q, k, v = _f32(q), _f32(k), _f32(v)
    b, s = q.shape[0], q.shape[1]
    d = cache.shape[3]
    out = np.empty((b, s, n_head, d), dtype=_dt(cache.prec))
    qn = _p(_f32(q_norm)) if q_norm is not None else None
    kn = _p(_f32(k_norm)) if k_norm is not None else None
    rc = _fn("lo_attention", cache.prec)(_p(q), _p(k), _p(v), C.c_long(s), cache.h, C.c_long(n_head),
                                         C.c_float(theta), C.c_long(rope_max), C.c_int(int(causal)), qn, kn,
                                         C.c_float(norm_eps), _p(out))
    if rc == -2:
        raise OverflowError("KV cache overflow")
    if rc:
        raise IndexError("RoPE index out of range")
    return out


class LlamaKVCache:
    """LlamaKVCache (src/kv_cache.rs:5-59)."""

    def __init__(self, kv_heads, max_seq, head_dim):
        self.head_num, self.max_seq_len, self.dim = kv_heads, max_seq, head_dim
        self.h = C.c_void_p(lib().lo_llama_kv_new(C.c_long(kv_heads), C.c_long(max_seq), C.c_long(head_dim)))

    def __del__(self):
        if getattr(self, "h", None):
            lib().lo_llama_kv_free(self.h)
            self.h = None

    def update(self, k, v, start_pos):
        k, v = _f32(k), _f32(v)
        s = k.shape[2]
        if lib().lo_llama_kv_update(self.h, _p(k), _p(v), C.c_long(s), C.c_long(start_pos)):
            raise OverflowError("KV Cache overflow!")

    def get_view(self, n):
        k = np.empty((1, self.head_num, n, self.dim), np.float32)
        v = np.empty_like(k)
        lib().lo_llama_kv_get_view(self.h, C.c_long(n), _p(k), _p(v))
        return k, v


class Llama:
    """LlamaModel inference methods (src/models/llama.rs:138-206) over borrowed f32 weights."""

    def __init__(self, cfg: dict, params: dict, prec="f32"):
        self.prec = prec
        self.cfg = Config(vocab=cfg["vocab_size"], hidden=cfg["hidden_size"], inter=cfg["intermediate_size"],
                          layers=cfg["num_hidden_layers"], heads=cfg["num_attention_heads"],
                          kv_heads=cfg["num_key_value_heads"], eps=cfg["rms_norm_eps"], max_seq=cfg["max_seq_len"],
                          theta=cfg["rope_theta"], head_dim=cfg.get("head_dim", 0) or 0,
                          qk_norm=int(bool(cfg.get("qk_norm", False))))
        self.head_dim = self.cfg.head_dim or self.cfg.hidden // self.cfg.heads
        self.h = C.c_void_p(_fn("lo_llama_new", prec)(C.byref(self.cfg)))
        self._keep = {}
        for name, arr in params.items():
            arr = _f32(arr)
            self._keep[name] = arr
            if _fn("lo_llama_set_param", prec)(self.h, name.encode(), _p(arr)):
                raise KeyError(name)

    def __del__(self):
        if getattr(self, "h", None):
            _fn("lo_llama_free", self.prec)(self.h)
            self.h = None

    def init_kv_caches(self, batch):
        c = self.cfg
        return [KVCache(batch, c.kv_heads, c.max_seq, self.head_dim, self.prec) for _ in range(c.layers)]

    def forward(self, ids, caches):
        """ids[B,S] (any numeric dtype; passed as f32 like the reference) -> logits[B,S,V]."""
        ids = _f32(ids)
        b, s = ids.shape
        if len(caches) != self.cfg.layers:
            raise ValueError("KV cache count mismatch")
        logits = np.empty((b, s, self.cfg.vocab), dtype=_dt(self.prec))
        arr = (C.c_void_p * len(caches))(*[c.h for c in caches])
        rc = _fn("lo_llama_forward", self.prec)(self.h, _p(ids), C.c_long(b), C.c_long(s), arr, _p(logits))
        if rc == -3:
            raise IndexError("Embedding index out of bounds")
        if rc == -2:
            raise OverflowError("KV cache overflow")
        if rc:
            raise IndexError("RoPE index out of range")
        return logits
