"""LlamaConfig / LlamaModel — host-side mirror of src/models/llama.rs (inference methods)."""
from __future__ import annotations

import ctypes as C
import weakref
from dataclasses import dataclass

import numpy as np

from . import _lib
from ._lib import BF16, F32, LlamaConfigC
from .layers import KVCacheInner
from .tensor import Context, default_context, f32_to_bf16_bits, require_no_grad


@dataclass
class LlamaConfig:
    """src/models/llama.rs:11-37 (TinyLlama defaults) plus what the reference lacks: `head_dim`
    (0 = hidden/heads), `qk_norm` (Qwen3 per-head q/k RMSNorm) and `weight_dtype` ("f32"/"bf16")."""

    vocab_size: int = 32000
    hidden_size: int = 2048
    intermediate_size: int = 5632
    num_hidden_layers: int = 22
    num_attention_heads: int = 32
    num_key_value_heads: int = 4
    rms_norm_eps: float = 1e-5
    max_seq_len: int = 2048
    rope_theta: float = 10000.0
    head_dim: int = 0
    qk_norm: bool = False
    weight_dtype: str = "f32"

    def to_c(self) -> LlamaConfigC:
        return LlamaConfigC(self.vocab_size, self.hidden_size, self.intermediate_size, self.num_hidden_layers,
                            self.num_attention_heads, self.num_key_value_heads, self.rms_norm_eps, self.max_seq_len,
                            self.rope_theta, self.head_dim, int(self.qk_norm), BF16 if self.weight_dtype == "bf16" else F32)

    @property
    def resolved_head_dim(self) -> int:
        return self.head_dim or self.hidden_size // self.num_attention_heads

    def param_shapes(self) -> dict:
        """Names and full shapes of `LlamaModel::named_parameters` (llama.rs:218-279)."""
        from .synth import param_shapes
        return param_shapes(self)


def tp_param_slice(config: "LlamaConfig", tp_rank: int, tp_size: int, name: str) -> dict:
    """The part of parameter `name` that rank `tp_rank` of `tp_size` keeps (`lumen_tp_param_slice`; host
    arithmetic, needs no GPU).  Returns full shape and the kept row / column ranges."""
    from ._lib import check, load
    out = (C.c_size_t * 6)()
    cfg_c = config.to_c()
    check(load().lumen_tp_param_slice(C.byref(cfg_c), tp_rank, tp_size, name.encode(), out))
    rows, cols, r0, nr, c0, nc = (int(v) for v in out)
    return {"shape": (rows,) if cols == 0 else (rows, cols), "rows": (r0, r0 + nr), "cols": (c0, c0 + nc)}


class _ParamRef:
    """What `named_parameters()` hands to a loader: `set_raw_data` uploads into the model's slab."""

    def __init__(self, model: "LlamaModel", name: str, shape: tuple):
        self.model, self.name, self.shape = model, name, shape

    def set_raw_data(self, shape, raw_data) -> None:
        self.model.set_param(self.name, np.asarray(raw_data, dtype=np.float32).reshape(shape))


class LlamaModel:
    """src/models/llama.rs:129-216.  Parameters start unset; fill them with `set_param` /
    `load_state` (the reference's random Kaiming init is not reproduced)."""

    def __init__(self, config: LlamaConfig, ctx: Context | None = None):
        self.ctx = ctx or default_context()
        self.config = config
        self.h = C.c_void_p()
        cfg_c = config.to_c()
        self.ctx.check(self.ctx._lib.lumen_llama_new(self.ctx.h, C.byref(cfg_c), C.byref(self.h)))
        self._finalizer = weakref.finalize(self, self.ctx._lib.lumen_llama_free, C.c_void_p(self.h.value))
        self._shapes = config.param_shapes()

    # ---- parameters ---------------------------------------------------------------------------------
    def named_parameters(self) -> dict:
        return {n: _ParamRef(self, n, s) for n, s in self._shapes.items()}

    def set_param(self, name: str, value: np.ndarray, as_bf16_bits: bool = False) -> None:
        """Upload one full (unsharded) tensor by its Hugging Face name.  `value` is f32, or uint16
        bf16 bit patterns when `as_bf16_bits`."""
        if as_bf16_bits:
            a = np.ascontiguousarray(value, dtype=np.uint16)
            dt = BF16
        else:
            a = np.ascontiguousarray(value, dtype=np.float32)
            dt = F32
        shape = (C.c_size_t * a.ndim)(*a.shape)
        self.ctx.check(self.ctx._lib.lumen_llama_set_param(self.h, name.encode(), a.ctypes.data, shape, a.ndim, dt))

    def load_state(self, params: dict) -> None:
        for name, value in params.items():
            self.set_param(name, value)

    def decode_trace(self) -> np.ndarray:
        """Device trace of the last persistent decode step (needs LUMEN_DECODE_TRACE=1 when the model is
        created).  With nph = 5 * layers + 1 phases (qkv, attention, o, gate/up, down per layer, then lm_head):
        `stamps` [nph, 3] ns at phase start / after its prologue / after its last tile, `end` ns,
        `producer` [nph] ns of the phase's first copy, `input_ready` [nph] ns, `wait_cycles` and
        `busy_cycles` [nph] of consumer warp 0 on weight tiles, `tile_issue` and `tile_release` [512] ns;
        `cta_input` and `cta_done` [nph, 160] ns per CTA (0 where a CTA has no part in the phase)."""
        nph = 5 * self.config.num_hidden_layers + 1
        base = 7 * nph + 1 + 1024
        n = base + 2 * nph * 160
        buf = (C.c_uint64 * n)()
        got = C.c_size_t()
        self.ctx.check(self.ctx._lib.lumen_llama_decode_trace(self.h, buf, n, C.byref(got)))
        a = np.frombuffer(buf, dtype=np.uint64, count=got.value).astype(np.int64)
        return {"stamps": a[:3 * nph].reshape(nph, 3), "end": int(a[3 * nph]),
                "producer": a[3 * nph + 1:4 * nph + 1], "input_ready": a[4 * nph + 1:5 * nph + 1],
                "wait_cycles": a[5 * nph + 1:6 * nph + 1], "busy_cycles": a[6 * nph + 1:7 * nph + 1],
                "tile_issue": a[7 * nph + 1:7 * nph + 513], "tile_release": a[7 * nph + 513:base],
                "cta_input": a[base:base + nph * 160].reshape(nph, 160),
                "cta_done": a[base + nph * 160:base + 2 * nph * 160].reshape(nph, 160)}

    @property
    def weight_bytes_per_step(self) -> int:
        return int(self.ctx._lib.lumen_llama_weight_bytes(self.h))

    # ---- caches (llama.rs:161-176) ----------------------------------------------------------------------
    def init_kv_caches(self, batch_size: int) -> list:
        n = self.config.num_hidden_layers
        arr = (C.c_void_p * max(n, 1))()
        self.ctx.check(self.ctx._lib.lumen_llama_init_kv_caches(self.h, batch_size, arr))
        tp = self.ctx.tp_size
        hkv = self.config.num_key_value_heads
        hkv_l = hkv // tp if hkv % tp == 0 else 1
        return [KVCacheInner(batch_size, hkv_l, self.config.max_seq_len, self.config.resolved_head_dim, self.ctx,
                             _handle=C.c_void_p(arr[i])) for i in range(n)]

    def reset_kv_caches(self, caches: list) -> None:
        for c in caches:
            c.reset()

    def _cache_array(self, caches):
        return (C.c_void_p * max(len(caches), 1))(*[c.h for c in caches])

    # ---- forward (llama.rs:181-206) -----------------------------------------------------------------------
    def forward(self, input_ids, caches: list, _pos: int = 0, last_only: bool = False) -> np.ndarray:
        """input_ids[B,S] (token ids, passed as f32 like the reference) -> logits [B,S,V] on the host.
        `last_only` returns [B,V] for the final position only."""
        require_no_grad("LlamaModel::forward")
        ids = np.ascontiguousarray(input_ids, dtype=np.float32)
        if ids.ndim != 2:
            raise _lib.LumenError(_lib.ERR_SHAPE, "input_ids must be [B,S]")
        b, s = ids.shape
        v = self.config.vocab_size
        logits = np.empty((b, v) if last_only else (b, s, v), dtype=np.float32)
        fn = self.ctx._lib.lumen_llama_forward_last if last_only else self.ctx._lib.lumen_llama_forward
        self.ctx.check(fn(self.h, ids.ctypes.data, b, s, self._cache_array(caches), len(caches), _pos, logits.ctypes.data))
        return logits

    def forward_sample(self, input_ids, caches: list, temperature: float, top_p: float, repetition_penalty: float,
                       recent_tokens, uniform: float) -> int:
        """`forward` on ids [1,S] followed by `sample_top_p` (src/main.rs:74-137) on the device; returns the
        sampled token id.  `uniform` is the draw in [0,1) the reference takes from its RNG."""
        require_no_grad("LlamaModel::forward")
        from ._lib import SampleParamsC
        ids = np.ascontiguousarray(input_ids, dtype=np.float32).reshape(-1)
        rec = np.ascontiguousarray(recent_tokens, dtype=np.int32)
        sp = SampleParamsC(temperature, top_p, repetition_penalty, rec.ctypes.data_as(C.POINTER(C.c_int32)), rec.size, uniform)
        tok = C.c_int32()
        self.ctx.check(self.ctx._lib.lumen_llama_forward_sample(self.h, ids.ctypes.data, ids.size, self._cache_array(caches),
                                                                len(caches), C.byref(sp), C.byref(tok)))
        return int(tok.value)

    def forward_device(self, ids_ptr: int, b: int, s: int, caches: list, logits_ptr: int) -> None:
        """Same step with device-resident ids and logits, asynchronous on the context's stream."""
        require_no_grad("LlamaModel::forward")
        self.ctx.check(self.ctx._lib.lumen_llama_forward_device(self.h, ids_ptr, b, s, self._cache_array(caches),
                                                                len(caches), logits_ptr))
