"""Seeded synthetic weights and token ids with the shapes of the benchmark configurations.

The reference publishes no weights-free benchmark data; the configurations name architectures
only, so weights are N(0, 0.02) draws and prompts are uniform token ids.  One numpy PCG64 stream
per seed, parameters drawn in sorted-name order, RMSNorm gains fixed at 1.0 (not drawn).

This module imports nothing from the rest of the package (numpy only), so a program that must not
load the CUDA library - the CPU arm of the benchmark - can load this file on its own by path.
"""
from __future__ import annotations

import numpy as np


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 bit patterns (uint16)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    rounded = u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))
    return (rounded >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def _field(cfg, name, default=None):
    return cfg.get(name, default) if isinstance(cfg, dict) else getattr(cfg, name, default)


def param_shapes(cfg) -> dict:
    """Names and full shapes of `LlamaModel::named_parameters` (src/models/llama.rs:218-279) for a config given
    as a `LlamaConfig` or as a dict with its field names."""
    H, I, V = _field(cfg, "hidden_size"), _field(cfg, "intermediate_size"), _field(cfg, "vocab_size")
    heads, kv_heads = _field(cfg, "num_attention_heads"), _field(cfg, "num_key_value_heads")
    D = _field(cfg, "head_dim", 0) or H // heads
    qd, kvd = heads * D, kv_heads * D
    shapes = {"model.embed_tokens.weight": (V, H), "model.norm.weight": (H,), "lm_head.weight": (V, H)}
    for i in range(_field(cfg, "num_hidden_layers")):
        p = f"model.layers.{i}."
        shapes.update({
            p + "self_attn.q_proj.weight": (qd, H), p + "self_attn.k_proj.weight": (kvd, H),
            p + "self_attn.v_proj.weight": (kvd, H), p + "self_attn.o_proj.weight": (H, qd),
            p + "mlp.gate_proj.weight": (I, H), p + "mlp.up_proj.weight": (I, H),
            p + "mlp.down_proj.weight": (H, I), p + "input_layernorm.weight": (H,),
            p + "post_attention_layernorm.weight": (H,),
        })
        if _field(cfg, "qk_norm", False):
            shapes.update({p + "self_attn.q_norm.weight": (D,), p + "self_attn.k_norm.weight": (D,)})
    return shapes

TINYLLAMA = dict(vocab_size=32000, hidden_size=2048, intermediate_size=5632, num_hidden_layers=22,
                 num_attention_heads=32, num_key_value_heads=4, rms_norm_eps=1e-5, max_seq_len=2048,
                 rope_theta=10000.0)
LLAMA2_7B = dict(vocab_size=32000, hidden_size=4096, intermediate_size=11008, num_hidden_layers=32,
                 num_attention_heads=32, num_key_value_heads=32, rms_norm_eps=1e-5, max_seq_len=1024,
                 rope_theta=10000.0)
QWEN3_8B = dict(vocab_size=151936, hidden_size=4096, intermediate_size=12288, num_hidden_layers=36,
                num_attention_heads=32, num_key_value_heads=8, rms_norm_eps=1e-6, max_seq_len=4352,
                rope_theta=1e6, head_dim=128, qk_norm=True)


def iter_params(cfg, seed: int, std: float = 0.02, round_bf16: bool = False):
    """Yield (name, f32 array) for every parameter of `cfg`, deterministically from `seed`.

    With `round_bf16` the matrices are rounded to bf16 (nearest even) and widened back, i.e. the
    values a bf16 checkpoint holds after the reference loader's upcast (src/loader.rs:50-64).
    """
    rng = np.random.default_rng(seed)
    for name, shape in sorted(param_shapes(cfg).items()):
        if len(shape) == 1:
            yield name, np.ones(shape, np.float32)
            continue
        w = rng.standard_normal(shape, dtype=np.float32)
        w *= np.float32(std)
        if round_bf16:
            w = bf16_bits_to_f32(f32_to_bf16_bits(w)).reshape(shape)
        yield name, w


def iter_params_tiled(cfg, seed: int, std: float = 0.02, round_bf16: bool = False, block: int = 1 << 22):
    """Like `iter_params`, for the multi-billion-parameter shapes where drawing every value would take
    minutes per rank: each matrix repeats one seeded block of `block` N(0, std) draws (rolled by a
    per-tensor offset).  Same shapes, dtype and value distribution; only throughput runs use it."""
    rng = np.random.default_rng(seed)
    base = rng.standard_normal(block, dtype=np.float32) * np.float32(std)
    if round_bf16:
        base = bf16_bits_to_f32(f32_to_bf16_bits(base)).reshape(-1)
    for i, (name, shape) in enumerate(sorted(param_shapes(cfg).items())):
        if len(shape) == 1:
            yield name, np.ones(shape, np.float32)
            continue
        n = int(np.prod(shape))
        yield name, np.resize(np.roll(base, 7919 * i), n).reshape(shape)


def token_ids(seed: int, n: int, vocab: int) -> np.ndarray:
    return np.random.default_rng(seed).integers(0, vocab, size=n).astype(np.float32)
