"""Shared helpers for the parity tests."""
from __future__ import annotations

import numpy as np

# Tolerances from the north star: per-step logits within rel 1e-4 for f32 weights, 1e-2 for bf16
# weights, where rel = max|a-b| / max|b| over one logits vector (error against the logit scale).
TOL_F32 = 1e-4
TOL_BF16 = 1e-2


def rel_err(a, b) -> float:
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    denom = max(float(np.max(np.abs(b))), 1e-30)
    return float(np.max(np.abs(a - b))) / denom


def small_cfg(**over) -> dict:
    cfg = dict(vocab_size=97, hidden_size=64, intermediate_size=160, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, rms_norm_eps=1e-5, max_seq_len=48, rope_theta=10000.0)
    cfg.update(over)
    return cfg


def cfg_obj(L, cfg: dict, weight_dtype="f32"):
    return L.LlamaConfig(**cfg, weight_dtype=weight_dtype)


def make_params(L, cfg: dict, seed: int, std: float = 0.02, round_bf16: bool = False, random_norms: bool = False) -> dict:
    from lumen_b200 import synth
    params = dict(synth.iter_params(L.LlamaConfig(**cfg), seed, std=std, round_bf16=round_bf16))
    if random_norms:
        rng = np.random.default_rng(seed + 1000)
        for k in params:
            if params[k].ndim == 1:
                params[k] = (1.0 + 0.1 * rng.standard_normal(params[k].shape)).astype(np.float32)
    return params
