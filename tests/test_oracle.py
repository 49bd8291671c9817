"""CPU tests of the oracle (the C restatement of the reference).  The reference has no golden vectors
(parity unpinned), so the oracle is checked three ways: against an independent float64 numpy model,
f32 against its own f64 shadow, and against the committed fixtures it generated."""
from pathlib import Path

import numpy as np
import pytest

import np_reference as NP
from helpers import make_params, rel_err, small_cfg

GOLD = Path(__file__).resolve().parent / "golden"


class _L:
    from lumen_b200.llama import LlamaConfig


def _run(oracle, cfg, params, ids, prompt_len, prec):
    m = oracle.Llama(cfg, params, prec)
    caches = m.init_kv_caches(ids.shape[0])
    outs = [m.forward(ids[:, :prompt_len], caches)]
    for t in range(prompt_len, ids.shape[1]):
        outs.append(m.forward(ids[:, t:t + 1], caches))
    assert caches[0].len == ids.shape[1]
    return np.concatenate(outs, axis=1)


@pytest.mark.parametrize("over", [dict(), dict(num_key_value_heads=4), dict(num_key_value_heads=1),
                                  dict(head_dim=32, qk_norm=True, rope_theta=1e6)])
def test_oracle_matches_independent_numpy_model(oracle, over):
    cfg = small_cfg(**over)
    params = make_params(_L, cfg, 3, std=0.08, random_norms=True)
    ids = np.random.default_rng(4).integers(0, cfg["vocab_size"], size=(2, 9)).astype(np.float32)
    want = NP.llama_logits(cfg, params, ids)
    got64 = _run(oracle, cfg, params, ids, 4, "f64")
    got32 = _run(oracle, cfg, params, ids, 4, "f32")
    # f64 shadow: the +1e-9 / libm differences only; f32: rounding of a 2-layer model
    assert rel_err(got64, want) < 1e-7
    assert rel_err(got32, want) < 2e-5


def test_decode_equals_prefill(oracle):
    cfg = small_cfg()
    params = make_params(_L, cfg, 5, std=0.08)
    ids = np.random.default_rng(6).integers(0, cfg["vocab_size"], size=(1, 8)).astype(np.float32)
    a = _run(oracle, cfg, params, ids, 8 - 1, "f64")
    b = _run(oracle, cfg, params, ids, 2, "f64")
    assert rel_err(a, b) < 1e-9


@pytest.mark.parametrize("name", ["llama_small_gqa", "llama_small_b3", "llama_small_qknorm"])
def test_oracle_reproduces_golden(oracle, name):
    g = np.load(GOLD / f"{name}.npz")
    cfg = {k[4:]: g[k].item() for k in g.files if k.startswith("cfg_")}
    params = make_params(_L, cfg, int(g["seed"]), std=float(g["std"]), random_norms=True)
    ids, pl = g["ids"], int(g["prompt_len"])
    out = _run(oracle, cfg, params, ids, pl, "f32")
    got = out[:, pl - 1:]
    # libm may dispatch different expf/cosf variants per CPU: last-ulp differences only
    assert rel_err(got, g["logits"]) < 1e-6


def test_ops_golden_and_shadow(oracle):
    g = np.load(GOLD / "ops.npz")
    pairs = [(oracle.rmsnorm(g["rms_x"], g["rms_w"], 1e-5), g["rms_out"]),
             (oracle.matmul(g["mm_a"], g["mm_w"]), g["mm_out"]),
             (oracle.rope_forward(g["rope_x"], 4, 32, 10000.0), g["rope_out"]),
             (oracle.fused_softmax(g["sm_x"], 0.25, True), g["sm_out"]),
             (oracle.silu(g["silu_x"]), g["silu_out"])]
    for got, want in pairs:
        assert rel_err(got, want) < 1e-6
    # the M == 1 product is a k-ordered f32 sum: identical to an explicit sequential loop
    a, w = g["mm_a"].reshape(-1), g["mm_w"]
    seq = np.zeros(w.shape[0], np.float32)
    for n in range(w.shape[0]):
        s = np.float32(0)
        for k in range(a.size):
            s = np.float32(s + np.float32(w[n, k] * a[k]))
        seq[n] = s
    assert np.array_equal(seq, oracle.matmul(g["mm_a"], g["mm_w"]).reshape(-1))
    assert rel_err(oracle.matmul(g["mm_a"], g["mm_w"], "f64"), g["mm_a"].astype(np.float64) @ w.T.astype(np.float64)) < 1e-14


def test_fused_softmax_semantics(oracle):
    x = np.random.default_rng(0).standard_normal((1, 2, 3, 5)).astype(np.float32)
    causal = oracle.fused_softmax(x, 0.5, True, "f64")
    assert np.all(causal[..., 0, 1:] == 0) and np.all(causal[..., 1, 2:] == 0)
    assert np.allclose(causal.sum(-1), 1.0, atol=1e-8)
    # q_len == 1: the mask is skipped even when causal (src/ops/fused.rs:51)
    one = oracle.fused_softmax(x[:, :, :1], 0.5, True, "f64")
    assert np.all(one > 0)


def test_error_conditions(oracle):
    cfg = small_cfg(max_seq_len=6)
    params = make_params(_L, cfg, 1)
    m = oracle.Llama(cfg, params)
    c = m.init_kv_caches(1)
    with pytest.raises(IndexError):   # embedding id >= vocab (embedding.rs:55)
        m.forward(np.array([[97.0]]), c)
    m.forward(np.zeros((1, 5)), c)
    m.forward(np.zeros((1, 1)), c)
    with pytest.raises(OverflowError):  # KV overflow (self_attention.rs:144-149)
        m.forward(np.zeros((1, 1)), c)
    with pytest.raises(ValueError):   # cache count (llama.rs:182-188)
        m.forward(np.zeros((1, 1)), c[:1])
    with pytest.raises(ValueError):   # K mismatch (matmul.rs:33-38)
        oracle.matmul(np.zeros((1, 4), np.float32), np.zeros((3, 5), np.float32))


def test_llama_kv_cache(oracle):
    c = oracle.LlamaKVCache(2, 8, 4)
    k = np.arange(2 * 3 * 4, dtype=np.float32).reshape(1, 2, 3, 4)
    c.update(k, -k, 2)
    kk, vv = c.get_view(5)
    assert kk.shape == (1, 2, 5, 4) and np.all(kk[:, :, :2] == 0)
    assert np.array_equal(kk[:, :, 2:], k) and np.array_equal(vv[:, :, 2:], -k)
    with pytest.raises(OverflowError):
        c.update(k, k, 6)


def test_bf16_rounding(oracle):
    from lumen_b200.tensor import bf16_bits_to_f32, f32_to_bf16_bits
    x = np.random.default_rng(2).standard_normal(10000).astype(np.float32)
    x[:4] = [1.00390625, 1.01171875, -0.0, 3.0e38]  # ties to even both ways
    assert np.array_equal(oracle.round_bf16(x), bf16_bits_to_f32(f32_to_bf16_bits(x)))
