"""GPU parity tests of LlamaModel::forward (prefill + teacher-forced decode) against the CPU oracle
and the committed fixtures.  Tolerances are the north star's: per-step logits within rel 1e-4 for
f32 weights, 1e-2 for bf16 weights (rel = max|a-b| / max|b| over one logits vector), and identical
argmax token ids under teacher forcing."""
import os
from pathlib import Path

import numpy as np
import pytest

from helpers import TOL_BF16, TOL_F32, cfg_obj, make_params, rel_err, small_cfg

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).resolve().parent / "golden"


def _gpu_run(L, cfg, params, ids, prompt_len, weight_dtype="f32", last_only=False):
    model = L.LlamaModel(cfg_obj(L, cfg, weight_dtype))
    model.load_state(params)
    caches = model.init_kv_caches(ids.shape[0])
    outs = []
    with L.no_grad():
        lg = model.forward(ids[:, :prompt_len], caches, 0, last_only=last_only)
        outs.append(lg[:, None] if last_only else lg)
        for t in range(prompt_len, ids.shape[1]):
            outs.append(model.forward(ids[:, t:t + 1], caches, 0))
    assert all(c.len == ids.shape[1] for c in caches)
    return np.concatenate(outs, axis=1), model, caches


def _oracle_run(oracle, cfg, params, ids, prompt_len, prec="f32"):
    m = oracle.Llama(cfg, params, prec)
    caches = m.init_kv_caches(ids.shape[0])
    outs = [m.forward(ids[:, :prompt_len], caches)]
    for t in range(prompt_len, ids.shape[1]):
        outs.append(m.forward(ids[:, t:t + 1], caches))
    return np.concatenate(outs, axis=1), caches


@pytest.mark.parametrize("name", ["llama_small_gqa", "llama_small_b3", "llama_small_qknorm"])
def test_golden_fixtures(L, name):
    g = np.load(GOLD / f"{name}.npz")
    cfg = {k[4:]: g[k].item() for k in g.files if k.startswith("cfg_")}
    params = make_params(L, cfg, int(g["seed"]), std=float(g["std"]), random_norms=True)
    pl = int(g["prompt_len"])
    got, _, _ = _gpu_run(L, cfg, params, g["ids"], pl)
    got = got[:, pl - 1:]
    want = g["logits"]
    for t in range(want.shape[1]):
        assert rel_err(got[:, t], want[:, t]) < TOL_F32, (name, t)
    assert np.array_equal(got.argmax(-1), want.argmax(-1))


@pytest.mark.parametrize("over,batch,prompt", [
    (dict(), 1, 5), (dict(num_key_value_heads=4), 2, 1), (dict(num_key_value_heads=1), 3, 7),
    (dict(hidden_size=128, num_attention_heads=2, intermediate_size=200, vocab_size=301), 9, 3),
    (dict(head_dim=32, qk_norm=True, rope_theta=1e6), 2, 4),
])
@pytest.mark.parametrize("wdt", ["f32", "bf16"])
def test_small_models_vs_oracle(L, oracle, over, batch, prompt, wdt):
    """Covers batch sizes on both sides of the vector-matrix / GEMM switch (M <= 8 vs M > 8)."""
    cfg = small_cfg(**over)
    params = make_params(L, cfg, 21, std=0.08, round_bf16=(wdt == "bf16"), random_norms=True)
    ids = np.random.default_rng(22).integers(0, cfg["vocab_size"], size=(batch, prompt + 6)).astype(np.float32)
    got, _, gc = _gpu_run(L, cfg, params, ids, prompt, wdt)
    want, oc = _oracle_run(oracle, cfg, params, ids, prompt, "f64")
    tol = TOL_BF16 if wdt == "bf16" else TOL_F32
    for t in range(ids.shape[1]):
        assert rel_err(got[:, t], want[:, t]) < tol, t
    # bf16-rounded weights are exactly representable, so the bf16 model is as close as the f32 one
    assert rel_err(got, want) < TOL_F32
    # KV cache contents (rotated keys, values) agree with the oracle's.  Rows written by the tensor-core kernel
    # (more than 8 rows at once, or more than one over bf16 weights) come from products of two-term bf16 splits
    # (~1e-5), the others from f32 FMAs.
    rows_for_tc = 1 if wdt == "bf16" else 8  # bf16 weights take the tensor-core kernel from two rows on
    kv_tol = 5e-5 if batch * prompt > rows_for_tc or batch > rows_for_tc else 1e-5
    for l in range(cfg["num_hidden_layers"]):
        k, v = gc[l].read()
        assert rel_err(k, oc[l].k) < kv_tol and rel_err(v, oc[l].v) < kv_tol, (l, rel_err(k, oc[l].k), rel_err(v, oc[l].v))


@pytest.mark.parametrize("over", [
    dict(hidden_size=256, intermediate_size=320, num_attention_heads=4, num_key_value_heads=2),                # head_dim 64
    dict(hidden_size=256, intermediate_size=320, num_attention_heads=2, num_key_value_heads=1, head_dim=128,
         qk_norm=True, rope_theta=1e6),                                                                        # Qwen3-style
])
@pytest.mark.parametrize("wdt", ["f32", "bf16"])
def test_long_prompt_slices_tensor_core_prefill(L, oracle, over, wdt):
    """Prompts of 64 positions and more run their attention on the tensor cores.  Two prompt slices (the second
    one into a partly filled cache), then decode steps over the cache both slices wrote."""
    cfg = small_cfg(max_seq_len=256, **over)
    params = make_params(L, cfg, 71, std=0.05, round_bf16=(wdt == "bf16"), random_norms=True)
    ids = np.random.default_rng(72).integers(0, cfg["vocab_size"], size=(2, 176)).astype(np.float32)
    model = L.LlamaModel(cfg_obj(L, cfg, wdt))
    model.load_state(params)
    caches = model.init_kv_caches(2)
    m = oracle.Llama(cfg, params, "f64")
    ocaches = m.init_kv_caches(2)
    tol = TOL_BF16 if wdt == "bf16" else TOL_F32
    with L.no_grad():
        for lo, hi in [(0, 100), (100, 170)] + [(t, t + 1) for t in range(170, 176)]:
            got = model.forward(ids[:, lo:hi], caches, 0)
            want = m.forward(ids[:, lo:hi], ocaches)
            for t in range(hi - lo):
                assert rel_err(got[:, t], want[:, t]) < tol, (lo, t, rel_err(got[:, t], want[:, t]))
            assert rel_err(got, want) < TOL_F32
            assert np.array_equal(got.argmax(-1), want.argmax(-1))
    for l in range(cfg["num_hidden_layers"]):
        k, v = caches[l].read()
        assert rel_err(k, ocaches[l].k) < 5e-5 and rel_err(v, ocaches[l].v) < 5e-5


def test_forward_last_and_device_entry_points(L, oracle):
    cfg = small_cfg()
    params = make_params(L, cfg, 31, std=0.08)
    ids = np.random.default_rng(32).integers(0, cfg["vocab_size"], size=(2, 6)).astype(np.float32)
    full, _, _ = _gpu_run(L, cfg, params, ids, 4)
    last, _, _ = _gpu_run(L, cfg, params, ids, 4, last_only=True)
    assert np.array_equal(last[:, 0], full[:, 3]) and np.array_equal(last[:, 1:], full[:, 4:])
    # device-resident ids / logits
    model = L.LlamaModel(cfg_obj(L, cfg))
    model.load_state(params)
    caches = model.init_kv_caches(2)
    d_out = L.Tensor.from_array_no_grad(np.zeros((2, 4, cfg["vocab_size"]), np.float32))
    d_ids4 = L.Tensor.from_array_no_grad(np.ascontiguousarray(ids[:, :4]))
    with L.no_grad():
        model.forward_device(d_ids4.data_ptr, 2, 4, caches, d_out.data_ptr)
    model.ctx.synchronize()
    assert np.array_equal(d_out.data(), full[:, :4])


def test_graph_replay_equals_eager(L, monkeypatch):
    """Decode steps replay a captured CUDA graph from the third call on; results are identical to the
    eager launches and the context length advances on the device."""
    cfg = small_cfg(max_seq_len=300)
    params = make_params(L, cfg, 41, std=0.08)
    ids = np.random.default_rng(42).integers(0, cfg["vocab_size"], size=(1, 280)).astype(np.float32)
    monkeypatch.setenv("LUMEN_NO_MEGA", "1")  # batch 1 would otherwise take the persistent kernel
    graph, _, _ = _gpu_run(L, cfg, params, ids, 3)
    monkeypatch.setenv("LUMEN_NO_GRAPH", "1")
    eager, _, _ = _gpu_run(L, cfg, params, ids, 3)
    assert np.array_equal(graph, eager)


@pytest.mark.parametrize("over", [dict(), dict(num_key_value_heads=1, hidden_size=96, num_attention_heads=6),
                                  dict(head_dim=32, qk_norm=True, rope_theta=1e6),
                                  dict(hidden_size=256, intermediate_size=2304, num_attention_heads=4, vocab_size=1000)])
@pytest.mark.parametrize("wdt", ["f32", "bf16"])
def test_persistent_kernel_equals_per_op_path(L, oracle, monkeypatch, over, wdt):
    """Batch-1 decode runs as one persistent kernel per token; the per-op kernels (one launch per
    operator) compute the same step.  Both are checked against the oracle and against each other over a
    context that crosses the attention split thresholds."""
    cfg = small_cfg(max_seq_len=200, **over)
    params = make_params(L, cfg, 61, std=0.08, round_bf16=(wdt == "bf16"), random_norms=True)
    ids = np.random.default_rng(62).integers(0, cfg["vocab_size"], size=(1, 180)).astype(np.float32)
    mega, _, gc = _gpu_run(L, cfg, params, ids, 2, wdt)
    monkeypatch.setenv("LUMEN_NO_MEGA", "1")
    per_op, _, _ = _gpu_run(L, cfg, params, ids, 2, wdt)
    want, oc = _oracle_run(oracle, cfg, params, ids, 2, "f64")
    for t in range(ids.shape[1]):
        assert rel_err(mega[:, t], want[:, t]) < TOL_F32, t
    assert rel_err(mega, per_op) < 2e-5
    for l in range(cfg["num_hidden_layers"]):
        k, v = gc[l].read()
        assert rel_err(k, oc[l].k) < 1e-5 and rel_err(v, oc[l].v) < 1e-5


def test_reset_and_reuse_caches(L):
    cfg = small_cfg()
    params = make_params(L, cfg, 51, std=0.08)
    ids = np.random.default_rng(52).integers(0, cfg["vocab_size"], size=(1, 9)).astype(np.float32)
    first, model, caches = _gpu_run(L, cfg, params, ids, 4)
    model.reset_kv_caches(caches)  # len = 0, slab contents kept (llama.rs:172-176)
    assert all(c.len == 0 for c in caches)
    with L.no_grad():
        again = [model.forward(ids[:, :4], caches)] + [model.forward(ids[:, t:t + 1], caches) for t in range(4, 9)]
    assert np.array_equal(first, np.concatenate(again, axis=1))


def test_error_conditions(L):
    cfg = small_cfg(max_seq_len=6)
    model = L.LlamaModel(cfg_obj(L, cfg))
    caches = model.init_kv_caches(1)
    one = np.zeros((1, 1), np.float32)
    with pytest.raises(NotImplementedError):
        model.forward(one, caches)  # outside no_grad: training path is out of scope
    with L.no_grad():
        with pytest.raises(L.LumenError) as e:
            model.forward(one, caches)
        assert e.value.code == L._lib.ERR_MISSING_PARAM
        model.load_state(make_params(L, cfg, 1))
        with pytest.raises(L.LumenError) as e:
            model.set_param("model.layers.9.mlp.up_proj.weight", np.zeros((160, 64), np.float32))
        assert e.value.code == L._lib.ERR_PARAM_NAME
        with pytest.raises(L.LumenError) as e:
            model.set_param("lm_head.weight", np.zeros((5, 5), np.float32))
        assert e.value.code == L._lib.ERR_SHAPE
        with pytest.raises(L.LumenError) as e:  # llama.rs:182-188
            model.forward(one, caches[:1])
        assert e.value.code == L._lib.ERR_CACHE_COUNT
        with pytest.raises(L.LumenError) as e:  # embedding.rs:55
            model.forward(np.full((1, 1), 97.0, np.float32), caches)
        assert e.value.code == L._lib.ERR_EMBED_RANGE
        assert caches[0].len == 0  # nothing ran
        with pytest.raises(L.LumenError) as e:  # prefill longer than the RoPE table
            model.forward(np.zeros((1, 7), np.float32), caches)
        assert e.value.code == L._lib.ERR_ROPE_RANGE
        model.forward(np.zeros((1, 5), np.float32), caches)
        model.forward(one, caches)
        with pytest.raises(L.LumenError) as e:  # self_attention.rs:144-149
            model.forward(one, caches)
        assert e.value.code == L._lib.ERR_KV_OVERFLOW
        assert caches[0].len == 6
        wrong = L.LlamaModel(cfg_obj(L, small_cfg(max_seq_len=6, num_key_value_heads=4)))
        with pytest.raises(L.LumenError) as e:
            model.forward(one, wrong.init_kv_caches(1))
        assert e.value.code == L._lib.ERR_SHAPE


@pytest.fixture(scope="module")
def tinyllama_f32(L, oracle):
    """Benchmark configuration 1 at full size (f32 weights N(0,0.02) from seed 0, gains 1.0) on both sides."""
    from lumen_b200 import synth
    cfg = dict(synth.TINYLLAMA)
    params = make_params(L, cfg, 0, std=0.02)
    model = L.LlamaModel(cfg_obj(L, cfg, "f32"))
    model.load_state(params)
    return cfg, params, model, oracle.Llama(cfg, params, "f32")


def _teacher_forced(L, model, ref, ids, prompt, caches=None, rcaches=None):
    caches = caches or model.init_kv_caches(1)
    rcaches = rcaches or ref.init_kv_caches(1)
    got, want = [], []
    with L.no_grad():
        if prompt:
            got.append(model.forward(ids[:, :prompt], caches)[:, -1:])
            want.append(ref.forward(ids[:, :prompt], rcaches)[:, -1:])
        for t in range(prompt, ids.shape[1]):
            got.append(model.forward(ids[:, t:t + 1], caches))
            want.append(ref.forward(ids[:, t:t + 1], rcaches))
    return np.concatenate(got, axis=1), np.concatenate(want, axis=1)


def test_tinyllama_config1_teacher_forced_f32(L, tinyllama_f32):
    """Benchmark configuration 1 at full size: TinyLlama-1.1B shape, 32 prompt ids from seed 1 and 128
    teacher-forced decode steps at batch 1, cache sized to 2048."""
    from lumen_b200 import synth
    cfg, _, model, ref = tinyllama_f32
    prompt, steps = 32, 128
    ids = synth.token_ids(1, prompt + steps, cfg["vocab_size"])[None, :]
    got, want = _teacher_forced(L, model, ref, ids, prompt)
    errs = [rel_err(got[0, t], want[0, t]) for t in range(got.shape[1])]
    print(f"\nconfig1 f32: max rel err over {len(errs)} steps = {max(errs):.3e}")
    assert max(errs) < TOL_F32
    assert np.array_equal(got[0].argmax(-1), want[0].argmax(-1))


def test_tinyllama_last_positions_of_the_cache(L, tinyllama_f32):
    """The same full-size model decoding across positions 2030..2047, the end of the static cache and of the
    RoPE table: both sides start from the same random cache contents of length 2030.  Covers the merge of the
    context splits and the f32 rotation angles at the far end of the table, then the overflow status."""
    cfg, _, model, ref = tinyllama_f32
    rng = np.random.default_rng(2030)
    start, max_seq = 2030, cfg["max_seq_len"]
    caches, rcaches = model.init_kv_caches(1), ref.init_kv_caches(1)
    shape = (1, cfg["num_key_value_heads"], max_seq, cfg["hidden_size"] // cfg["num_attention_heads"])
    for c, rc in zip(caches, rcaches):
        k = np.zeros(shape, np.float32)
        v = np.zeros(shape, np.float32)
        k[:, :, :start] = 0.5 * rng.standard_normal((shape[0], shape[1], start, shape[3]), dtype=np.float32)
        v[:, :, :start] = 0.5 * rng.standard_normal((shape[0], shape[1], start, shape[3]), dtype=np.float32)
        c.write(k, v, start)
        rc.k[...] = k
        rc.v[...] = v
        rc.len = start
    ids = rng.integers(0, cfg["vocab_size"], size=(1, max_seq - start)).astype(np.float32)
    got, want = _teacher_forced(L, model, ref, ids, 0, caches, rcaches)
    errs = [rel_err(got[0, t], want[0, t]) for t in range(got.shape[1])]
    print(f"\nconfig1 f32, positions {start}..{max_seq - 1}: max rel err = {max(errs):.3e}")
    assert max(errs) < TOL_F32
    assert np.array_equal(got[0].argmax(-1), want[0].argmax(-1))
    assert all(c.len == max_seq for c in caches)
    with L.no_grad(), pytest.raises(L.LumenError) as e:  # self_attention.rs:144-149
        model.forward(ids[:, :1], caches)
    assert e.value.code == L._lib.ERR_KV_OVERFLOW


def test_tinyllama_config1_teacher_forced_bf16(L, oracle):
    """Configuration 1 with the same weights rounded to bf16 (f32 accumulation); fewer steps to bound the CPU
    oracle's time."""
    from lumen_b200 import synth
    cfg = dict(synth.TINYLLAMA)
    prompt, steps = 32, 24
    params = make_params(L, cfg, 0, std=0.02, round_bf16=True)
    ids = synth.token_ids(1, prompt + steps, cfg["vocab_size"])[None, :]
    got, _, _ = _gpu_run(L, cfg, params, ids, prompt, "bf16")
    want, _ = _oracle_run(oracle, cfg, params, ids, prompt, "f32")
    errs = [rel_err(got[0, t], want[0, t]) for t in range(prompt - 1, prompt + steps)]
    print(f"\nconfig1 bf16: max rel err over {len(errs)} steps = {max(errs):.3e}")
    assert max(errs) < TOL_BF16
    assert np.array_equal(got[0, prompt - 1:].argmax(-1), want[0, prompt - 1:].argmax(-1))


def _tiled_params(L, cfg, seed, random_norms=False):
    """bf16-representable N(0, 0.02) weights for the multi-billion-parameter geometries: every matrix repeats one
    seeded block of draws whose length is not a multiple of any row length, so no two rows are equal (drawing
    1.6 G values one by one would take minutes)."""
    from lumen_b200 import synth
    params = dict(synth.iter_params_tiled(L.LlamaConfig(**cfg), seed, std=0.02, round_bf16=True, block=(1 << 22) + 7))
    if random_norms:
        rng = np.random.default_rng(seed + 1000)
        for k in params:
            if params[k].ndim == 1:
                params[k] = (1.0 + 0.1 * rng.standard_normal(params[k].shape)).astype(np.float32)
    return params


def test_llama2_7b_geometry_two_layers(L, oracle):
    """Benchmark configuration 4's geometry (hidden 4096, 32 heads of 128 without grouping, intermediate 11008,
    vocabulary 32000, bf16 weights with f32 accumulation) cut to two layers: a 64-token prompt (tensor-core GEMMs
    and prefill attention) and 8 teacher-forced decode steps through the persistent kernel."""
    from lumen_b200 import synth
    cfg = dict(synth.LLAMA2_7B, num_hidden_layers=2, max_seq_len=128)
    params = _tiled_params(L, cfg, 4)
    prompt, steps = 64, 8
    ids = synth.token_ids(4, prompt + steps, cfg["vocab_size"])[None, :]
    got, _, _ = _gpu_run(L, cfg, params, ids, prompt, "bf16")
    want, _ = _oracle_run(oracle, cfg, params, ids, prompt, "f32")
    errs = [rel_err(got[0, t], want[0, t]) for t in range(prompt + steps)]
    print(f"\nLlama-2-7B geometry, 2 layers, bf16: max rel err over {len(errs)} positions = {max(errs):.3e}")
    assert max(errs) < TOL_BF16
    assert np.array_equal(got[0].argmax(-1), want[0].argmax(-1))


def test_qwen3_8b_geometry_two_layers_batched(L, oracle):
    """Benchmark configuration 5's geometry (32 query heads and 8 KV heads of 128, per-head q/k RMSNorm, intermediate
    12288, vocabulary 151936, theta 1e6, bf16 weights) cut to two layers and two sequences: a 128-token prefix in two
    slices of 64 (the second into a partly filled cache), then 4 batched decode steps."""
    from lumen_b200 import synth
    cfg = dict(synth.QWEN3_8B, num_hidden_layers=2, max_seq_len=192)
    params = _tiled_params(L, cfg, 5, random_norms=True)
    b, prefix, steps = 2, 128, 4
    ids = synth.token_ids(5, b * (prefix + steps), cfg["vocab_size"]).reshape(b, prefix + steps)
    model = L.LlamaModel(cfg_obj(L, cfg, "bf16"))
    model.load_state(params)
    caches = model.init_kv_caches(b)
    ref = oracle.Llama(cfg, params, "f32")
    rcaches = ref.init_kv_caches(b)
    worst = 0.0
    with L.no_grad():
        for lo, hi in [(0, 64), (64, 128)] + [(t, t + 1) for t in range(prefix, prefix + steps)]:
            got = model.forward(ids[:, lo:hi], caches)
            want = ref.forward(ids[:, lo:hi], rcaches)
            for t in range(hi - lo):
                worst = max(worst, rel_err(got[:, t], want[:, t]))
            assert np.array_equal(got.argmax(-1), want.argmax(-1)), (lo, hi)
    print(f"\nQwen3-8B geometry, 2 layers, batch {b}, bf16: max rel err = {worst:.3e}")
    assert worst < TOL_BF16
    assert all(c.len == prefix + steps for c in caches)
