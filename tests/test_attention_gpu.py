"""GPU parity tests of GQA attention over the static KV cache against the CPU oracle."""
import numpy as np
import pytest

from helpers import rel_err

pytestmark = pytest.mark.gpu


def _decode_case(L, oracle, ctx, b, hq, hkv, d, ctx_len, max_seq, seed, steps=1, theta=1e4):
    """Fill both caches with the same random K/V of length ctx_len - 1... then decode `steps` tokens."""
    rng = np.random.default_rng(seed)
    past = ctx_len - 1
    k = np.zeros((b, hkv, max_seq, d), np.float32)
    v = np.zeros((b, hkv, max_seq, d), np.float32)
    k[:, :, :past] = rng.standard_normal((b, hkv, past, d), dtype=np.float32)
    v[:, :, :past] = rng.standard_normal((b, hkv, past, d), dtype=np.float32)
    gc = L.KVCacheInner(b, hkv, max_seq, d)
    gc.write(k, v, past)
    oc = oracle.KVCache(b, hkv, max_seq, d, "f64")
    oc32 = oracle.KVCache(b, hkv, max_seq, d, "f32")
    for c in (oc, oc32):
        c.k[...] = k
        c.v[...] = v
        c.len = past
    rope = L.RotaryEmbedding(d, max_seq, theta)
    worst = 0.0
    for _ in range(steps):
        q = rng.standard_normal((b, 1, hq * d), dtype=np.float32)
        kn = rng.standard_normal((b, 1, hkv * d), dtype=np.float32)
        vn = rng.standard_normal((b, 1, hkv * d), dtype=np.float32)
        want = oracle.attention(q, kn, vn, oc, hq, theta, max_seq)  # [B,1,Hq,D] float64
        want32 = oracle.attention(q, kn, vn, oc32, hq, theta, max_seq)
        tq, tk, tv = (L.Tensor.from_array_no_grad(a) for a in (q, kn, vn))
        out = L.Tensor.from_array_no_grad(np.zeros((b, hq * d), np.float32))
        L.attention_decode(ctx, tq.data_ptr, tk.data_ptr, tv.data_ptr, hq, gc, rope, out.data_ptr)
        got = out.data().reshape(b, 1, hq, d)
        # the f64 shadow also evaluates the RoPE angles in f64, which moves far positions by ~pos*6e-8 rad;
        # the f32 oracle shares the reference's f32 table recipe
        worst = max(worst, min(rel_err(got, want), rel_err(got, want32)))
        assert rel_err(got, want) < 1e-3
        assert gc.len == oc.len
    # the appended rows are bit-identical to the f32 oracle's (same f32 table, unfused f32 mul/add/sub)
    gk, gv = gc.read()
    n = gc.len
    assert np.array_equal(gk[:, :, :n], oc32.k[:, :, :n])
    assert np.array_equal(gv[:, :, :n], oc32.v[:, :, :n])
    assert np.all(gk[:, :, n:] == 0)
    return worst


# Benchmark configuration 3: 32 q heads, 4 KV heads, head_dim 64; contexts 128..8192; batch 1 and 16
@pytest.mark.parametrize("ctx_len", [128, 512, 2048, 8192])
@pytest.mark.parametrize("b", [1, 16])
def test_decode_attention_config3(L, oracle, ctx, ctx_len, b):
    err = _decode_case(L, oracle, ctx, b, 32, 4, 64, ctx_len, ctx_len + 8, seed=3, steps=2)
    assert err < 2e-5, err


@pytest.mark.parametrize("ctx_len", [1, 2, 3, 63, 64, 65, 129, 1000])
def test_decode_attention_split_boundaries(L, oracle, ctx, ctx_len):
    err = _decode_case(L, oracle, ctx, 2, 8, 2, 64, ctx_len, 1024, seed=ctx_len, steps=3)
    assert err < 2e-5, err


@pytest.mark.parametrize("hq,hkv,d", [(16, 4, 128), (16, 2, 128), (16, 4, 64), (32, 4, 64)])
def test_decode_attention_tiled_kernel_geometries(L, oracle, ctx, hq, hkv, d):
    """Long contexts of grouped-query models (groups of 4 and 8, head_dim 64 and 128) at a batch large enough
    that each split holds several tiles of rows: the TMA-fed tiled kernel.  The context is not a multiple of
    the tile, the appended row falls inside a tile, and the second step crosses into a new row."""
    err = _decode_case(L, oracle, ctx, 8, hq, hkv, d, 1499, 1536, seed=hq + hkv + d, steps=2, theta=1e6)
    assert err < 2e-5, err


@pytest.mark.parametrize("hq,hkv,d", [(32, 32, 128), (32, 8, 128), (6, 2, 32), (4, 4, 16), (5, 1, 48), (2, 1, 256)])
def test_decode_attention_head_geometries(L, oracle, ctx, hq, hkv, d):
    err = _decode_case(L, oracle, ctx, 2, hq, hkv, d, 200, 256, seed=hq + d, steps=2, theta=1e6)
    assert err < 2e-5, err


def test_decode_fills_cache_to_max_then_overflows(L, oracle, ctx):
    err = _decode_case(L, oracle, ctx, 1, 4, 2, 32, 15, 16, seed=1, steps=2)  # 14 -> 16 rows
    assert err < 2e-5
    gc = L.KVCacheInner(1, 2, 4, 32)
    rope = L.RotaryEmbedding(32, 4, 1e4)
    z = L.Tensor.from_array_no_grad(np.ones((1, 4 * 32), np.float32))
    out = L.Tensor.from_array_no_grad(np.zeros((1, 4 * 32), np.float32))
    for _ in range(4):
        L.attention_decode(ctx, z.data_ptr, z.data_ptr, z.data_ptr, 4, gc, rope, out.data_ptr)
    with pytest.raises(L.LumenError) as e:  # assert at self_attention.rs:144-149
        L.attention_decode(ctx, z.data_ptr, z.data_ptr, z.data_ptr, 4, gc, rope, out.data_ptr)
    assert e.value.code == L._lib.ERR_KV_OVERFLOW
    assert gc.len == 4
    gc.reset()  # len = 0, contents kept (self_attention.rs:41-43)
    assert gc.len == 0
    k, _ = gc.read()
    assert np.any(k != 0)


def _self_attention_case(L, oracle, e, hq, hkv, max_seq, b, chunks, seed, bf16=False):
    rng = np.random.default_rng(seed)
    d = e // hq
    kvd = hkv * d
    ws = [rng.standard_normal(s, dtype=np.float32) * np.float32(e ** -0.5) for s in ((e, e), (kvd, e), (kvd, e), (e, e))]
    if bf16:
        ws = [oracle.round_bf16(w) for w in ws]
    mk = L.Tensor.from_bf16 if bf16 else L.Tensor.from_array_no_grad
    attn = L.SelfAttention(e, hq, hkv, max_seq, 10000.0, True)
    attn.set_weights(*[mk(w) for w in ws])
    oc = oracle.KVCache(b, hkv, max_seq, d, "f64")
    cache = None
    worst = 0.0
    with L.no_grad():
        for s in chunks:
            x = rng.standard_normal((b, s, e), dtype=np.float32)
            out, cache = attn.forward(L.Tensor.from_array_no_grad(x), cache)
            q, k, v = (oracle.matmul(x, w, "f64").astype(np.float32) for w in ws[:3])
            ctx_ = oracle.attention(q, k, v, oc, hq, 10000.0, max_seq)
            want = oracle.matmul(ctx_.reshape(b, s, e).astype(np.float32), ws[3], "f64")
            worst = max(worst, rel_err(out.data(), want))
            assert cache.len == oc.len
    return worst


@pytest.mark.parametrize("chunks", [[7, 1, 1, 1], [1, 1, 5, 1], [32, 1], [3, 9, 1, 1]])
def test_self_attention_prefill_then_decode(L, oracle, chunks):
    """SelfAttention::forward: cache created when None, S > 1 prefill (also into a non-empty cache:
    the absolute-position causal mask `j > past_len + i`) and S == 1 decode."""
    err = _self_attention_case(L, oracle, 64, 4, 2, 64, 2, chunks, seed=sum(chunks))
    assert err < 2e-5, err


def test_self_attention_tinyllama_geometry(L, oracle):
    err = _self_attention_case(L, oracle, 2048, 32, 4, 128, 1, [32, 1, 1], seed=0)
    assert err < 2e-5, err
    err = _self_attention_case(L, oracle, 2048, 32, 4, 128, 1, [16, 1], seed=1, bf16=True)
    assert err < 2e-5, err


@pytest.mark.parametrize("e,hq,hkv", [(256, 4, 2), (512, 4, 1), (512, 4, 4)])
@pytest.mark.parametrize("chunks", [[200, 1], [64, 130, 1, 70], [129], [300, 1, 1]])
def test_self_attention_tensor_core_prefill(L, oracle, e, hq, hkv, chunks):
    """Prompts of 64 positions and more with head dimensions 64 / 128 take the tensor-core prefill kernel
    (tiles of 128 queries x 64 cached rows, hi/lo bf16 products): ragged tile edges, a second prompt into a
    non-empty cache (mask j > past_len + i), grouped and ungrouped heads, two batch rows."""
    err = _self_attention_case(L, oracle, e, hq, hkv, 512, 2, chunks, seed=e + sum(chunks))
    assert err < 5e-5, err


def test_self_attention_errors(L):
    attn = L.SelfAttention(32, 4, 2, 6, 10000.0, True)
    w = [np.zeros(s, np.float32) for s in ((32, 32), (16, 32), (16, 32), (32, 32))]
    with L.no_grad():
        with pytest.raises(L.LumenError) as e:
            attn.forward(L.Tensor.from_array_no_grad(np.zeros((1, 2, 32), np.float32)))
        assert e.value.code == L._lib.ERR_MISSING_PARAM
        attn.set_weights(*[L.Tensor.from_array_no_grad(a) for a in w])
        _, cache = attn.forward(L.Tensor.from_array_no_grad(np.zeros((1, 5, 32), np.float32)))
        with pytest.raises(L.LumenError) as e:  # prefill past the RoPE table (encoding.rs:62-68)
            attn.forward(L.Tensor.from_array_no_grad(np.zeros((1, 2, 32), np.float32)), cache)
        assert e.value.code == L._lib.ERR_ROPE_RANGE
        attn.forward(L.Tensor.from_array_no_grad(np.zeros((1, 1, 32), np.float32)), cache)
        with pytest.raises(L.LumenError) as e:  # decode past max_seq (self_attention.rs:144-149)
            attn.forward(L.Tensor.from_array_no_grad(np.zeros((1, 1, 32), np.float32)), cache)
        assert e.value.code == L._lib.ERR_KV_OVERFLOW
    with pytest.raises(NotImplementedError):  # training path is out of scope
        attn.forward(L.Tensor.from_array_no_grad(np.zeros((1, 1, 32), np.float32)))
    with pytest.raises(L.LumenError):
        L.SelfAttention(30, 4, 2, 6, 10000.0, True)  # embed dim not divisible by heads (:69-73)
