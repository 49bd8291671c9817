"""GPU parity tests of the operator-level C ABI against the CPU oracle.

Element-wise ops (no reduction) must match the oracle's f32 arithmetic bit for bit, apart from
`expf` whose last ulp differs between glibc and CUDA.  Reductions (dot products, sums of
squares) use a different summation order than the reference's sequential loops, so they are
compared within f32 rounding and against the f64 shadow."""
import numpy as np
import pytest

from helpers import rel_err

pytestmark = pytest.mark.gpu

# Benchmark configuration 2: (K, N) of the standalone M = 1 sweep
SWEEP = [(2048, 2048), (2048, 256), (2048, 5632), (5632, 2048), (2048, 32000), (4096, 11008), (11008, 4096)]


def _gemv_case(L, oracle, k, n, seed, bf16):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((1, 1, k), dtype=np.float32)
    w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)
    if bf16:
        w = oracle.round_bf16(w)
    xt = L.Tensor.from_array_no_grad(x)
    wt = L.Tensor.from_bf16(w) if bf16 else L.Tensor.from_array_no_grad(w)
    got = L.matmul(xt, wt).data()
    assert got.shape == (1, 1, n)
    want32 = oracle.matmul(x, w, "f32")
    want64 = oracle.matmul(x, w, "f64")
    scale = np.abs(want64).max()
    err_gpu = np.abs(got - want64).max() / scale
    err_cpu = np.abs(want32 - want64).max() / scale
    # both f32 results bracket the f64 value; the tree sum is at least as accurate as the sequential one
    assert err_gpu < 2e-6, (k, n, err_gpu)
    assert err_gpu <= 4 * err_cpu + 1e-7
    assert rel_err(got, want32) < 1e-5
    return x, w, got


@pytest.mark.parametrize("k,n", SWEEP)
@pytest.mark.parametrize("bf16", [False, True])
def test_gemv_sweep_shapes(L, oracle, k, n, bf16):
    _gemv_case(L, oracle, k, n, 2, bf16)


@pytest.mark.parametrize("k,n", [(1, 1), (3, 5), (77, 13), (130, 9), (64, 1), (2050, 17), (8, 4000)])
@pytest.mark.parametrize("bf16", [False, True])
def test_gemv_ragged_shapes(L, oracle, k, n, bf16):
    """K not a multiple of the vector width, tiny N, N not a multiple of the warps per CTA."""
    _gemv_case(L, oracle, k, n, 5, bf16)


@pytest.mark.parametrize("m", [2, 3, 5, 8, 9, 32, 70])
@pytest.mark.parametrize("bf16", [False, True])
def test_matmul_m_gt_1(L, oracle, m, bf16):
    """M > 1 branch (matmul.rs:70-92): small M streams the weights once, larger M uses GEMM tiles."""
    rng = np.random.default_rng(m)
    k, n = 200, 150
    a = rng.standard_normal((m, k), dtype=np.float32)
    w = rng.standard_normal((n, k), dtype=np.float32)
    if bf16:
        w = oracle.round_bf16(w)
    wt = L.Tensor.from_bf16(w) if bf16 else L.Tensor.from_array_no_grad(w)
    got = L.matmul(L.Tensor.from_array_no_grad(a), wt).data()
    # M > 8 (M > 1 over bf16 weights) runs on the tensor cores with the f32 operands split into two bf16 terms each
    # (x = hi + lo to ~2^-17), f32 accumulation: a few 1e-6 instead of f32 rounding
    on_tensor_cores = m > 8 or (bf16 and m > 1)  # bf16 weights take that kernel from two rows on
    assert rel_err(got, oracle.matmul(a, w, "f64")) < (2e-5 if on_tensor_cores else 2e-6)


@pytest.mark.parametrize("bf16", [True, False])
@pytest.mark.parametrize("m,k,n", [(9, 64, 8), (32, 2048, 2560), (130, 200, 150), (512, 4096, 1000), (257, 5632, 2048), (64, 72, 136),
                                   (64, 128, 40), (33, 64, 24)])
def test_tensor_core_gemm_shapes(L, oracle, m, k, n, bf16):
    """tcgen05 path (bf16 weights, M > 8): tile edges in M, N and K (K not a multiple of the 64-element block,
    M and N not multiples of 128), several K blocks more than ring stages, and against the SIMT path."""
    import os
    rng = np.random.default_rng(m + k + n)
    a = rng.standard_normal((m, k), dtype=np.float32)
    w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.05)
    if bf16:
        w = oracle.round_bf16(w)
    wt = L.Tensor.from_bf16(w) if bf16 else L.Tensor.from_array_no_grad(w)  # f32 weights are split on the fly
    got = L.matmul(L.Tensor.from_array_no_grad(a), wt).data()
    want = a.astype(np.float64) @ w.astype(np.float64).T
    assert got.shape == (m, n)
    assert rel_err(got, want) < 2e-5, rel_err(got, want)


def test_matmul_batched_leading_dims_and_errors(L, oracle):
    rng = np.random.default_rng(0)
    a = rng.standard_normal((2, 3, 16), dtype=np.float32)
    w = rng.standard_normal((7, 16), dtype=np.float32)
    got = L.matmul(L.Tensor.from_array_no_grad(a), L.Tensor.from_array_no_grad(w)).data()
    assert got.shape == (2, 3, 7)
    assert rel_err(got, oracle.matmul(a, w, "f64")) < 2e-6
    with pytest.raises(L.LumenError) as e:  # K mismatch panics in the reference (matmul.rs:33-38)
        L.matmul(L.Tensor.from_array_no_grad(a), L.Tensor.from_array_no_grad(np.zeros((7, 15), np.float32)))
    assert e.value.code == L._lib.ERR_SHAPE
    with pytest.raises(L.LumenError) as e:  # RHS must be 2-D (matmul.rs:24-26)
        L.matmul(L.Tensor.from_array_no_grad(a), L.Tensor.from_array_no_grad(np.zeros((7, 4, 4), np.float32)))
    assert e.value.code == L._lib.ERR_SHAPE


@pytest.mark.parametrize("k,n", [(2048, 2048), (2048, 256), (5632, 2048), (2048, 32000), (100, 37), (33, 5)])
@pytest.mark.parametrize("bf16", [False, True])
def test_gemv_kn_layout_raw_pointers(L, oracle, ctx, k, n, bf16):
    """`lumen_gemv` with W stored [K,N] row-major (the layout benchmark configuration 2 names), on raw device
    pointers, with canaries around y."""
    rng = np.random.default_rng(9)
    x = rng.standard_normal(k, dtype=np.float32)
    w_nk = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)
    if bf16:
        w_nk = oracle.round_bf16(w_nk)
    w_kn = np.ascontiguousarray(w_nk.T)
    xt = L.Tensor.from_array_no_grad(x)
    wt = L.Tensor.from_bf16(w_kn) if bf16 else L.Tensor.from_array_no_grad(w_kn)
    pad = 64
    ybuf = L.Tensor.from_array_no_grad(np.full(n + 2 * pad, 12345.0, np.float32))
    L.gemv(ctx, xt.data_ptr, wt.data_ptr, L.BF16 if bf16 else L.F32, True, k, n, ybuf.data_ptr + 4 * pad)
    y = ybuf.data()
    assert np.all(y[:pad] == 12345.0) and np.all(y[-pad:] == 12345.0)
    assert rel_err(y[pad:-pad], oracle.matmul(x[None], w_nk, "f64")[0]) < 2e-6
    # and the [N,K] layout through the same entry point
    wt2 = L.Tensor.from_bf16(w_nk) if bf16 else L.Tensor.from_array_no_grad(w_nk)
    L.gemv(ctx, xt.data_ptr, wt2.data_ptr, L.BF16 if bf16 else L.F32, False, k, n, ybuf.data_ptr + 4 * pad)
    y = ybuf.data()
    assert np.all(y[:pad] == 12345.0) and np.all(y[-pad:] == 12345.0)
    assert rel_err(y[pad:-pad], oracle.matmul(x[None], w_nk, "f64")[0]) < 2e-6


def test_linear_with_bias(L, oracle):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((2, 4, 24), dtype=np.float32)
    w = rng.standard_normal((10, 24), dtype=np.float32)
    b = rng.standard_normal(10, dtype=np.float32)
    lin = L.Linear(L.Tensor.from_array_no_grad(w), L.Tensor.from_array_no_grad(b))
    got = lin.forward(L.Tensor.from_array_no_grad(x)).data()
    assert rel_err(got, oracle.matmul(x, w, "f64") + b) < 2e-6


@pytest.mark.parametrize("rows,dim", [(1, 2048), (3, 50), (5, 4096), (2, 1), (1, 12288)])
def test_rmsnorm(L, oracle, rows, dim):
    rng = np.random.default_rng(dim)
    x = rng.standard_normal((rows, dim), dtype=np.float32)
    w = (1 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
    got = L.RMSNorm(dim, 1e-5, weight=L.Tensor.from_array_no_grad(w)).forward(L.Tensor.from_array_no_grad(x)).data()
    assert rel_err(got, oracle.rmsnorm(x, w, 1e-5, "f64")) < 1e-6
    # the f32 oracle's sequential sum of squares is the less accurate side for long rows
    assert rel_err(got, oracle.rmsnorm(x, w, 1e-5, "f32")) < 5e-6


def test_elementwise_bit_exact(L, oracle):
    rng = np.random.default_rng(1)
    a = rng.standard_normal((3, 7, 33), dtype=np.float32)
    b = rng.standard_normal((3, 7, 33), dtype=np.float32)
    ta, tb = L.Tensor.from_array_no_grad(a), L.Tensor.from_array_no_grad(b)
    assert np.array_equal((ta + tb).data(), oracle.add(a, b))
    assert np.array_equal((ta * tb).data(), oracle.mul(a, b))
    # SiLU: expf differs in the last ulp between glibc and CUDA
    assert rel_err(L.SiLU().forward(ta).data(), oracle.silu(a)) < 5e-7
    # reshape is a view (shape.rs:9-49)
    r = ta.reshape([-1, 33])
    assert r.shape == (21, 33) and r.data_ptr == ta.data_ptr
    assert np.array_equal(r.data(), a.reshape(21, 33))
    with pytest.raises(L.LumenError):
        ta.reshape([5, 5])
    # empty tensors are legal
    e = L.Tensor.from_array_no_grad(np.zeros((0, 4), np.float32))
    assert (e + e).data().shape == (0, 4)


def test_embedding(L, oracle):
    rng = np.random.default_rng(8)
    table = rng.standard_normal((50, 24), dtype=np.float32)
    ids = np.array([[0, 49, 7], [3, 3, 12]], np.float32)
    emb = L.Embedding(L.Tensor.from_array_no_grad(table))
    got = emb.forward(L.Tensor.from_array_no_grad(ids)).data()
    assert np.array_equal(got, oracle.embedding(ids, table))
    # `as usize` saturation: negative and NaN ids read row 0 (embedding.rs:50)
    odd = np.array([[-3.0, np.nan, 4.9]], np.float32)
    assert np.array_equal(emb.forward(L.Tensor.from_array_no_grad(odd)).data(), oracle.embedding(odd, table))
    with pytest.raises(L.LumenError) as e:  # id >= vocab panics (embedding.rs:55)
        emb.forward(L.Tensor.from_array_no_grad(np.array([[50.0]], np.float32)))
    assert e.value.code == L._lib.ERR_EMBED_RANGE
    # the context stays usable after the error
    assert np.array_equal(emb.forward(L.Tensor.from_array_no_grad(ids)).data(), oracle.embedding(ids, table))
    # bf16 table
    tb = oracle.round_bf16(table)
    got = L.Embedding(L.Tensor.from_bf16(table)).forward(L.Tensor.from_array_no_grad(ids)).data()
    assert np.array_equal(got, oracle.embedding(ids, tb))


@pytest.mark.parametrize("d,theta", [(16, 1e4), (64, 1e4), (128, 1e6)])
def test_rope_forward_bit_exact(L, oracle, d, theta):
    rng = np.random.default_rng(d)
    x = rng.standard_normal((2, 3, 5, d), dtype=np.float32)
    rope = L.RotaryEmbedding(d, 40, theta)
    got = rope.forward(L.Tensor.from_array_no_grad(x), 7).data()
    # tables come from the same host libm recipe and the rotation uses unfused f32 mul/add/sub
    assert np.array_equal(got, oracle.rope_forward(x, 7, 40, theta))
    with pytest.raises(L.LumenError) as e:  # offset + len > max (encoding.rs:62-68)
        rope.forward(L.Tensor.from_array_no_grad(x), 36)
    assert e.value.code == L._lib.ERR_ROPE_RANGE
    rope.forward(L.Tensor.from_array_no_grad(x), 35)  # exactly fills the table


@pytest.mark.parametrize("shape", [(2, 2, 4, 6), (1, 3, 1, 9), (1, 1, 5, 700)])
@pytest.mark.parametrize("causal", [False, True])
def test_fused_softmax(L, oracle, shape, causal):
    x = np.random.default_rng(4).standard_normal(shape).astype(np.float32) * 3
    got = L.fused_softmax(L.Tensor.from_array_no_grad(x), 0.3, causal).data()
    want = oracle.fused_softmax(x, 0.3, causal, "f64")
    assert np.abs(got - want).max() < 1e-6
    if causal and shape[2] > 1:
        assert np.all(got[..., 0, 1:] == 0)


def test_llama_kv_cache_interface(L, oracle):
    """LlamaKVCache::{new, update, get_view} (kv_cache.rs:14-59)."""
    cfg = L.LlamaConfig(hidden_size=64, num_attention_heads=4, num_key_value_heads=2, max_seq_len=8)
    c = L.LlamaKVCache(cfg)
    assert (c.head_num, c.max_seq_len, c.dim) == (2, 8, 16)
    ref = oracle.LlamaKVCache(2, 8, 16)
    rng = np.random.default_rng(0)
    k = rng.standard_normal((1, 2, 3, 16), dtype=np.float32)
    v = rng.standard_normal((1, 2, 3, 16), dtype=np.float32)
    c.update(L.Tensor.from_array_no_grad(k), L.Tensor.from_array_no_grad(v), 2)
    ref.update(k, v, 2)
    gk, gv = c.get_view(6)
    rk, rv = ref.get_view(6)
    assert gk.shape == (1, 2, 6, 16)
    assert np.array_equal(gk.data(), rk) and np.array_equal(gv.data(), rv)
    with pytest.raises(L.LumenError) as e:  # overflow panics (kv_cache.rs:34-36)
        c.update(L.Tensor.from_array_no_grad(k), L.Tensor.from_array_no_grad(v), 6)
    assert e.value.code == L._lib.ERR_KV_OVERFLOW
    c.update(L.Tensor.from_array_no_grad(k), L.Tensor.from_array_no_grad(v), 5)  # exactly to the end


def test_tensor_roundtrip_and_set_raw_data(L):
    a = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    t = L.Tensor.from_array_no_grad(a)
    assert t.shape == (2, 3, 4)
    shape, raw = t.get_raw_data()
    assert shape == [2, 3, 4] and np.array_equal(raw, a.reshape(-1))
    t.set_raw_data([2, 3, 4], -a)
    assert np.array_equal(t.data(), -a)
