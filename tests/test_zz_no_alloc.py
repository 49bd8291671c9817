"""`lumen_gemv_kn_static`: the [K,N] vector-matrix product whose split-K partial sums live in a fixed device
array of the library.  Collected last (file name) so that it also runs after every other GPU test has used
the device; it passes alone as well.  Calls go through the C ABI on raw device pointers."""
import numpy as np
import pytest

from helpers import rel_err

pytestmark = pytest.mark.gpu


def _run_both(L, ctx, oracle, k, n, bf16, seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal(k, dtype=np.float32)
    w_nk = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)
    if bf16:
        w_nk = oracle.round_bf16(w_nk)
    w_kn = np.ascontiguousarray(w_nk.T)
    xt = L.Tensor.from_array_no_grad(x)
    wt = L.Tensor.from_bf16(w_kn) if bf16 else L.Tensor.from_array_no_grad(w_kn)
    dt = L.BF16 if bf16 else L.F32
    pad = 64
    y_ref = L.Tensor.from_array_no_grad(np.full(n + 2 * pad, 777.0, np.float32))
    y_new = L.Tensor.from_array_no_grad(np.full(n + 2 * pad, 777.0, np.float32))
    L.gemv(ctx, xt.data_ptr, wt.data_ptr, dt, True, k, n, y_ref.data_ptr + 4 * pad)
    L.gemv_kn_static(ctx, xt.data_ptr, wt.data_ptr, dt, k, n, y_new.data_ptr + 4 * pad)
    a, b = y_ref.data(), y_new.data()
    assert np.all(b[:pad] == 777.0) and np.all(b[-pad:] == 777.0)  # nothing written outside y
    assert np.array_equal(a, b), (k, n, bf16)  # same kernels, same split plan: bit-identical
    assert rel_err(b[pad:-pad], oracle.matmul(x[None], w_nk, "f64")[0]) < 2e-6


@pytest.mark.parametrize("bf16", [False, True])
def test_two_calls_in_a_row_equal_the_allocating_entry_point(L, ctx, oracle, bf16):
    # back to back, with different split counts, so the second call finds the first one's partial sums
    # in the array; then the first shape once more
    _run_both(L, ctx, oracle, 5632, 2048, bf16, 1)
    _run_both(L, ctx, oracle, 100, 37, bf16, 2)
    _run_both(L, ctx, oracle, 5632, 2048, bf16, 3)
    _run_both(L, ctx, oracle, 2048, 32000, bf16, 4)


def test_sizes_beyond_the_fixed_array_are_refused(L, ctx):
    # 64 x 1200000 f32 wants 2 slices x 1200000 floats = 9.6 MB of partial sums: more than the 8 MiB array.
    # The refusal happens on the host before anything is launched, so small stand-in buffers are enough.
    t = L.Tensor.from_array_no_grad(np.zeros(16, np.float32))
    launches = ctx.launch_count
    with pytest.raises(L.LumenError) as e:
        L.gemv_kn_static(ctx, t.data_ptr, t.data_ptr, L.F32, 64, 1200000, t.data_ptr)
    assert e.value.code == L._lib.ERR_UNSUPPORTED
    assert "8388608" in str(e.value)
    assert ctx.launch_count == launches
    # an empty product is a no-op, like lumen_gemv
    L.gemv_kn_static(ctx, t.data_ptr, t.data_ptr, L.F32, 0, 5, t.data_ptr)
    assert ctx.launch_count == launches
