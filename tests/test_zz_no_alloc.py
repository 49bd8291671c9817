"""`lumen_gemv_kn_static`: the [K,N] vector-matrix product whose split-K partial sums live in a fixed device
array of the library.  Collected last (file name) so that it also runs after every other GPU test has used
the device; it passes alone as well.  Calls go through the C ABI on raw device pointers."""
import numpy as np
import pytest

from helpers import rel_err

pytestmark = pytest.mark.gpu


class _AllocProbe:
    """Device-memory bookkeeping around a call, read through the CUDA runtime (ctypes on libcudart): free memory of
    the device (moves when anything calls cudaMalloc / cudaFree) and the high-water mark of the device's default
    memory pool (moves when anything calls cudaMallocAsync, which is what the library's temporaries use)."""

    USED_MEM_HIGH = 8  # cudaMemPoolAttrUsedMemHigh

    def __init__(self):
        import ctypes as C
        import glob
        paths = sorted(glob.glob("/usr/local/cuda/lib64/libcudart.so*")) or ["libcudart.so"]
        self.C, self.rt = C, C.CDLL(paths[-1])
        assert self.rt.cudaSetDevice(0) == 0
        self.pool = C.c_void_p()
        assert self.rt.cudaDeviceGetDefaultMemPool(C.byref(self.pool), 0) == 0

    def _high(self):
        v = self.C.c_uint64()
        assert self.rt.cudaMemPoolGetAttribute(self.pool, self.USED_MEM_HIGH, self.C.byref(v)) == 0
        return int(v.value)

    def _free(self):
        free, total = self.C.c_size_t(), self.C.c_size_t()
        assert self.rt.cudaMemGetInfo(self.C.byref(free), self.C.byref(total)) == 0
        return int(free.value)

    def start(self):
        zero = self.C.c_uint64(0)  # writing 0 resets the high-water mark to the pool's current use
        assert self.rt.cudaMemPoolSetAttribute(self.pool, self.USED_MEM_HIGH, self.C.byref(zero)) == 0
        self.free0, self.high0 = self._free(), self._high()

    def stop(self):
        return self._free() - self.free0, self._high() - self.high0


def _run_both(L, ctx, oracle, k, n, bf16, seed, probe=None):
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
    ctx.synchronize()
    if probe is not None:
        probe.start()
    L.gemv_kn_static(ctx, xt.data_ptr, wt.data_ptr, dt, k, n, y_new.data_ptr + 4 * pad)
    ctx.synchronize()
    if probe is not None:
        # the entry point took nothing from the device or from the stream-ordered pool ...
        assert probe.stop() == (0, 0), (k, n, bf16)
        # ... while the allocating one does draw its partial sums from the pool (the probe sees what it should)
        probe.start()
        L.gemv(ctx, xt.data_ptr, wt.data_ptr, dt, True, k, n, y_ref.data_ptr + 4 * pad)
        ctx.synchronize()
        assert probe.stop()[1] > 0
    a, b = y_ref.data(), y_new.data()
    assert np.all(b[:pad] == 777.0) and np.all(b[-pad:] == 777.0)  # nothing written outside y
    assert np.array_equal(a, b), (k, n, bf16)  # same kernels, same split plan: bit-identical
    assert rel_err(b[pad:-pad], oracle.matmul(x[None], w_nk, "f64")[0]) < 2e-6


@pytest.mark.parametrize("bf16", [False, True])
def test_two_calls_in_a_row_equal_the_allocating_entry_point(L, ctx, oracle, bf16):
    # back to back, with different split counts, so the second call finds the first one's partial sums
    # in the array; then the first shape once more.  From the second pair on (the first call on a device resolves
    # the array's address, which may load the module) the calls are also watched for allocations.
    try:
        probe = _AllocProbe()
    except Exception:  # no CUDA runtime binding for Python in this environment: results are still compared
        probe = None
    _run_both(L, ctx, oracle, 5632, 2048, bf16, 1)
    _run_both(L, ctx, oracle, 100, 37, bf16, 2, probe)
    _run_both(L, ctx, oracle, 5632, 2048, bf16, 3, probe)
    _run_both(L, ctx, oracle, 2048, 32000, bf16, 4, probe)


def test_sizes_beyond_the_fixed_array_are_refused(L, ctx):
    # 64 x 2400000 f32 wants more partial sums than the 8 MiB array holds (the message names both sizes).
    # The refusal happens on the host before anything is launched, so small stand-in buffers are enough.
    t = L.Tensor.from_array_no_grad(np.zeros(16, np.float32))
    launches = ctx.launch_count
    with pytest.raises(L.LumenError) as e:
        L.gemv_kn_static(ctx, t.data_ptr, t.data_ptr, L.F32, 64, 2400000, t.data_ptr)
    assert e.value.code == L._lib.ERR_UNSUPPORTED
    assert "8388608" in str(e.value)
    assert ctx.launch_count == launches
    # an empty product is a no-op, like lumen_gemv
    L.gemv_kn_static(ctx, t.data_ptr, t.data_ptr, L.F32, 0, 5, t.data_ptr)
    assert ctx.launch_count == launches
