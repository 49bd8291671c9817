"""Context, Tensor and the no-grad switches — host-side mirror of src/autograd.rs (data surface only).

The reference's `Tensor` is `Rc<RefCell<TensorData>>` over an ndarray; here it is a handle to a
device buffer owned by the C library.  Only the inference surface exists: constructors
(`from_array_no_grad`, autograd.rs:150-163), `shape` / `data` (autograd.rs:82-112), `get_raw_data` /
`set_raw_data` (autograd.rs:251-262) and the global no-grad state that selects the inference
branches (autograd.rs:9-51).  Gradients and `backward` are training and are not provided.
"""
from __future__ import annotations

import contextlib
import ctypes as C
import weakref

import numpy as np

from . import _lib
from ._lib import BF16, F32, check
from .synth import bf16_bits_to_f32, f32_to_bf16_bits  # noqa: F401  (numpy-only helpers, re-exported here)

_NO_GRAD_DEPTH = 0
_INFERENCE_MODE = False


def set_inference_mode(on: bool) -> None:
    """autograd.rs:29-31."""
    global _INFERENCE_MODE
    _INFERENCE_MODE = bool(on)


def is_inference_mode() -> bool:
    return _INFERENCE_MODE


def is_no_grad() -> bool:
    """autograd.rs:43-45: inside a no_grad scope, or inference mode is on."""
    return _NO_GRAD_DEPTH > 0 or _INFERENCE_MODE


@contextlib.contextmanager
def no_grad():
    """autograd.rs:48-51 (`no_grad(|| ...)`) as a context manager."""
    global _NO_GRAD_DEPTH
    _NO_GRAD_DEPTH += 1
    try:
        yield
    finally:
        _NO_GRAD_DEPTH -= 1


def require_no_grad(what: str) -> None:
    if not is_no_grad():
        raise NotImplementedError(
            f"{what}: only the inference (no_grad / eval_mode) path is implemented on the GPU; "
            "the reference's training path (autograd graph, backward) is out of scope")


class Context:
    """One GPU (or one tensor-parallel rank) with its stream.  No counterpart in the reference."""

    def __init__(self, device: int = 0, tp_rank: int = 0, tp_size: int = 1, nccl_id: bytes | None = None):
        self._lib = _lib.load()
        self.h = C.c_void_p()
        idbuf = C.create_string_buffer(nccl_id, _lib.NCCL_ID_BYTES) if nccl_id is not None else None
        check(self._lib.lumen_ctx_create(device, tp_rank, tp_size, idbuf, C.byref(self.h)))
        self.device, self.tp_rank, self.tp_size = device, tp_rank, tp_size
        self._finalizer = weakref.finalize(self, self._lib.lumen_ctx_destroy, C.c_void_p(self.h.value))

    @staticmethod
    def nccl_unique_id() -> bytes:
        buf = C.create_string_buffer(_lib.NCCL_ID_BYTES)
        check(_lib.load().lumen_nccl_unique_id(buf))
        return buf.raw

    def synchronize(self) -> None:
        check(self._lib.lumen_ctx_synchronize(self.h), self.h)

    @property
    def stream(self) -> int:
        """Raw cudaStream_t of this context (for CUDA-event timing on the launching stream)."""
        return int(self._lib.lumen_ctx_stream(self.h) or 0)

    @property
    def launch_count(self) -> int:
        """Kernels this context has enqueued so far (graph replays count their kernel nodes)."""
        return int(self._lib.lumen_ctx_launch_count(self.h))

    def check(self, status: int) -> None:
        check(status, self.h)


_default_ctx: Context | None = None


def default_context() -> Context:
    global _default_ctx
    if _default_ctx is None:
        _default_ctx = Context(0)
    return _default_ctx


def _shape_arr(shape):
    return (C.c_size_t * len(shape))(*shape)


class Tensor:
    """Device tensor handle (f32 activations, f32 or bf16 weights)."""

    def __init__(self, handle: C.c_void_p, ctx: Context):
        self.h, self.ctx = handle, ctx
        self._finalizer = weakref.finalize(self, ctx._lib.lumen_tensor_free, C.c_void_p(handle.value))

    # ---- constructors -----------------------------------------------------------------------------
    @classmethod
    def from_array_no_grad(cls, data, ctx: Context | None = None) -> "Tensor":
        """Tensor::from_array_no_grad (autograd.rs:161-163): an f32 constant."""
        ctx = ctx or default_context()
        a = np.ascontiguousarray(data, dtype=np.float32)
        h = C.c_void_p()
        ctx.check(ctx._lib.lumen_tensor_from_host(ctx.h, a.ctypes.data, _shape_arr(a.shape), a.ndim, C.byref(h)))
        return cls(h, ctx)

    from_data_no_grad = from_array_no_grad
    new = from_array_no_grad
    parameter = from_array_no_grad  # Tensor::parameter (autograd.rs:166); gradients are not tracked here

    @classmethod
    def from_bf16(cls, data_f32, ctx: Context | None = None) -> "Tensor":
        """A weight stored as bf16 on the device (rounded to nearest even from f32)."""
        ctx = ctx or default_context()
        bits = f32_to_bf16_bits(np.asarray(data_f32, dtype=np.float32))
        h = C.c_void_p()
        ctx.check(ctx._lib.lumen_tensor_from_host_bf16(ctx.h, bits.ctypes.data, _shape_arr(bits.shape), bits.ndim, C.byref(h)))
        return cls(h, ctx)

    # ---- accessors --------------------------------------------------------------------------------
    @property
    def shape(self) -> tuple:
        n = self.ctx._lib.lumen_tensor_ndim(self.h)
        out = (C.c_size_t * max(n, 1))()
        self.ctx.check(self.ctx._lib.lumen_tensor_shape(self.h, out))
        return tuple(out[i] for i in range(n))

    @property
    def dtype(self) -> int:
        return int(self.ctx._lib.lumen_tensor_dtype(self.h))

    @property
    def data_ptr(self) -> int:
        return int(self.ctx._lib.lumen_tensor_data(self.h) or 0)

    def data(self) -> np.ndarray:
        """Tensor::data() (autograd.rs:106-108): an owned host copy (bf16 is widened to f32)."""
        out = np.empty(self.shape, dtype=np.float32)
        self.ctx.check(self.ctx._lib.lumen_tensor_to_host(self.h, out.ctypes.data))
        return out

    numpy = data

    def get_raw_data(self):
        d = self.data()
        return list(d.shape), d.reshape(-1)

    def set_raw_data(self, shape, raw_data) -> None:
        a = np.ascontiguousarray(raw_data, dtype=np.float32)
        if tuple(shape) != self.shape:
            raise _lib.LumenError(_lib.ERR_SHAPE, "set_raw_data keeps the tensor's shape on the device")
        self.ctx.check(self.ctx._lib.lumen_tensor_set(self.h, a.ctypes.data))

    def requires_grad(self) -> bool:
        return False

    def reshape(self, shape) -> "Tensor":
        """ops::shape::reshape (src/ops/shape.rs:9-49) as a zero-copy view."""
        arr = (C.c_int64 * len(shape))(*[int(s) for s in shape])
        h = C.c_void_p()
        self.ctx.check(self.ctx._lib.lumen_tensor_reshape(self.h, arr, len(shape), C.byref(h)))
        return Tensor(h, self.ctx)

    # ---- operators (src/ops/arithmetic.rs:48-52, :105-109) -------------------------------------------
    def _binary(self, other: "Tensor", fn) -> "Tensor":
        h = C.c_void_p()
        self.ctx.check(fn(self.ctx.h, self.h, other.h, C.byref(h)))
        return Tensor(h, self.ctx)

    def __add__(self, other: "Tensor") -> "Tensor":
        return self._binary(other, self.ctx._lib.lumen_add)

    def __mul__(self, other: "Tensor") -> "Tensor":
        return self._binary(other, self.ctx._lib.lumen_mul)
