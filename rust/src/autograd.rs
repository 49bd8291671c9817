//! `Tensor` and the no-grad switches (reference: src/autograd.rs:9-51, :63-64, :82-112, :150-187, :251-269).
//! A `Tensor` is a shared handle to a device buffer owned by the library; the data surface of the reference's
//! type is kept, the gradient surface is not (inference only).
use crate::context::{check, ctx};
use crate::ffi;
use ndarray::{ArrayD, IxDyn};
use std::cell::Cell;
use std::rc::Rc;

thread_local! {
    static NO_GRAD_DEPTH: Cell<usize> = Cell::new(0);
    static INFERENCE_MODE: Cell<bool> = Cell::new(false);
}

/// autograd.rs:12-27
pub struct NoGradGuard {
    _private: (),
}

impl NoGradGuard {
    pub fn enter() -> Self {
        NO_GRAD_DEPTH.with(|d| d.set(d.get() + 1));
        NoGradGuard { _private: () }
    }
}

impl Drop for NoGradGuard {
    fn drop(&mut self) {
        NO_GRAD_DEPTH.with(|d| d.set(d.get().saturating_sub(1)));
    }
}

/// autograd.rs:30-32
pub fn set_inference_mode(on: bool) {
    INFERENCE_MODE.with(|m| m.set(on));
}

/// autograd.rs:35-37
pub fn is_inference_mode() -> bool {
    INFERENCE_MODE.with(|m| m.get())
}

/// autograd.rs:43-45
pub fn is_no_grad() -> bool {
    is_inference_mode() || NO_GRAD_DEPTH.with(|d| d.get() > 0)
}

/// autograd.rs:48-51
pub fn no_grad<R>(f: impl FnOnce() -> R) -> R {
    let _guard = NoGradGuard::enter();
    f()
}

pub(crate) fn require_no_grad(what: &str) {
    if !is_no_grad() {
        panic!("{}: only the inference branches exist on this backend; call it inside no_grad", what);
    }
}

pub(crate) struct TensorHandle(pub *mut ffi::lumen_tensor);

impl Drop for TensorHandle {
    fn drop(&mut self) {
        unsafe { ffi::lumen_tensor_free(self.0) };
    }
}

/// autograd.rs:63-64: a cheaply clonable handle (`Rc`), `!Send` like the reference's.
#[derive(Clone)]
pub struct Tensor(pub(crate) Rc<TensorHandle>);

impl Tensor {
    pub(crate) fn from_raw(h: *mut ffi::lumen_tensor) -> Tensor {
        Tensor(Rc::new(TensorHandle(h)))
    }

    pub(crate) fn raw(&self) -> *mut ffi::lumen_tensor {
        (self.0).0
    }

    /// autograd.rs:70-80 (`new`) and :144-148 (`from_data`): on this backend every tensor is a constant.
    pub fn new(data: ArrayD<f32>) -> Self {
        Tensor::from_array_no_grad(data)
    }

    pub fn from_data(data: ArrayD<f32>) -> Tensor {
        Tensor::from_array_no_grad(data)
    }

    /// autograd.rs:161-163
    pub fn from_array_no_grad(data: ArrayD<f32>) -> Tensor {
        let data = data.as_standard_layout().into_owned();
        let shape: Vec<usize> = data.shape().to_vec();
        let mut out = std::ptr::null_mut();
        check(unsafe {
            ffi::lumen_tensor_from_host(ctx(), data.as_ptr(), shape.as_ptr(), shape.len() as i32, &mut out)
        });
        Tensor::from_raw(out)
    }

    /// autograd.rs:166-169: parameters are plain tensors here (no gradient is ever attached).
    pub fn parameter(data: ArrayD<f32>) -> Tensor {
        Tensor::from_array_no_grad(data)
    }

    /// bf16 weights (`src/loader.rs:50-64` widens them; here the bits go to the device as they are).
    pub fn from_bf16_bits(bits: &[u16], shape: &[usize]) -> Tensor {
        let mut out = std::ptr::null_mut();
        check(unsafe {
            ffi::lumen_tensor_from_host_bf16(ctx(), bits.as_ptr(), shape.as_ptr(), shape.len() as i32, &mut out)
        });
        Tensor::from_raw(out)
    }

    pub fn shape(&self) -> Vec<usize> {
        let n = unsafe { ffi::lumen_tensor_ndim(self.raw()) } as usize;
        let mut s = vec![0usize; n];
        check(unsafe { ffi::lumen_tensor_shape(self.raw(), s.as_mut_ptr()) });
        s
    }

    /// autograd.rs:105-108: an owned host copy (synchronises the stream).
    pub fn data(&self) -> ArrayD<f32> {
        let (shape, raw) = self.get_raw_data();
        ArrayD::from_shape_vec(IxDyn(&shape), raw).expect("shape and data length agree")
    }

    pub fn requires_grad(&self) -> bool {
        false
    }

    /// autograd.rs:179-181: `-1` infers one dimension; shares the storage.
    pub fn reshape(&self, shape: Vec<i32>) -> Tensor {
        let s: Vec<i64> = shape.iter().map(|&v| v as i64).collect();
        let mut out = std::ptr::null_mut();
        check(unsafe { ffi::lumen_tensor_reshape(self.raw(), s.as_ptr(), s.len() as i32, &mut out) });
        Tensor::from_raw(out)
    }

    /// autograd.rs:251-257
    pub fn get_raw_data(&self) -> (Vec<usize>, Vec<f32>) {
        let shape = self.shape();
        let n = unsafe { ffi::lumen_tensor_numel(self.raw()) };
        let mut raw = vec![0f32; n];
        check(unsafe { ffi::lumen_tensor_to_host(self.raw(), raw.as_mut_ptr()) });
        (shape, raw)
    }

    /// autograd.rs:259-263: the shape must match the tensor's (the device buffer is not reallocated).
    pub fn set_raw_data(&self, shape: Vec<usize>, raw_data: Vec<f32>) {
        assert_eq!(shape, self.shape(), "set_raw_data: shape mismatch");
        assert_eq!(raw_data.len(), shape.iter().product::<usize>(), "set_raw_data: length mismatch");
        check(unsafe { ffi::lumen_tensor_set(self.raw(), raw_data.as_ptr()) });
    }

    /// autograd.rs:265-269: nothing to detach from; returns the same storage.
    pub fn detach(&self) -> Tensor {
        self.clone()
    }
}

/// autograd.rs:272-274
pub fn detach(t: &Tensor) -> Tensor {
    t.detach()
}
