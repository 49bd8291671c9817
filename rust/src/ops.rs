//! Operators (reference: src/ops/matmul.rs:10-103, src/ops/arithmetic.rs:48-52 and :105-109,
//! src/ops/fused.rs:39-83).
use crate::autograd::{require_no_grad, Tensor};
use crate::context::{check, ctx};
use crate::ffi;

/// `matmul(a, w)`: a[..., K] times w[N, K] transposed; M = 1 takes the vector-matrix kernels (matmul.rs:42-69).
pub fn matmul(a: &Tensor, w: &Tensor) -> Tensor {
    require_no_grad("matmul");
    let mut out = std::ptr::null_mut();
    check(unsafe { ffi::lumen_matmul(ctx(), a.raw(), w.raw(), &mut out) });
    Tensor::from_raw(out)
}

/// fused.rs:39-83 (forward)
pub fn fused_softmax(x: &Tensor, scale: f32, causal: bool) -> Tensor {
    require_no_grad("fused_softmax");
    let mut out = std::ptr::null_mut();
    check(unsafe { ffi::lumen_fused_softmax(ctx(), x.raw(), scale, causal as i32, &mut out) });
    Tensor::from_raw(out)
}

fn binary(a: &Tensor, b: &Tensor, mul: bool) -> Tensor {
    require_no_grad(if mul { "Tensor * Tensor" } else { "Tensor + Tensor" });
    let mut out = std::ptr::null_mut();
    check(unsafe {
        if mul {
            ffi::lumen_mul(ctx(), a.raw(), b.raw(), &mut out)
        } else {
            ffi::lumen_add(ctx(), a.raw(), b.raw(), &mut out)
        }
    });
    Tensor::from_raw(out)
}

impl std::ops::Add for Tensor {
    type Output = Tensor;
    fn add(self, rhs: Tensor) -> Tensor {
        binary(&self, &rhs, false)
    }
}

impl std::ops::Mul for Tensor {
    type Output = Tensor;
    fn mul(self, rhs: Tensor) -> Tensor {
        binary(&self, &rhs, true)
    }
}

impl<'a> std::ops::Add<&'a Tensor> for &'a Tensor {
    type Output = Tensor;
    fn add(self, rhs: &Tensor) -> Tensor {
        binary(self, rhs, false)
    }
}

impl<'a> std::ops::Mul<&'a Tensor> for &'a Tensor {
    type Output = Tensor;
    fn mul(self, rhs: &Tensor) -> Tensor {
        binary(self, rhs, true)
    }
}
