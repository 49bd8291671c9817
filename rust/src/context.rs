//! The process-wide library context (device, stream, error text).  The reference has no such object: its tensors
//! live in host memory.  One context per thread, created on first use on CUDA device `LUMEN_DEVICE` (default 0).
use crate::ffi;
use std::cell::Cell;
use std::ffi::CStr;

thread_local! {
    static CTX: Cell<*mut ffi::lumen_ctx> = Cell::new(std::ptr::null_mut());
}

/// The calling thread's context (created on first use; panics when no B200 is visible: there is no CPU path).
pub fn ctx() -> *mut ffi::lumen_ctx {
    CTX.with(|c| {
        if c.get().is_null() {
            let device: i32 = std::env::var("LUMEN_DEVICE").ok().and_then(|s| s.parse().ok()).unwrap_or(0);
            let mut out = std::ptr::null_mut();
            let rc = unsafe { ffi::lumen_ctx_create(device, 0, 1, std::ptr::null(), &mut out) };
            if rc != ffi::LUMEN_OK {
                panic!("lumen_ctx_create failed: {}", status_text(rc));
            }
            c.set(out);
        }
        c.get()
    })
}

/// Installs a context made by the caller (tensor-parallel ranks create theirs with an NCCL id).
pub fn set_ctx(ctx: *mut ffi::lumen_ctx) {
    CTX.with(|c| c.set(ctx));
}

pub fn status_text(rc: i32) -> String {
    unsafe { CStr::from_ptr(ffi::lumen_status_string(rc)).to_string_lossy().into_owned() }
}

/// Turns a non-zero status into the panic the reference would have raised at the same place.
pub fn check(rc: i32) {
    if rc != ffi::LUMEN_OK {
        let msg = unsafe { CStr::from_ptr(ffi::lumen_last_error(ctx())).to_string_lossy().into_owned() };
        panic!("{}: {}", status_text(rc), msg);
    }
}
