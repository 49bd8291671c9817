//! `LlamaKVCache` (reference: src/kv_cache.rs:5-59): `[1, kv_heads, max_seq_len, head_dim]` slabs with `update` and
//! `get_view`.  The reference crate never uses it on its own decode path; it is kept as interface.
use crate::autograd::Tensor;
use crate::context::{check, ctx};
use crate::ffi;
use crate::models::LlamaConfig;

pub struct LlamaKVCache {
    handle: *mut ffi::lumen_llama_kv_cache,
    pub max_seq_len: usize,
    pub dim: usize,
    pub head_num: usize,
}

impl LlamaKVCache {
    /// kv_cache.rs:14-29
    pub fn new(config: &LlamaConfig) -> Self {
        let dim = config.hidden_size / config.num_attention_heads;
        let mut handle = std::ptr::null_mut();
        check(unsafe { ffi::lumen_llama_kv_new(ctx(), config.num_key_value_heads, config.max_seq_len, dim, &mut handle) });
        LlamaKVCache { handle, max_seq_len: config.max_seq_len, dim, head_num: config.num_key_value_heads }
    }

    /// kv_cache.rs:31-49: k, v `[1, H, S, D]` copied into rows `start_pos..start_pos + S`; overflow panics.
    pub fn update(&mut self, k: &Tensor, v: &Tensor, start_pos: usize) {
        check(unsafe { ffi::lumen_llama_kv_update(self.handle, k.raw(), v.raw(), start_pos) });
    }

    /// kv_cache.rs:51-59: owned copies of the first `current_len` rows.
    pub fn get_view(&self, current_len: usize) -> (Tensor, Tensor) {
        let (mut k, mut v) = (std::ptr::null_mut(), std::ptr::null_mut());
        check(unsafe { ffi::lumen_llama_kv_get_view(self.handle, current_len, &mut k, &mut v) });
        (Tensor::from_raw(k), Tensor::from_raw(v))
    }
}

impl Drop for LlamaKVCache {
    fn drop(&mut self) {
        unsafe { ffi::lumen_llama_kv_free(self.handle) };
    }
}
