//! Layers of the decode path (reference: src/layers/basic/linear.rs:7-41, src/layers/basic/embedding.rs:9-57,
//! src/layers/norm/rms_norm.rs:8-62, src/layers/activation.rs:139-147, src/layers/attention/encoding.rs:6-123,
//! src/layers/attention/self_attention.rs:24-127).  Parameters start as zeros (ones for norm gains): the reference's
//! random initialisers are not reproduced, weights come from a loader through `set_raw_data` / `named_parameters`.
use crate::autograd::{require_no_grad, Tensor};
use crate::context::{check, ctx};
use crate::ffi;
use crate::module::Module;
use ndarray::{ArrayD, IxDyn};
use std::cell::RefCell;
use std::rc::Rc;

fn zeros(shape: &[usize]) -> Tensor {
    Tensor::from_array_no_grad(ArrayD::zeros(IxDyn(shape)))
}

/// linear.rs:7-41: weight `[out_features, in_features]`, optional bias `[out_features]`.
pub struct Linear {
    pub weight: Tensor,
    pub bias: Option<Tensor>,
}

impl Linear {
    pub fn new(in_features: usize, out_features: usize) -> Self {
        Linear { weight: zeros(&[out_features, in_features]), bias: Some(zeros(&[out_features])) }
    }

    pub fn new_no_bias(in_features: usize, out_features: usize) -> Self {
        Linear { weight: zeros(&[out_features, in_features]), bias: None }
    }
}

impl Module for Linear {
    fn forward(&self, input: Tensor) -> Tensor {
        require_no_grad("Linear::forward");
        let mut out = std::ptr::null_mut();
        let bias = self.bias.as_ref().map_or(std::ptr::null(), |b| b.raw() as *const _);
        check(unsafe { ffi::lumen_linear_forward(ctx(), input.raw(), self.weight.raw(), bias, &mut out) });
        Tensor::from_raw(out)
    }

    fn parameters(&self) -> Vec<Tensor> {
        let mut p = vec![self.weight.clone()];
        if let Some(b) = &self.bias {
            p.push(b.clone());
        }
        p
    }
}

/// embedding.rs:9-57: token ids are f32, an id >= vocab_size panics.
pub struct Embedding {
    pub weight: Tensor,
    pub vocab_size: usize,
    pub embed_dim: usize,
}

impl Embedding {
    pub fn new(vocab_size: usize, embed_dim: usize) -> Self {
        Embedding { weight: zeros(&[vocab_size, embed_dim]), vocab_size, embed_dim }
    }

    pub fn forward(&self, indices: &Tensor) -> Tensor {
        require_no_grad("Embedding::forward");
        let mut out = std::ptr::null_mut();
        check(unsafe { ffi::lumen_embedding(ctx(), indices.raw(), self.weight.raw(), &mut out) });
        // the range check runs on the device: surface it here, where the reference panics
        check(unsafe { ffi::lumen_ctx_synchronize(ctx()) });
        Tensor::from_raw(out)
    }
}

impl Module for Embedding {
    fn forward(&self, input: Tensor) -> Tensor {
        Embedding::forward(self, &input)
    }

    fn parameters(&self) -> Vec<Tensor> {
        vec![self.weight.clone()]
    }
}

/// rms_norm.rs:8-62
pub struct RMSNorm {
    pub weight: Tensor,
    pub eps: f32,
}

impl RMSNorm {
    pub fn new(dim: usize, eps: f32) -> Self {
        RMSNorm { weight: Tensor::from_array_no_grad(ArrayD::ones(IxDyn(&[dim]))), eps }
    }
}

impl Module for RMSNorm {
    fn forward(&self, input: Tensor) -> Tensor {
        require_no_grad("RMSNorm::forward");
        let mut out = std::ptr::null_mut();
        check(unsafe { ffi::lumen_rmsnorm(ctx(), input.raw(), self.weight.raw(), self.eps, &mut out) });
        Tensor::from_raw(out)
    }

    fn parameters(&self) -> Vec<Tensor> {
        vec![self.weight.clone()]
    }
}

/// activation.rs:139-147
pub struct SiLU;

impl SiLU {
    pub fn new() -> Self {
        SiLU
    }
}

impl Module for SiLU {
    fn forward(&self, input: Tensor) -> Tensor {
        require_no_grad("SiLU::forward");
        let mut out = std::ptr::null_mut();
        check(unsafe { ffi::lumen_silu(ctx(), input.raw(), &mut out) });
        Tensor::from_raw(out)
    }

    fn parameters(&self) -> Vec<Tensor> {
        Vec::new()
    }
}

/// encoding.rs:6-123: cos/sin tables for positions 0..max_seq_len, half-split rotation.
pub struct RotaryEmbedding {
    handle: *mut ffi::lumen_rope,
    pub dim: usize,
    pub max_seq_len: usize,
}

impl RotaryEmbedding {
    pub fn new(dim: usize, max_seq_len: usize, theta: f32) -> Self {
        let mut handle = std::ptr::null_mut();
        check(unsafe { ffi::lumen_rope_new(ctx(), dim, max_seq_len, theta, &mut handle) });
        RotaryEmbedding { handle, dim, max_seq_len }
    }

    /// x `[B, H, S, D]` rotated at positions `offset..offset + S`; out of range panics (encoding.rs:62-68).
    pub fn forward(&self, x: &Tensor, offset: usize) -> Tensor {
        let mut out = std::ptr::null_mut();
        check(unsafe { ffi::lumen_rope_forward(self.handle, x.raw(), offset, &mut out) });
        Tensor::from_raw(out)
    }

    pub(crate) fn raw(&self) -> *mut ffi::lumen_rope {
        self.handle
    }
}

impl Drop for RotaryEmbedding {
    fn drop(&mut self) {
        unsafe { ffi::lumen_rope_free(self.handle) };
    }
}

/// self_attention.rs:24-44: `k`, `v` `[B, H_kv, max_seq, D]` zero-initialised, `len`; `reset` keeps the contents.
pub struct KVCacheInner {
    pub(crate) handle: *mut ffi::lumen_kv_cache,
    pub shape: [usize; 4],
}

impl KVCacheInner {
    pub fn new(b: usize, h_kv: usize, max_seq: usize, d: usize) -> Self {
        let mut handle = std::ptr::null_mut();
        check(unsafe { ffi::lumen_kv_new(ctx(), b, h_kv, max_seq, d, &mut handle) });
        KVCacheInner { handle, shape: [b, h_kv, max_seq, d] }
    }

    pub(crate) fn from_raw(handle: *mut ffi::lumen_kv_cache, shape: [usize; 4]) -> Self {
        KVCacheInner { handle, shape }
    }

    pub fn reset(&mut self) {
        check(unsafe { ffi::lumen_kv_reset(self.handle) });
    }

    /// The reference's public field `len`.
    pub fn len(&self) -> usize {
        unsafe { ffi::lumen_kv_len(self.handle) }
    }

    /// Host copies of the reference's public fields `k` and `v`.
    pub fn read(&self) -> (Vec<f32>, Vec<f32>) {
        let n: usize = self.shape.iter().product();
        let (mut k, mut v) = (vec![0f32; n], vec![0f32; n]);
        check(unsafe { ffi::lumen_kv_read(self.handle, k.as_mut_ptr(), v.as_mut_ptr()) });
        (k, v)
    }

    pub fn write(&mut self, k: &[f32], v: &[f32], len: usize) {
        let n: usize = self.shape.iter().product();
        assert!(k.len() == n && v.len() == n, "KVCacheInner::write: slab size mismatch");
        check(unsafe { ffi::lumen_kv_write(self.handle, k.as_ptr(), v.as_ptr(), len) });
    }
}

impl Drop for KVCacheInner {
    fn drop(&mut self) {
        unsafe { ffi::lumen_kv_free(self.handle) };
    }
}

/// self_attention.rs:30
pub type KVCache = Rc<RefCell<KVCacheInner>>;

/// self_attention.rs:46-127: four bias-free projections, RoPE, grouped-query attention over the static cache.
pub struct SelfAttention {
    handle: *mut ffi::lumen_self_attention,
    pub w_q: Linear,
    pub w_k: Linear,
    pub w_v: Linear,
    pub w_o: Linear,
    pub n_head: usize,
    pub n_kv_head: usize,
    pub head_dim: usize,
    pub causal: bool,
    pub max_seq: usize,
}

impl SelfAttention {
    pub fn new(embed_dim: usize, n_head: usize, n_kv_head: usize, max_seq_len: usize, rope_theta: f32, causal: bool) -> Self {
        assert_eq!(embed_dim % n_head, 0, "Embed dim must be divisible by n_head");
        let head_dim = embed_dim / n_head;
        let kv_dim = n_kv_head * head_dim;
        let mut handle = std::ptr::null_mut();
        check(unsafe {
            ffi::lumen_self_attention_new(ctx(), embed_dim, n_head, n_kv_head, max_seq_len, rope_theta, causal as i32, &mut handle)
        });
        let s = SelfAttention {
            handle,
            w_q: Linear::new_no_bias(embed_dim, embed_dim),
            w_k: Linear::new_no_bias(embed_dim, kv_dim),
            w_v: Linear::new_no_bias(embed_dim, kv_dim),
            w_o: Linear::new_no_bias(embed_dim, embed_dim),
            n_head,
            n_kv_head,
            head_dim,
            causal,
            max_seq: max_seq_len,
        };
        s.bind_weights();
        s
    }

    /// Hands the four weight tensors to the library (they are shared, not copied: later `set_raw_data` calls on
    /// `w_q.weight` etc. are seen by `forward`).
    pub fn bind_weights(&self) {
        for (which, lin) in [(ffi::LUMEN_W_Q, &self.w_q), (ffi::LUMEN_W_K, &self.w_k), (ffi::LUMEN_W_V, &self.w_v), (ffi::LUMEN_W_O, &self.w_o)] {
            check(unsafe { ffi::lumen_self_attention_set_weight(self.handle, which, lin.weight.raw()) });
        }
    }

    /// self_attention.rs:96-127: `S == 1` with a cache is the decode step, `S > 1` the prefill; a cache is created when
    /// `None` is passed.
    pub fn forward(&self, x: Tensor, cache: Option<KVCache>) -> (Tensor, Option<KVCache>) {
        require_no_grad("SelfAttention::forward");
        let mut out = std::ptr::null_mut();
        let mut cache_out = std::ptr::null_mut();
        let cache_in = cache.as_ref().map_or(std::ptr::null_mut(), |c| c.borrow().handle);
        check(unsafe { ffi::lumen_self_attention_forward(self.handle, x.raw(), cache_in, &mut out, &mut cache_out) });
        let cache = match cache {
            Some(c) => c,
            None => {
                let b = x.shape()[0];
                Rc::new(RefCell::new(KVCacheInner::from_raw(cache_out, [b, self.n_kv_head, self.max_seq, self.head_dim])))
            }
        };
        (Tensor::from_raw(out), Some(cache))
    }
}

impl Module for SelfAttention {
    fn forward(&self, input: Tensor) -> Tensor {
        SelfAttention::forward(self, input, None).0
    }

    fn parameters(&self) -> Vec<Tensor> {
        vec![self.w_q.weight.clone(), self.w_k.weight.clone(), self.w_v.weight.clone(), self.w_o.weight.clone()]
    }
}

impl Drop for SelfAttention {
    fn drop(&mut self) {
        unsafe { ffi::lumen_self_attention_free(self.handle) };
    }
}
