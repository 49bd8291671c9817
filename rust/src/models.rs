//! `LlamaConfig` and `LlamaModel` (reference: src/models/llama.rs:11-37, :129-216, :218-279, :282-290).
//! The whole model lives behind one library handle (one weight slab, one KV slab, persistent decode kernel);
//! `named_parameters` hands out per-parameter proxies whose `set_raw_data` uploads into that slab, which is what
//! the reference's safetensors loader (src/loader.rs:10-80) calls.
use crate::autograd::{require_no_grad, Tensor};
use crate::context::{check, ctx};
use crate::ffi;
use crate::layers::{KVCache, KVCacheInner};
use crate::module::Module;
use ndarray::{ArrayD, IxDyn};
use std::cell::RefCell;
use std::collections::HashMap;
use std::ffi::CString;
use std::rc::Rc;

/// llama.rs:11-21 (defaults :23-37 = TinyLlama-1.1B)
#[derive(Clone, Debug)]
pub struct LlamaConfig {
    pub vocab_size: usize,
    pub hidden_size: usize,
    pub intermediate_size: usize,
    pub num_hidden_layers: usize,
    pub num_attention_heads: usize,
    pub num_key_value_heads: usize,
    pub rms_norm_eps: f32,
    pub max_seq_len: usize,
    pub rope_theta: f32,
}

impl Default for LlamaConfig {
    fn default() -> Self {
        LlamaConfig {
            vocab_size: 32000,
            hidden_size: 2048,
            intermediate_size: 5632,
            num_hidden_layers: 22,
            num_attention_heads: 32,
            num_key_value_heads: 4,
            rms_norm_eps: 1e-5,
            max_seq_len: 2048,
            rope_theta: 10000.0,
        }
    }
}

/// What the reference's config lacks: an explicit head size, Qwen3's per-head q/k RMSNorm, bf16 weight storage.
#[derive(Clone, Copy, Debug, Default)]
pub struct LlamaExtras {
    pub head_dim: usize,
    pub qk_norm: bool,
    pub bf16_weights: bool,
}

/// One named parameter of the model: `set_raw_data` uploads the full (unsharded) tensor.
pub struct ParamRef {
    model: *mut ffi::lumen_llama,
    name: CString,
    pub shape: Vec<usize>,
}

impl ParamRef {
    pub fn set_raw_data(&self, shape: Vec<usize>, raw_data: Vec<f32>) {
        check(unsafe {
            ffi::lumen_llama_set_param(self.model, self.name.as_ptr(), raw_data.as_ptr() as *const _, shape.as_ptr(),
                                       shape.len() as i32, ffi::LUMEN_F32)
        });
    }

    /// bf16 checkpoints: the bit patterns go to the device unwidened.
    pub fn set_raw_bf16(&self, shape: Vec<usize>, bits: Vec<u16>) {
        check(unsafe {
            ffi::lumen_llama_set_param(self.model, self.name.as_ptr(), bits.as_ptr() as *const _, shape.as_ptr(),
                                       shape.len() as i32, ffi::LUMEN_BF16)
        });
    }
}

pub struct LlamaModel {
    handle: *mut ffi::lumen_llama,
    pub config: LlamaConfig,
    extras: LlamaExtras,
}

impl LlamaModel {
    /// llama.rs:138-159.  Parameters start unset: fill them through `named_parameters` before `forward`.
    pub fn new(config: LlamaConfig) -> Self {
        LlamaModel::with_extras(config, LlamaExtras::default())
    }

    pub fn with_extras(config: LlamaConfig, extras: LlamaExtras) -> Self {
        let c = ffi::lumen_llama_config {
            vocab_size: config.vocab_size,
            hidden_size: config.hidden_size,
            intermediate_size: config.intermediate_size,
            num_hidden_layers: config.num_hidden_layers,
            num_attention_heads: config.num_attention_heads,
            num_key_value_heads: config.num_key_value_heads,
            rms_norm_eps: config.rms_norm_eps,
            max_seq_len: config.max_seq_len,
            rope_theta: config.rope_theta,
            head_dim: extras.head_dim,
            qk_norm: extras.qk_norm as i32,
            weight_dtype: if extras.bf16_weights { ffi::LUMEN_BF16 } else { ffi::LUMEN_F32 },
        };
        let mut handle = std::ptr::null_mut();
        check(unsafe { ffi::lumen_llama_new(ctx(), &c, &mut handle) });
        LlamaModel { handle, config, extras }
    }

    fn head_dim(&self) -> usize {
        if self.extras.head_dim != 0 { self.extras.head_dim } else { self.config.hidden_size / self.config.num_attention_heads }
    }

    /// llama.rs:161-170: one preallocated cache per layer (all carved out of one device slab).
    pub fn init_kv_caches(&self, batch_size: usize) -> Vec<KVCache> {
        let n = self.config.num_hidden_layers;
        let mut raw = vec![std::ptr::null_mut(); n.max(1)];
        check(unsafe { ffi::lumen_llama_init_kv_caches(self.handle, batch_size, raw.as_mut_ptr()) });
        let shape = [batch_size, self.config.num_key_value_heads, self.config.max_seq_len, self.head_dim()];
        raw.into_iter().take(n).map(|h| Rc::new(RefCell::new(KVCacheInner::from_raw(h, shape)))).collect()
    }

    /// llama.rs:172-176
    pub fn reset_kv_caches(&self, caches: &mut [KVCache]) {
        for c in caches.iter() {
            c.borrow_mut().reset();
        }
    }

    /// llama.rs:181-206: `input_ids` `[B, S]` (ids as f32) -> logits `[B, S, vocab]`; `_pos` is ignored as in the
    /// reference; a wrong number of caches panics (:182-188).
    pub fn forward(&self, input_ids: Tensor, caches: &mut Vec<KVCache>, _pos: usize) -> Tensor {
        require_no_grad("LlamaModel::forward");
        let (shape, ids) = input_ids.get_raw_data();
        assert_eq!(shape.len(), 2, "input_ids must be [B, S]");
        let (b, s) = (shape[0], shape[1]);
        let mut raw: Vec<*mut ffi::lumen_kv_cache> = caches.iter().map(|c| c.borrow().handle).collect();
        let mut logits = vec![0f32; b * s * self.config.vocab_size];
        check(unsafe {
            ffi::lumen_llama_forward(self.handle, ids.as_ptr(), b, s, raw.as_mut_ptr(), raw.len(), _pos, logits.as_mut_ptr())
        });
        Tensor::from_array_no_grad(
            ArrayD::from_shape_vec(IxDyn(&[b, s, self.config.vocab_size]), logits).expect("logits shape"))
    }

    /// The same step returning the last position's logits as a host vector (what the chat loop of src/main.rs:334-372
    /// uses), without the round trip through a device tensor.
    pub fn forward_last(&self, ids: &[f32], b: usize, s: usize, caches: &mut Vec<KVCache>) -> Vec<f32> {
        require_no_grad("LlamaModel::forward");
        let mut raw: Vec<*mut ffi::lumen_kv_cache> = caches.iter().map(|c| c.borrow().handle).collect();
        let mut logits = vec![0f32; b * self.config.vocab_size];
        check(unsafe {
            ffi::lumen_llama_forward_last(self.handle, ids.as_ptr(), b, s, raw.as_mut_ptr(), raw.len(), 0, logits.as_mut_ptr())
        });
        logits
    }

    /// llama.rs:209-216: training is out of scope on this backend.
    pub fn forward_train(&self, _input_ids: Tensor) -> Tensor {
        panic!("LlamaModel::forward_train: the training path is not provided by this backend");
    }

    /// llama.rs:218-279: the Hugging Face parameter names.
    pub fn named_parameters(&self) -> HashMap<String, ParamRef> {
        let c = &self.config;
        let d = self.head_dim();
        let (qd, kvd) = (c.num_attention_heads * d, c.num_key_value_heads * d);
        let mut shapes: Vec<(String, Vec<usize>)> = vec![
            ("model.embed_tokens.weight".into(), vec![c.vocab_size, c.hidden_size]),
            ("model.norm.weight".into(), vec![c.hidden_size]),
            ("lm_head.weight".into(), vec![c.vocab_size, c.hidden_size]),
        ];
        for i in 0..c.num_hidden_layers {
            let p = format!("model.layers.{}.", i);
            shapes.push((format!("{}self_attn.q_proj.weight", p), vec![qd, c.hidden_size]));
            shapes.push((format!("{}self_attn.k_proj.weight", p), vec![kvd, c.hidden_size]));
            shapes.push((format!("{}self_attn.v_proj.weight", p), vec![kvd, c.hidden_size]));
            shapes.push((format!("{}self_attn.o_proj.weight", p), vec![c.hidden_size, qd]));
            shapes.push((format!("{}mlp.gate_proj.weight", p), vec![c.intermediate_size, c.hidden_size]));
            shapes.push((format!("{}mlp.up_proj.weight", p), vec![c.intermediate_size, c.hidden_size]));
            shapes.push((format!("{}mlp.down_proj.weight", p), vec![c.hidden_size, c.intermediate_size]));
            shapes.push((format!("{}input_layernorm.weight", p), vec![c.hidden_size]));
            shapes.push((format!("{}post_attention_layernorm.weight", p), vec![c.hidden_size]));
            if self.extras.qk_norm {
                shapes.push((format!("{}self_attn.q_norm.weight", p), vec![d]));
                shapes.push((format!("{}self_attn.k_norm.weight", p), vec![d]));
            }
        }
        shapes
            .into_iter()
            .map(|(name, shape)| {
                let cname = CString::new(name.clone()).expect("parameter names hold no NUL");
                (name, ParamRef { model: self.handle, name: cname, shape })
            })
            .collect()
    }

    /// Weight bytes one decode step streams from HBM on this rank.
    pub fn weight_bytes_per_step(&self) -> usize {
        unsafe { ffi::lumen_llama_weight_bytes(self.handle) }
    }
}

impl Module for LlamaModel {
    /// llama.rs:282-290: `Module::forward` is the training entry of the reference.
    fn forward(&self, input: Tensor) -> Tensor {
        self.forward_train(input)
    }

    fn parameters(&self) -> Vec<Tensor> {
        Vec::new()  // the weights live in the library's slab: use `named_parameters`
    }
}

impl Drop for LlamaModel {
    fn drop(&mut self) {
        unsafe { ffi::lumen_llama_free(self.handle) };
    }
}
