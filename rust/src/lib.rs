//! lumen_b200: drop-in for the Llama inference path of chen-197/Lumen on one or more B200 GPUs.
//!
//! The public items keep the reference's names and signatures (`Tensor`, `no_grad`, `Module`, `Linear`,
//! `Embedding`, `RMSNorm`, `SiLU`, `RotaryEmbedding`, `SelfAttention`, `KVCacheInner`, `KVCache`, `LlamaKVCache`,
//! `LlamaConfig`, `LlamaModel`), so that the reference's `src/main.rs` builds against this crate once its `use`
//! paths point here.  Every method forwards to the C ABI in `ffi` (include/lumen_b200.h); there is no CPU path.
//! Where the reference panics, the shim panics with the library's message (`Cargo.toml` of the reference makes a
//! panic an abort).  Only inference exists: gradients, `backward` and the training branches are not provided.
//!
//! Not compiled where it was written (the build image has no Rust toolchain).
pub mod autograd;
pub mod context;
pub mod ffi;
pub mod kv_cache;
pub mod layers;
pub mod models;
pub mod module;
pub mod ops;

pub use autograd::{is_inference_mode, is_no_grad, no_grad, set_inference_mode, NoGradGuard, Tensor};
pub use kv_cache::LlamaKVCache;
pub use layers::{Embedding, KVCache, KVCacheInner, Linear, RMSNorm, RotaryEmbedding, SelfAttention, SiLU};
pub use models::{LlamaConfig, LlamaModel};
pub use module::Module;
