//! `Module` (reference: src/module.rs:12-24).  `save` / `load` of the reference's bincode checkpoints are not part of
//! the decode path and are left to the caller (`parameters()` + `get_raw_data` / `set_raw_data` are enough for them).
use crate::autograd::{set_inference_mode, Tensor};

pub trait Module {
    fn forward(&self, input: Tensor) -> Tensor;
    fn parameters(&self) -> Vec<Tensor>;

    fn train_mode(&mut self) {
        set_inference_mode(false);
    }

    fn eval_mode(&mut self) {
        set_inference_mode(true);
    }
}
