"""The Rust shim crate (rust/) cannot be compiled in the build image (no rustc), so it is checked as text:
its `extern "C"` block must be exactly what rust/gen_ffi.py derives from include/lumen_b200.h, every declared function
must be exported by the built library, every `ffi::` call of a wrapper must be declared, and the wrappers must carry
the reference's signatures (src/autograd.rs, src/module.rs, src/models/llama.rs, src/kv_cache.rs,
src/layers/attention/self_attention.rs of the reference)."""
import ctypes as C
import re
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
RUST = ROOT / "rust"


def _ffi_names():
    return re.findall(r"pub fn (lumen_[a-z0-9_]+)\(", (RUST / "src" / "ffi.rs").read_text())


def test_extern_block_is_generated_from_the_header():
    r = subprocess.run([sys.executable, str(RUST / "gen_ffi.py"), "--check"])
    assert r.returncode == 0, "rust/src/ffi.rs is out of date: run python rust/gen_ffi.py"
    header = (ROOT / "include" / "lumen_b200.h").read_text()
    declared = set(re.findall(r"\b(lumen_[a-z0-9_]+)\s*\(", re.sub(r"/\*.*?\*/", " ", header, flags=re.S)))
    assert set(_ffi_names()) == declared


def test_every_declared_function_is_exported_by_the_library():
    lib = C.CDLL(str(ROOT / "lumen_b200" / "lib" / "liblumen_b200.so"))
    for name in _ffi_names():
        assert hasattr(lib, name), name


def test_wrappers_call_only_declared_functions_and_cover_the_hot_path():
    declared = set(_ffi_names())
    used = set()
    for f in (RUST / "src").glob("*.rs"):
        if f.name != "ffi.rs":
            used |= set(re.findall(r"ffi::(lumen_[a-z0-9_]+)\s*\(", f.read_text()))  # calls, not type names
    assert used <= declared, used - declared
    # everything a decode loop written against the reference needs goes through the shim
    for name in ("lumen_llama_new", "lumen_llama_set_param", "lumen_llama_init_kv_caches", "lumen_llama_forward",
                 "lumen_self_attention_forward", "lumen_matmul", "lumen_rmsnorm", "lumen_embedding", "lumen_rope_forward",
                 "lumen_kv_new", "lumen_kv_reset", "lumen_llama_kv_update", "lumen_llama_kv_get_view", "lumen_silu",
                 "lumen_mul", "lumen_add", "lumen_fused_softmax", "lumen_tensor_to_host", "lumen_tensor_set"):
        assert name in used, name


SIGNATURES = {
    "autograd.rs": ["pub fn no_grad<R>(f: impl FnOnce() -> R) -> R", "pub fn is_no_grad() -> bool",
                    "pub fn set_inference_mode(on: bool)", "pub fn from_array_no_grad(data: ArrayD<f32>) -> Tensor",
                    "pub fn data(&self) -> ArrayD<f32>", "pub fn reshape(&self, shape: Vec<i32>) -> Tensor",
                    "pub fn get_raw_data(&self) -> (Vec<usize>, Vec<f32>)",
                    "pub fn set_raw_data(&self, shape: Vec<usize>, raw_data: Vec<f32>)"],
    "module.rs": ["fn forward(&self, input: Tensor) -> Tensor;", "fn parameters(&self) -> Vec<Tensor>;"],
    "models.rs": ["pub fn new(config: LlamaConfig) -> Self", "pub fn init_kv_caches(&self, batch_size: usize) -> Vec<KVCache>",
                  "pub fn reset_kv_caches(&self, caches: &mut [KVCache])",
                  "pub fn forward(&self, input_ids: Tensor, caches: &mut Vec<KVCache>, _pos: usize) -> Tensor",
                  "pub fn named_parameters(&self)"],
    "kv_cache.rs": ["pub fn new(config: &LlamaConfig) -> Self", "pub fn update(&mut self, k: &Tensor, v: &Tensor, start_pos: usize)",
                    "pub fn get_view(&self, current_len: usize) -> (Tensor, Tensor)"],
    "layers.rs": ["pub fn new(b: usize, h_kv: usize, max_seq: usize, d: usize) -> Self", "pub fn reset(&mut self)",
                  "pub type KVCache = Rc<RefCell<KVCacheInner>>;",
                  "pub fn forward(&self, x: Tensor, cache: Option<KVCache>) -> (Tensor, Option<KVCache>)",
                  "pub fn new_no_bias(in_features: usize, out_features: usize) -> Self",
                  "pub fn forward(&self, x: &Tensor, offset: usize) -> Tensor",
                  "pub fn new(dim: usize, max_seq_len: usize, theta: f32) -> Self"],
}


def test_wrappers_keep_the_reference_signatures():
    for fname, sigs in SIGNATURES.items():
        text = " ".join((RUST / "src" / fname).read_text().split())
        for sig in sigs:
            assert " ".join(sig.split()) in text, (fname, sig)
