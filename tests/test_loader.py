"""safetensors loader (src/loader.rs:10-80): container parsing on CPU; on a GPU a model filled from a file
(f32 and bf16 tensors) must equal the model filled by `set_param`."""
import numpy as np
import pytest

from helpers import TOL_BF16, rel_err, small_cfg


def _params(L, cfg, seed=3):
    from lumen_b200 import synth
    return {n: w for n, w in synth.iter_params(L.LlamaConfig(**cfg), seed, std=0.05)}


def test_container_round_trip_and_errors(tmp_path):
    from lumen_b200.loader import SafeTensorsFile, save_safetensors
    from lumen_b200.tensor import f32_to_bf16_bits
    rng = np.random.default_rng(0)
    a = rng.standard_normal((3, 5), dtype=np.float32)
    b = f32_to_bf16_bits(rng.standard_normal((7,), dtype=np.float32))
    save_safetensors(tmp_path / "t.safetensors", {"a": a, "b.weight": b})
    with SafeTensorsFile(tmp_path / "t.safetensors") as f:
        assert sorted(f.names()) == ["a", "b.weight"]
        dt, shape, arr = f.tensor("a")
        assert dt == "F32" and shape == (3, 5) and np.array_equal(np.array(arr), a)
        dt, shape, arr = f.tensor("b.weight")
        assert dt == "BF16" and shape == (7,) and np.array_equal(np.array(arr), b)
        del arr
    # an unsupported dtype is an error, as in the reference (loader.rs:67)
    import json, struct
    hdr = json.dumps({"x": {"dtype": "I64", "shape": [1], "data_offsets": [0, 8]}}).encode()
    (tmp_path / "bad.safetensors").write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with SafeTensorsFile(tmp_path / "bad.safetensors") as f:
        with pytest.raises(ValueError, match="Unsupported dtype"):
            f.tensor("x")
    (tmp_path / "short.safetensors").write_bytes(b"abc")
    with pytest.raises(ValueError, match="too short"):
        SafeTensorsFile(tmp_path / "short.safetensors")


@pytest.mark.gpu
def test_model_loaded_from_file_equals_set_param(L, tmp_path):
    from lumen_b200.loader import load_llama_weights, save_safetensors
    from lumen_b200.tensor import bf16_bits_to_f32, f32_to_bf16_bits
    cfg = small_cfg()
    params = _params(L, cfg)
    ids = np.arange(6, dtype=np.float32)[None] % cfg["vocab_size"]

    def logits(model):
        caches = model.init_kv_caches(1)
        with L.no_grad():
            return model.forward(ids, caches)

    ref = L.LlamaModel(L.LlamaConfig(**cfg))
    ref.load_state(params)
    want = logits(ref)

    save_safetensors(tmp_path / "f32.safetensors", params)
    m1 = L.LlamaModel(L.LlamaConfig(**cfg))
    assert load_llama_weights(tmp_path / "f32.safetensors", m1) == []
    assert np.array_equal(logits(m1), want)

    # bf16 checkpoint into an f32 model: equals the f32 model holding the widened values (loader.rs:50-64)
    bits = {n: (f32_to_bf16_bits(w) if w.ndim == 2 else w) for n, w in params.items()}
    save_safetensors(tmp_path / "bf16.safetensors", bits)
    widened = {n: (bf16_bits_to_f32(b).reshape(params[n].shape) if params[n].ndim == 2 else params[n]) for n, b in bits.items()}
    ref2 = L.LlamaModel(L.LlamaConfig(**cfg))
    ref2.load_state(widened)
    m2 = L.LlamaModel(L.LlamaConfig(**cfg))
    assert load_llama_weights(tmp_path / "bf16.safetensors", m2) == []
    assert np.array_equal(logits(m2), logits(ref2))
    # ... and into a bf16-weight model: the bits are kept
    m3 = L.LlamaModel(L.LlamaConfig(**cfg, weight_dtype="bf16"))
    load_llama_weights(tmp_path / "bf16.safetensors", m3)
    assert rel_err(logits(m3), logits(ref2)) < TOL_BF16

    # a parameter missing from the file is reported, not fatal (loader.rs:72-77); forward then refuses
    partial = {n: w for n, w in params.items() if n != "lm_head.weight"}
    save_safetensors(tmp_path / "partial.safetensors", partial)
    m4 = L.LlamaModel(L.LlamaConfig(**cfg))
    assert load_llama_weights(tmp_path / "partial.safetensors", m4) == ["lm_head.weight"]
    with pytest.raises(L.LumenError) as e:
        logits(m4)
    assert e.value.code == L._lib.ERR_MISSING_PARAM
