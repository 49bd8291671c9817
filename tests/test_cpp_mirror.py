"""The C++ host mirror (include/lumen_b200.hpp): compiles and links against the library on CPU; on a GPU
it drives a small Llama through the reference's prefill + per-token loop and must match the oracle."""
import subprocess
from pathlib import Path

import numpy as np
import pytest

from helpers import TOL_F32, rel_err, small_cfg

ROOT = Path(__file__).resolve().parents[1]
LIBDIR = ROOT / "lumen_b200" / "lib"


@pytest.fixture(scope="module")
def mirror_binary(tmp_path_factory, L):
    out = tmp_path_factory.mktemp("cppmirror") / "host_mirror_check"
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-Wextra", "-Werror", "-I", str(ROOT / "include"),
           str(ROOT / "tests" / "cpp" / "host_mirror_check.cpp"), "-L", str(LIBDIR), "-llumen_b200",
           f"-Wl,-rpath,{LIBDIR}", "-o", str(out)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    return out


def test_header_compiles_links_and_reports_missing_device(mirror_binary):
    import torch
    if torch.cuda.is_available():
        pytest.skip("covers the no-device path")
    r = subprocess.run([str(mirror_binary), "--no-gpu"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "Error code=7" in r.stdout  # LUMEN_ERR_CUDA: no CPU fallback


@pytest.mark.gpu
def test_cpp_mirror_matches_oracle(mirror_binary, oracle, L, tmp_path):
    from lumen_b200 import synth
    cfg = small_cfg(vocab_size=96, hidden_size=128, num_attention_heads=8, num_key_value_heads=2, intermediate_size=320,
                    num_hidden_layers=3, max_seq_len=32)
    lcfg = L.LlamaConfig(**cfg)
    params = {n: w for n, w in synth.iter_params(lcfg, 4, std=0.05)}
    prompt, steps = 6, 5
    ids = synth.token_ids(8, prompt + steps, cfg["vocab_size"])
    order = ["model.embed_tokens.weight"]
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        order += [p + s for s in ("self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight",
                                  "self_attn.o_proj.weight", "mlp.gate_proj.weight", "mlp.up_proj.weight",
                                  "mlp.down_proj.weight", "input_layernorm.weight", "post_attention_layernorm.weight")]
    order += ["model.norm.weight", "lm_head.weight"]
    np.concatenate([params[n].astype(np.float32).ravel() for n in order]).tofile(tmp_path / "params.bin")
    ids.astype(np.float32).tofile(tmp_path / "ids.bin")
    (tmp_path / "cfg.txt").write_text(" ".join(str(v) for v in (
        cfg["vocab_size"], cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"], cfg["num_attention_heads"],
        cfg["num_key_value_heads"], cfg["rms_norm_eps"], cfg["max_seq_len"], cfg["rope_theta"], prompt, steps)))
    r = subprocess.run([str(mirror_binary), str(tmp_path)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    got = np.fromfile(tmp_path / "logits.bin", dtype=np.float32).reshape(steps + 1, cfg["vocab_size"])
    om = oracle.Llama(cfg, params, "f64")
    oc = om.init_kv_caches(1)
    want = [om.forward(ids[None, :prompt], oc)[0, -1]]
    for t in range(steps):
        want.append(om.forward(ids[None, prompt + t:prompt + t + 1], oc)[0, 0])
    want = np.stack(want)
    for g, w in zip(got, want):
        assert rel_err(g, w) < TOL_F32
    assert (got.argmax(-1) == want.argmax(-1)).all()
