"""CPU checks of the drop-in boundary: the shared library loads, exports every symbol declared in
include/lumen_b200.h, the ctypes prototypes cover the same set, and there is no CPU fallback."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "lumen_b200.h"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(lumen_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(L):
    lib = L._lib.load()
    names = declared_symbols()
    assert len(names) >= 50
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
    assert sorted(L._lib.PROTOTYPES) == names


def test_status_strings_and_version(L):
    lib = L._lib.load()
    assert lib.lumen_version() >= 100
    assert lib.lumen_status_string(0) == b"ok"
    assert b"overflow" in lib.lumen_status_string(L._lib.ERR_KV_OVERFLOW)


def test_no_cpu_fallback(L):
    """Without a CUDA device a context cannot be created: nothing falls back to the host."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(L.LumenError) as e:
        L.Context(0)
    assert e.value.code == L._lib.ERR_CUDA


def test_null_arguments_are_rejected(L):
    lib = L._lib.load()
    assert lib.lumen_ctx_create(0, 0, 1, None, None) == L._lib.ERR_INVALID
    assert lib.lumen_ctx_create(0, 3, 2, None, C.byref(C.c_void_p())) == L._lib.ERR_INVALID
    assert lib.lumen_tensor_free(None) == L._lib.ERR_INVALID
    assert lib.lumen_kv_len(None) == 0
    assert lib.lumen_tensor_ndim(None) == -1


def test_product_does_not_import_the_oracle():
    """The oracle is test infrastructure: nothing under lumen_b200/ may reference it."""
    for p in (ROOT / "lumen_b200").rglob("*"):
        if p.suffix in {".py", ".cu", ".cuh", ".h", ".hpp", ".cpp"}:
            assert "oracle" not in p.read_text().lower(), p


def test_host_side_config_and_synth(L):
    from lumen_b200 import synth
    cfg = L.LlamaConfig()
    shapes = cfg.param_shapes()
    assert len(shapes) == 3 + 22 * 9
    n = sum(int(np.prod(s)) for k, s in shapes.items() if k != "model.embed_tokens.weight")
    assert n == 1_034_512_384  # parameters one TinyLlama decode step streams
    small = L.LlamaConfig(vocab_size=11, hidden_size=8, intermediate_size=12, num_hidden_layers=1,
                          num_attention_heads=2, num_key_value_heads=1)
    a = dict(synth.iter_params(small, 0))
    b = dict(synth.iter_params(small, 0))
    assert all(np.array_equal(a[k], b[k]) for k in a)
    assert np.all(a["model.norm.weight"] == 1.0)
    r = dict(synth.iter_params(small, 0, round_bf16=True))
    w = r["lm_head.weight"].view(np.uint32)
    assert np.all((w & 0xFFFF) == 0)
    assert np.array_equal(synth.token_ids(1, 5, 11), synth.token_ids(1, 5, 11))


def test_no_grad_switches(L):
    assert not L.is_no_grad()
    with L.no_grad():
        assert L.is_no_grad()
    L.set_inference_mode(True)
    assert L.is_no_grad()
    L.set_inference_mode(False)
    assert not L.is_no_grad()


def test_cpu_arm_of_the_benchmark_does_not_load_the_cuda_library():
    """`bench.py --impl reference` times the CPU restatement and must not map liblumen_b200.so: its helpers take the
    seeded generators from lumen_b200/synth.py by file path, without importing the package."""
    import subprocess
    import sys
    code = (
        "import sys, importlib.util\n"
        f"spec = importlib.util.spec_from_file_location('bench', r'{ROOT / 'bench.py'}')\n"
        "b = importlib.util.module_from_spec(spec); spec.loader.exec_module(b)\n"
        "cfg = b.tinyllama_cfg('f32', 2048)\n"
        "small = dict(cfg, num_hidden_layers=1, vocab_size=64, hidden_size=64, intermediate_size=128, num_attention_heads=4, num_key_value_heads=2)\n"
        "params = dict(b.gen_params(small, 'f32'))\n"
        "ids = b.load_synth().token_ids(1, 40, 64)\n"
        "b.PROMPT_LEN = 8\n"
        "tps, steps, threads, lg = b.cpu_decode(small, params, ids, 5.0, 3, 2)\n"
        "assert steps == 3 and lg.shape == (5, 64) and threads >= 1\n"
        "assert 'lumen_b200' not in sys.modules, 'the package was imported'\n"
        "maps = open('/proc/self/maps').read()\n"
        "assert 'liblumen_b200' not in maps, 'the CUDA library was mapped'\n"
        "assert 'liblumen_oracle' in maps\n"
        "assert b.stream_bytes(cfg, 'f32') == 4 * 1034512384, b.stream_bytes(cfg, 'f32')\n"
        "print('ok')\n")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300,
                       env=dict(__import__("os").environ, OMP_NUM_THREADS="1"))
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), r.stdout + r.stderr
