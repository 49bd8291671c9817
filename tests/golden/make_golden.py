"""Regenerates tests/golden/*.npz from the CPU oracle.

The reference (chen-197/Lumen) ships no golden vectors and cannot be run here, so these fixtures
pin the ORACLE's own output (a regression anchor for the C restatement, and a CPU-box-independent
target for the GPU parity tests); they are not outputs of the reference.

    python tests/golden/make_golden.py
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

from helpers import make_params, small_cfg  # noqa: E402
from oracle import binding as O  # noqa: E402

OUT = Path(__file__).resolve().parent


class _L:  # make_params only needs LlamaConfig; avoid loading the CUDA library here
    from lumen_b200.llama import LlamaConfig


def llama_case(name, cfg, seed, prompt_len, steps, batch=1, std=0.08):
    params = make_params(_L, cfg, seed, std=std, random_norms=True)
    model = O.Llama(cfg, params, "f32")
    caches = model.init_kv_caches(batch)
    rng = np.random.default_rng(seed + 1)
    ids = rng.integers(0, cfg["vocab_size"], size=(batch, prompt_len + steps)).astype(np.float32)
    outs = [model.forward(ids[:, :prompt_len], caches)[:, -1]]
    for t in range(steps):
        outs.append(model.forward(ids[:, prompt_len + t:prompt_len + t + 1], caches)[:, 0])
    np.savez_compressed(OUT / f"{name}.npz", ids=ids, logits=np.stack(outs, 1).astype(np.float32),
                        seed=seed, prompt_len=prompt_len, steps=steps, batch=batch, std=std,
                        **{f"cfg_{k}": v for k, v in cfg.items()})


def op_cases():
    rng = np.random.default_rng(7)
    d = {}
    x = rng.standard_normal((3, 50), dtype=np.float32)
    w = rng.standard_normal((50,), dtype=np.float32)
    d["rms_x"], d["rms_w"], d["rms_out"] = x, w, O.rmsnorm(x, w, 1e-5)
    a = rng.standard_normal((1, 1, 77), dtype=np.float32)
    wm = rng.standard_normal((13, 77), dtype=np.float32)
    d["mm_a"], d["mm_w"], d["mm_out"] = a, wm, O.matmul(a, wm)
    xr = rng.standard_normal((2, 3, 5, 16), dtype=np.float32)
    d["rope_x"], d["rope_out"] = xr, O.rope_forward(xr, 4, 32, 10000.0)
    s = rng.standard_normal((2, 2, 4, 6), dtype=np.float32)
    d["sm_x"], d["sm_out"] = s, O.fused_softmax(s, 0.25, True)
    g = rng.standard_normal((40,), dtype=np.float32)
    d["silu_x"], d["silu_out"] = g, O.silu(g)
    np.savez_compressed(OUT / "ops.npz", **d)


if __name__ == "__main__":
    O.build()
    llama_case("llama_small_gqa", small_cfg(), seed=11, prompt_len=5, steps=6)
    llama_case("llama_small_b3", small_cfg(num_key_value_heads=1, hidden_size=96, num_attention_heads=6), seed=12,
               prompt_len=4, steps=4, batch=3)
    llama_case("llama_small_qknorm", small_cfg(head_dim=32, qk_norm=True, rope_theta=1e6), seed=13, prompt_len=6, steps=5)
    op_cases()
    print("wrote", sorted(p.name for p in OUT.glob("*.npz")))
