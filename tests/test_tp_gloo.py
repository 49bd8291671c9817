"""Tensor-parallel host logic on CPU: the shard plan the library applies at `set_param`, and a multi-process
(gloo) forward on the planned slices with the exchanges where the CUDA path has them."""
import json
import os
import socket
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from helpers import small_cfg

ROOT = Path(__file__).resolve().parents[1]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run_ranks(cfg: dict, world: int):
    port = _free_port()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   TP_TEST_CFG=json.dumps(cfg), OMP_NUM_THREADS="1")
        procs.append(subprocess.Popen([sys.executable, str(ROOT / "tests" / "tp_gloo_worker.py")], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    outs = []
    try:
        for p in procs:
            outs.append(p.communicate(timeout=240))
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
    for p, (so, se) in zip(procs, outs):
        assert p.returncode == 0, se[-2000:]
    return json.loads(outs[0][0].strip().splitlines()[-1])


@pytest.mark.parametrize("world,cfg", [
    (2, small_cfg(vocab_size=96)),                                      # 4 q heads, 2 KV heads -> 2 + 1 per rank
    (4, small_cfg(vocab_size=96, num_attention_heads=8, hidden_size=64)),  # 2 KV heads on 4 ranks: replicated
])
def test_sharded_forward_equals_unsharded(world, cfg):
    res = _run_ranks(cfg, world)
    assert res["world"] == world and res["max_rel_err"] < 1e-12


def test_plan_partitions_every_parameter():
    from lumen_b200.llama import LlamaConfig, tp_param_slice
    cfg = LlamaConfig(**small_cfg(vocab_size=96, num_attention_heads=8, num_key_value_heads=4, hidden_size=64,
                                  intermediate_size=160, qk_norm=True))
    d = 64 // 8
    for T in (1, 2, 4, 8):
        for name, shape in cfg.param_shapes().items():
            sl = [tp_param_slice(cfg, r, T, name) for r in range(T)]
            assert all(tuple(s["shape"]) == tuple(shape) for s in sl)
            if len(shape) == 1 or "embed_tokens" in name:
                assert all(s["rows"] == (0, shape[0]) for s in sl)  # replicated
                continue
            cover = np.zeros(shape, np.int32)
            for s in sl:
                cover[s["rows"][0]:s["rows"][1], s["cols"][0]:s["cols"][1]] += 1
            if "k_proj" in name or "v_proj" in name:
                rep = max(1, T // 4)  # 4 KV heads: replicated T/4 times once T > 4
                assert np.all(cover == rep), (name, T)
                assert all((s["rows"][1] - s["rows"][0]) % d == 0 for s in sl)
            else:
                assert np.all(cover == 1), (name, T)
        # each rank's q heads must read KV heads it holds
        for r in range(T):
            q = tp_param_slice(cfg, r, T, "model.layers.0.self_attn.q_proj.weight")["rows"]
            k = tp_param_slice(cfg, r, T, "model.layers.0.self_attn.k_proj.weight")["rows"]
            heads = range(q[0] // d, q[1] // d)
            assert all(k[0] // d <= h // 2 < k[1] // d for h in heads)


def test_plan_errors():
    from lumen_b200 import LumenError, _lib
    from lumen_b200.llama import LlamaConfig, tp_param_slice
    cfg = LlamaConfig(**small_cfg(vocab_size=96))
    with pytest.raises(LumenError) as e:
        tp_param_slice(cfg, 0, 2, "model.layers.0.self_attn.nope.weight")
    assert e.value.code == _lib.ERR_PARAM_NAME
    with pytest.raises(LumenError) as e:
        tp_param_slice(cfg, 0, 2, "model.layers.9.mlp.up_proj.weight")  # only 2 layers
    assert e.value.code == _lib.ERR_PARAM_NAME
    with pytest.raises(LumenError) as e:
        tp_param_slice(cfg, 0, 3, "lm_head.weight")  # 4 heads on 3 ranks
    assert e.value.code == _lib.ERR_UNSUPPORTED
    with pytest.raises(LumenError) as e:
        tp_param_slice(cfg, 2, 2, "lm_head.weight")  # rank out of range
    assert e.value.code == _lib.ERR_INVALID
