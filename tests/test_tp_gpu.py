"""Tensor parallelism on real GPUs (one process per GPU; the sums over the ranks run inside the persistent decode kernel
for batch 1, in the fused peer-memory sum kernel for batched steps and short prefills, through NCCL for long prefill
slices): TP=N logits against the CPU oracle.  Skipped on a box with a single GPU."""
import json
import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest

from helpers import TOL_BF16, TOL_F32, small_cfg

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def _gpu_count() -> int:
    import torch
    return torch.cuda.device_count()


def _run(cfg: dict, world: int, dtype: str, prompt: int = 7, batch: int = 1, extra_env: dict | None = None):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   TP_TEST_CFG=json.dumps(cfg), TP_TEST_DTYPE=dtype, TP_TEST_PROMPT=str(prompt), TP_TEST_BATCH=str(batch), NCCL_NVLS_ENABLE="0",
                   **(extra_env or {}))
        procs.append(subprocess.Popen([sys.executable, str(ROOT / "tests" / "tp_gpu_worker.py")], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    outs = []
    try:
        for p in procs:
            outs.append(p.communicate(timeout=300))
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
    for p, (so, se) in zip(procs, outs):
        assert p.returncode == 0, se[-3000:]
    return json.loads(outs[0][0].strip().splitlines()[-1])


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_tp2_matches_oracle(dtype):
    if _gpu_count() < 2:
        pytest.skip("needs 2 GPUs")
    cfg = small_cfg(vocab_size=96, hidden_size=128, num_attention_heads=8, num_key_value_heads=2, intermediate_size=320,
                    num_hidden_layers=3, max_seq_len=32)
    res = _run(cfg, 2, dtype)
    assert res["max_rel_err"] < (TOL_F32 if dtype == "f32" else TOL_BF16), res
    assert res["argmax_equal"]


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_tp2_long_prompt(dtype):
    """A 100-token prompt: per-rank heads through the tensor-core GEMM and prefill attention, all-reduce per block."""
    if _gpu_count() < 2:
        pytest.skip("needs 2 GPUs")
    cfg = small_cfg(vocab_size=96, hidden_size=256, num_attention_heads=4, num_key_value_heads=2, intermediate_size=320,
                    num_hidden_layers=2, max_seq_len=128)
    res = _run(cfg, 2, dtype, prompt=100)
    assert res["max_rel_err"] < (TOL_F32 if dtype == "f32" else TOL_BF16), res
    assert res["argmax_equal"]


@pytest.mark.parametrize("dtype,batch,prompt", [("f32", 12, 20), ("bf16", 3, 20), ("f32", 12, 100)])
def test_tp2_batched_steps_fused_sum(dtype, batch, prompt):
    """Batched prefill + batched decode steps (replayed as a CUDA graph): the sum over the ranks runs as one kernel over peer
    memory behind each row-parallel product (split-K slices of the tensor-core product included, RMSNorm of the next block
    fused where the tiled product follows).  12 x 100 prompt rows exceed that kernel's buffer and take NCCL instead."""
    if _gpu_count() < 2:
        pytest.skip("needs 2 GPUs")
    cfg = small_cfg(vocab_size=96, hidden_size=256, num_attention_heads=4, num_key_value_heads=2, intermediate_size=320,
                    num_hidden_layers=3, max_seq_len=128)
    res = _run(cfg, 2, dtype, prompt=prompt, batch=batch)
    assert res["max_rel_err"] < (TOL_F32 if dtype == "f32" else TOL_BF16), res
    assert res["argmax_equal"]


def test_tp2_batched_steps_nccl_switch():
    """LUMEN_TP_NCCL=1 keeps the NCCL all-reduce per block (the comparison arm of the fused sum)."""
    if _gpu_count() < 2:
        pytest.skip("needs 2 GPUs")
    cfg = small_cfg(vocab_size=96, hidden_size=256, num_attention_heads=4, num_key_value_heads=2, intermediate_size=320,
                    num_hidden_layers=2, max_seq_len=128)
    res = _run(cfg, 2, "f32", prompt=20, batch=12, extra_env={"LUMEN_TP_NCCL": "1"})
    assert res["max_rel_err"] < TOL_F32 and res["argmax_equal"], res


def test_tp4_with_replicated_kv_heads():
    if _gpu_count() < 4:
        pytest.skip("needs 4 GPUs")
    cfg = small_cfg(vocab_size=96, hidden_size=128, num_attention_heads=8, num_key_value_heads=2, intermediate_size=320,
                    num_hidden_layers=2, max_seq_len=32)
    res = _run(cfg, 4, "f32")
    assert res["max_rel_err"] < TOL_F32 and res["argmax_equal"], res
