"""One rank of the CPU tensor-parallel check (launched by test_tp_gloo.py, one process per rank, gloo).

Each rank asks the library for its slice of every parameter (`lumen_tp_param_slice`, the plan
`lumen_llama_set_param` applies), runs a float64 numpy forward on its slices with the exchanges placed where
the CUDA path places them (allreduce of the o_proj and down_proj partial sums, allgather of the logits), and
rank 0 compares the result with the unsharded model."""
import json
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import np_reference as NP  # noqa: E402


def main():
    cfg = json.loads(os.environ["TP_TEST_CFG"])
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{os.environ['MASTER_PORT']}", rank=rank, world_size=world)
    from lumen_b200 import synth
    from lumen_b200.llama import LlamaConfig, tp_param_slice

    lcfg = LlamaConfig(**cfg)
    full = {n: w for n, w in synth.iter_params(lcfg, 7, std=0.05)}
    rng = np.random.default_rng(11)
    for n in full:  # non-trivial norm gains
        if n.endswith("norm.weight") or "layernorm" in n:
            full[n] = (1 + 0.1 * rng.standard_normal(full[n].shape)).astype(np.float32)
    ids = synth.token_ids(2, 18, cfg["vocab_size"]).reshape(2, 9)

    P = {}
    for n, w in full.items():
        sl = tp_param_slice(lcfg, rank, world, n)
        assert tuple(sl["shape"]) == w.shape, (n, sl, w.shape)
        part = w[sl["rows"][0]:sl["rows"][1]]
        if w.ndim == 2:
            part = part[:, sl["cols"][0]:sl["cols"][1]]
        P[n] = part.astype(np.float64)

    def allreduce(a):
        t = torch.from_numpy(np.ascontiguousarray(a))
        dist.all_reduce(t)
        return t.numpy()

    H, hq, hkv = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d = cfg.get("head_dim") or H // hq
    eps, theta = cfg["rms_norm_eps"], cfg["rope_theta"]
    b, s = ids.shape
    x = P["model.embed_tokens.weight"][ids.astype(np.int64)]
    pos = np.arange(s)
    mask = np.triu(np.full((s, s), -np.inf), k=1)
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        hq_l = P[p + "self_attn.q_proj.weight"].shape[0] // d
        hkv_l = P[p + "self_attn.k_proj.weight"].shape[0] // d
        nx = NP.rmsnorm(x, P[p + "input_layernorm.weight"], eps)
        q = (nx @ P[p + "self_attn.q_proj.weight"].T).reshape(b, s, hq_l, d).transpose(0, 2, 1, 3)
        k = (nx @ P[p + "self_attn.k_proj.weight"].T).reshape(b, s, hkv_l, d).transpose(0, 2, 1, 3)
        v = (nx @ P[p + "self_attn.v_proj.weight"].T).reshape(b, s, hkv_l, d).transpose(0, 2, 1, 3)
        if cfg.get("qk_norm"):
            q = NP.rmsnorm(q, P[p + "self_attn.q_norm.weight"], eps)
            k = NP.rmsnorm(k, P[p + "self_attn.k_norm.weight"], eps)
        q, k = NP.rope(q, pos, theta), NP.rope(k, pos, theta)
        k = np.repeat(k, hq_l // hkv_l, axis=1)  # local q head j reads local KV head j // (hq_l / hkv_l)
        v = np.repeat(v, hq_l // hkv_l, axis=1)
        sc = q @ k.transpose(0, 1, 3, 2) / np.sqrt(d) + mask
        sc = np.exp(sc - sc.max(-1, keepdims=True))
        att = ((sc / sc.sum(-1, keepdims=True)) @ v).transpose(0, 2, 1, 3).reshape(b, s, hq_l * d)
        x = x + allreduce(att @ P[p + "self_attn.o_proj.weight"].T)          # exchange 1 of the block
        nh = NP.rmsnorm(x, P[p + "post_attention_layernorm.weight"], eps)
        g = nh @ P[p + "mlp.gate_proj.weight"].T
        u = nh @ P[p + "mlp.up_proj.weight"].T
        x = x + allreduce(((g / (1.0 + np.exp(-g))) * u) @ P[p + "mlp.down_proj.weight"].T)  # exchange 2
    x = NP.rmsnorm(x, P["model.norm.weight"], eps)
    local = torch.from_numpy(np.ascontiguousarray(x @ P["lm_head.weight"].T))
    parts = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(parts, local)
    logits = np.concatenate([t.numpy() for t in parts], axis=-1)

    if rank == 0:
        want = NP.llama_logits(cfg, full, ids)
        err = float(np.abs(logits - want).max() / np.abs(want).max())
        print(json.dumps({"world": world, "max_rel_err": err}), flush=True)
        assert err < 1e-12, err
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
