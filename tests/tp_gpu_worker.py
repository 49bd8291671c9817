"""One rank of the multi-GPU tensor-parallel parity check (launched by test_tp_gpu.py, one process per GPU).
The NCCL id travels over a gloo group; rank 0 compares the gathered logits with the CPU oracle."""
import json
import os
import sys
from pathlib import Path

import numpy as np
import torch.distributed as dist

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def main():
    cfg = json.loads(os.environ["TP_TEST_CFG"])
    wdt = os.environ.get("TP_TEST_DTYPE", "f32")
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{os.environ['MASTER_PORT']}", rank=rank, world_size=world)
    import lumen_b200 as L
    from lumen_b200 import synth

    box = [L.Context.nccl_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    ctx = L.Context(rank, rank, world, box[0])
    lcfg = L.LlamaConfig(**cfg, weight_dtype=wdt)
    model = L.LlamaModel(lcfg, ctx)
    params = {n: w for n, w in synth.iter_params(lcfg, 3, std=0.05, round_bf16=(wdt == "bf16"))}
    for n, w in params.items():
        model.set_param(n, w)  # every rank passes the full tensor; the library keeps its slice
    prompt, steps = int(os.environ.get("TP_TEST_PROMPT", "7")), 6
    batch = int(os.environ.get("TP_TEST_BATCH", "1"))
    ids = synth.token_ids(5, batch * (prompt + steps), cfg["vocab_size"]).reshape(batch, prompt + steps)
    caches = model.init_kv_caches(batch)
    got = []
    with L.no_grad():
        got.append(model.forward(ids[:, :prompt], caches)[:, -1])
        for t in range(steps):
            got.append(model.forward(ids[:, prompt + t:prompt + t + 1], caches)[:, 0])
    got = np.stack(got)  # [1 + steps, batch, vocab]
    ctx.synchronize()
    if rank == 0:
        from oracle import binding as O
        O.build()
        om = O.Llama(cfg, params, "f64")
        oc = om.init_kv_caches(batch)
        want = [om.forward(ids[:, :prompt], oc)[:, -1]]
        for t in range(steps):
            want.append(om.forward(ids[:, prompt + t:prompt + t + 1], oc)[:, 0])
        want = np.stack(want)
        errs = [float(np.abs(g - w).max() / np.abs(w).max()) for g, w in zip(got.reshape(-1, got.shape[-1]), want.reshape(-1, want.shape[-1]))]
        print(json.dumps({"world": world, "max_rel_err": max(errs),
                          "argmax_equal": bool((got.argmax(-1) == want.argmax(-1)).all())}), flush=True)
    dist.barrier()
    del model, caches
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
