#!/usr/bin/env python
"""Benchmark of the Llama decode hot path: decode tokens/s, TinyLlama-1.1B shape, batch 1.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--dtype f32|bf16] [--impl lumen|reference]

One "step" is one teacher-forced decode token (one pass over all the weights).  Synthetic data:
weights N(0, 0.02) from seed 0 with RMSNorm gains 1.0, a 32-token prompt and the forced ids from
seed 1 (benchmark configuration 1); the static KV cache is sized to max_seq_len 2048.

Own arm (default): prints ONE JSON line with
  value     device-resident throughput (ids and logits stay in HBM), CUDA events on the library's stream
  e2e       the same metric through the public host API: per step the token id is copied host->device
            and the logits [vocab] device->host, inside the timed region
  roofline  algorithmic HBM bytes per step / measured step time against the measured copy bandwidth
  cpu_baseline  the CPU restatement of the reference's Rayon path, timed on this box's host cores on a
            bounded sample of the same workload (rank 0, N = 1 only)
With N > 1 (launched by torchrun, one rank per GPU) the model is tensor-parallel over the N GPUs; the all-reduce after
the o/down projections and the gather of the logits happen inside the persistent kernel over NVLink peer stores
("scaling": "strong": the work per token is fixed).  Rank 0 also compares its logits with the CPU restatement
(`parity_vs_cpu`) and the line carries a short Llama-2-7B run (`extra`).  The timed region is exactly --steps steps; it
is repeated (fresh prompt and warm-up each time) and the median repetition is reported, with the spread beside it.

Reference arm (--impl reference): the reference is Rust and cannot be built on this box, so the arm
times its CPU restatement (oracle/) with all host threads on the same workload and prints the same
line with "impl": "reference".  It loads neither the package nor the CUDA library.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

PROMPT_LEN = 32
METRIC = "decode_tokens_per_s"
UNIT = "tokens/s"
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0


def measured_hbm_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) every few ms."""

    def __init__(self, index: int, period_s: float = 0.004):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._halt = threading.Event()
        self.active = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
            "hw_power_brake": getattr(nv, "nvmlClocksThrottleReasonHwPowerBrakeSlowdown", 0x80),
        }
        while not self._halt.is_set():
            if self.active:
                try:
                    self.samples.append(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                    self.reasons.update(n for n, bit in names.items() if r & bit)
                except Exception:
                    pass
            time.sleep(self.period)

    def stop(self):
        self._halt.set()

    def summary(self):
        return {"sm_mhz": (statistics.median(self.samples) if self.samples else None), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# dram__bytes_read + dram__bytes_write of one persistent-kernel launch divided by its algorithmic bytes,
# from an ncu capture of a 4-layer truncation of the same model (973.0 MB / 967.3 MB; f32 weights, one GPU); its
# summary is committed with the other profiler summaries.
MEGA_TRAFFIC_RATIO = 1.0058


WORKLOADS = {  # name -> (synth config, label, default weight dtype)
    "tinyllama": ("TINYLLAMA", "tinyllama_1.1b", "f32"),    # configuration 1: the one the metric is quoted on
    "llama2_7b": ("LLAMA2_7B", "llama2_7b", "bf16"),        # configuration 4's shape (tensor-parallel scaling)
    "qwen3_8b": ("QWEN3_8B", "qwen3_8b", "bf16"),           # configuration 5's shape
}


def load_synth():
    """The seeded generators (lumen_b200/synth.py, numpy only) loaded by file path: the CPU arm must not import
    the package, whose import loads the CUDA library."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("_lumen_synth", ROOT / "lumen_b200" / "synth.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def tinyllama_cfg(dtype: str, max_seq: int, layers: int = 0, workload: str = "tinyllama"):
    synth = load_synth()
    cfg = dict(getattr(synth, WORKLOADS[workload][0]))
    cfg["max_seq_len"] = max_seq
    if layers:
        cfg["num_hidden_layers"] = layers
    return cfg


def gen_params(cfg: dict, dtype: str, workload: str = "tinyllama"):
    synth = load_synth()
    gen = synth.iter_params if workload == "tinyllama" else synth.iter_params_tiled
    return gen(cfg, 0, std=0.02, round_bf16=(dtype == "bf16"))


def stream_bytes(cfg: dict, dtype: str, tp: int = 1) -> int:
    """Weight bytes one decode step reads on one rank (the embedding contributes one row per token, not counted)."""
    e = 2 if dtype == "bf16" else 4
    h, i, v, l = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    d = cfg.get("head_dim") or h // cfg["num_attention_heads"]
    hq, hkv = cfg["num_attention_heads"] // tp, max(1, cfg["num_key_value_heads"] // tp)
    qkv_rows = (hq + 2 * hkv) * d
    per_layer = (qkv_rows * h + h * hq * d + 3 * (i // tp) * h) * e + 2 * h * 4 + (2 * d * 4 if cfg.get("qk_norm") else 0)
    return l * per_layer + h * 4 + (v // tp) * h * e


def make_config(args, workload: str, dtype: str, batch: int, max_seq: int, world: int, cfg: dict) -> dict:
    """The `config` object of the JSON line: the same for the GPU arm and the CPU arm."""
    return {"workload": f"{WORKLOADS[workload][1]}_{dtype}_batch{batch}_decode", "weights": dtype, "batch": batch,
            "prompt_len": PROMPT_LEN, "max_seq_len": max_seq, "parallelism": f"tp{world}",
            "l2": "inputs larger than L2: every step streams %.2f GB of weights per GPU" % (stream_bytes(cfg, dtype, world) / 1e9)}


def algorithmic_bytes_per_step(cfg: dict, weight_bytes: int, ctx_len_mean: float, tp: int, batch: int = 1) -> float:
    """Weights of this rank once + per sequence: K/V rows of the context once per KV head, the embedding row, logits."""
    d = cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]
    hkv_local = max(1, cfg["num_key_value_heads"] // tp)
    kv = cfg["num_hidden_layers"] * 2 * hkv_local * d * 4 * (ctx_len_mean + 1)
    return weight_bytes + batch * (kv + cfg["hidden_size"] * 4 + cfg["vocab_size"] * 4 / tp)


def cpu_decode(cfg: dict, params: dict, ids: np.ndarray, budget_s: float, max_steps: int, warmup: int = 0):
    """Times the CPU restatement on a bounded sample: full prompt prefill and `warmup` untimed decode steps, then
    decode steps until `max_steps` or the budget is reached.  Every host core is used whatever OMP_NUM_THREADS says
    (launchers such as torchrun set it to 1).  Returns (tokens/s over the timed steps, timed steps, threads,
    logits of the warm-up and timed steps)."""
    from oracle import binding as O
    threads = O.set_num_threads()
    model = O.Llama(cfg, params, "f32")
    caches = model.init_kv_caches(1)
    model.forward(ids[None, :PROMPT_LEN], caches)
    logits = []
    pos = PROMPT_LEN
    for _ in range(warmup):
        logits.append(model.forward(ids[None, pos:pos + 1], caches)[0, 0])
        pos += 1
    t0 = time.perf_counter()
    steps = 0
    while steps < max_steps:
        logits.append(model.forward(ids[None, pos:pos + 1], caches)[0, 0])
        pos += 1
        steps += 1
        if time.perf_counter() - t0 > budget_s:
            break
    dt = time.perf_counter() - t0
    return steps / dt, steps, threads, np.stack(logits)


def run_reference(args):
    """--impl reference: the reference's CPU path (restated in C; the Rust crate cannot be built here) on all host
    cores: the same prompt, `--warmup` untimed and `--steps` timed teacher-forced decode steps (bounded by a time
    budget).  Loads neither the package nor the CUDA library."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    cfg = tinyllama_cfg(args.dtype, 2048)
    params = dict(gen_params(cfg, args.dtype))
    ids = load_synth().token_ids(1, PROMPT_LEN + args.warmup + args.steps + 1, cfg["vocab_size"])
    budget = 120.0
    tps, steps, threads, _ = cpu_decode(cfg, params, ids, budget, max(1, args.steps), args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": args.warmup, "ms_per_step": 1000.0 / tps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": make_config(args, "tinyllama", args.dtype, 1, 2048, args.gpus, cfg),
        "note": "the Rust reference cannot be built here (no rustc): this times its C/OpenMP restatement on the host cores",
        "cpu_baseline": {"value": tps, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"{PROMPT_LEN}-token prefill and {args.warmup} warm-up steps (untimed) + {steps} decode steps, "
                                   f"<= {budget:.0f} s"},
        "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


GEMV_SWEEP = [(2048, 2048), (2048, 256), (2048, 5632), (5632, 2048), (2048, 32000), (4096, 11008), (11008, 4096)]
GEMM_SWEEP = [(32, 2048, 5632), (512, 4096, 4096), (512, 4096, 11008), (512, 11008, 4096), (4096, 4096, 12288), (4096, 4096, 4096)]
ATTN_SWEEP = [(1, 128), (1, 512), (1, 2048), (1, 8192), (16, 128), (16, 512), (16, 2048), (16, 8192)]


def _event_time_ms(ctx, stream, fn, iters: int, warm: int = 3) -> float:
    import torch
    for _ in range(warm):
        fn()
    ctx.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(iters):
        fn()
    e1.record(stream)
    ctx.synchronize()
    return e0.elapsed_time(e1) / iters


def run_micro(args):
    """Secondary measurements (benchmark configurations 2 and 3): the standalone vector-matrix product over the
    sweep of shapes, and decode attention over a static KV cache.  One JSON line per case; the working set
    is rotated over several copies so that it exceeds L2 whenever that takes at most 64 copies."""
    import torch
    import lumen_b200 as L
    torch.cuda.set_device(0)
    ctx = L.Context(0)
    stream = torch.cuda.ExternalStream(ctx.stream, device=torch.device("cuda", 0))
    peak, peak_kind = measured_hbm_peak()
    rng = np.random.default_rng(2)
    if args.micro == "gemv":
        for k, n in GEMV_SWEEP:
            x = L.Tensor.from_array_no_grad(rng.standard_normal(k, dtype=np.float32), ctx)
            y = L.Tensor.from_array_no_grad(np.zeros(n, np.float32), ctx)
            w_nk = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)
            for dt in ("f32", "bf16"):
                esz = 4 if dt == "f32" else 2
                copies = int(min(64, max(2, -(-300e6 // (k * n * esz)))))
                for layout in ("nk", "kn"):
                    w_host = w_nk if layout == "nk" else np.ascontiguousarray(w_nk.T)
                    ws = [(L.Tensor.from_bf16(w_host, ctx) if dt == "bf16" else L.Tensor.from_array_no_grad(w_host, ctx))
                          for _ in range(copies)]
                    # back-to-back calls from compiled code between two CUDA events (no per-call host cost in the number)
                    us = L.gemv_repeat(ctx, x.data_ptr, [w.data_ptr for w in ws], L.BF16 if dt == "bf16" else L.F32, layout == "kn", k, n,
                                       y.data_ptr, max(50, 3 * copies))
                    ms = us / 1000.0
                    nbytes = esz * k * n + 4 * k + 4 * n
                    gbs = nbytes / (ms * 1e-3) / 1e9
                    print(json.dumps({"micro": "gemv", "k": k, "n": n, "weights": dt, "layout": layout, "us": ms * 1e3,
                                      "algorithmic_bytes": nbytes, "gbs": gbs, "frac_of_measured_peak": gbs / peak,
                                      "peak_kind": peak_kind, "working_set_mb": copies * k * n * esz / 1e6}), flush=True)
                    del ws
    elif args.micro == "gemm":
        # M > 8 branch of matmul with bf16 weights (prefill / batched decode): tensor-core roofline
        try:
            tpeak = float(json.loads((ROOT / "MEASURED_PEAKS.json").read_text())["bf16_tflops"])
            tkind = "measured"
        except Exception:
            tpeak, tkind = 1590.0, "fallback"
        for m, k, n in GEMM_SWEEP:
            a = L.Tensor.from_array_no_grad(rng.standard_normal((m, k), dtype=np.float32), ctx)
            w = L.Tensor.from_bf16(rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02), ctx)
            keep = []

            def step():
                keep.append(L.matmul(a, w))
                if len(keep) > 4:
                    keep.pop(0)

            ms = _event_time_ms(ctx, stream, step, iters=20)
            tf = 2.0 * m * k * n / (ms * 1e-3) / 1e12
            print(json.dumps({"micro": "gemm_bf16_weights", "m": m, "k": k, "n": n, "us": ms * 1e3, "tflops": tf,
                              "frac_of_peak": tf / tpeak, "peak_tflops": tpeak, "peak_kind": tkind,
                              "note": "algorithmic flops 2*M*K*N; the kernel issues twice that (activations as hi+lo bf16)"}),
                  flush=True)
            del keep
    elif args.micro == "prefill":
        # SelfAttention::forward over a whole prompt at the Qwen3-8B / Llama-7B attention geometry (32 query heads of
        # 128, 8 KV heads, f32 weights): four projections on the tensor-core GEMM + the tensor-core prefill attention.
        # The time is the whole forward; per-kernel times are in the profiler launch list of this command.
        e, hq, hkv = 4096, 32, 8
        d = e // hq
        ws = [L.Tensor.from_array_no_grad(rng.standard_normal(sh, dtype=np.float32) * np.float32(e ** -0.5), ctx)
              for sh in ((e, e), (hkv * d, e), (hkv * d, e), (e, e))]
        for b, s_len in ((1, 512), (1, 2048), (2, 4096)):
            attn = L.SelfAttention(e, hq, hkv, s_len + 8, 1e6, True, ctx)
            attn.set_weights(*ws)
            x = L.Tensor.from_array_no_grad(rng.standard_normal((b, s_len, e), dtype=np.float32), ctx)
            with L.no_grad():
                _, cache = attn.forward(x, None)
                state = {}

                def step():
                    cache.reset()
                    state["out"] = attn.forward(x, cache)[0]

                ms = _event_time_ms(ctx, stream, step, iters=5)
            attn_flops = b * hq * s_len * (s_len + 1) / 2 * 4 * d
            proj_flops = 2.0 * b * s_len * e * (2 * e + 2 * hkv * d)
            print(json.dumps({"micro": "self_attention_prefill", "batch": b, "positions": s_len, "heads": hq, "kv_heads": hkv,
                              "head_dim": d, "ms": ms, "attention_gflop": attn_flops / 1e9, "projection_gflop": proj_flops / 1e9,
                              "tflops_whole_forward": (attn_flops + proj_flops) / (ms * 1e-3) / 1e12,
                              "note": "algorithmic flops (causal half for the attention); f32 operands go through the tensor "
                                      "cores as hi/lo bf16 pairs, three products per term"}), flush=True)
            del attn, x, cache
    else:
        # configuration 3's geometry over its sweep, then the Qwen3-8B geometry (32 query heads of 128, 8 KV heads) at the
        # context of configuration 5
        cases = [(32, 4, 64, b, n) for b, n in ATTN_SWEEP] + [(32, 8, 128, 16, 4096), (32, 8, 128, 64, 4096)]
        for hq, hkv, d, b, ctx_len in cases:
            iters = 50
            kv_bytes = b * hkv * ctx_len * d * 4 * 2
            copies = int(min(16, max(1, -(-300e6 // kv_bytes))))
            max_seq = ctx_len + iters + 8  # every call appends a row to the cache it uses
            rope = L.RotaryEmbedding(d, max_seq, 10000.0, ctx)
            caches = []
            for _ in range(copies):
                c = L.KVCacheInner(b, hkv, max_seq, d, ctx)
                kk = rng.standard_normal((b, hkv, max_seq, d), dtype=np.float32)
                vv = rng.standard_normal((b, hkv, max_seq, d), dtype=np.float32)
                c.write(kk, vv, ctx_len)
                caches.append(c)
            q = L.Tensor.from_array_no_grad(rng.standard_normal((b, hq, d), dtype=np.float32), ctx)
            kn = L.Tensor.from_array_no_grad(rng.standard_normal((b, hkv, d), dtype=np.float32), ctx)
            vn = L.Tensor.from_array_no_grad(rng.standard_normal((b, hkv, d), dtype=np.float32), ctx)
            out = L.Tensor.from_array_no_grad(np.zeros((b, hq, d), np.float32), ctx)
            us = L.attention_decode_repeat(ctx, q.data_ptr, kn.data_ptr, vn.data_ptr, hq, caches, rope, out.data_ptr, iters)
            ms = us / 1000.0
            nbytes = kv_bytes + b * hq * d * 8 + b * hkv * d * 8
            gbs = nbytes / (ms * 1e-3) / 1e9
            print(json.dumps({"micro": "attention_decode", "heads": hq, "kv_heads": hkv, "head_dim": d, "batch": b, "context": ctx_len, "us": ms * 1e3,
                              "algorithmic_bytes": nbytes, "gbs": gbs, "frac_of_measured_peak": gbs / peak,
                              "peak_kind": peak_kind, "working_set_mb": copies * kv_bytes / 1e6}), flush=True)
            del caches
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--dtype", choices=["f32", "bf16"], default=None, help="weight storage (default: the workload's)")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="tinyllama",
                    help="model shape; the default is the configuration the metric is quoted on")
    ap.add_argument("--impl", choices=["lumen", "reference"], default="lumen")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-budget-s", type=float, default=12.0)
    ap.add_argument("--profile-layers", type=int, default=0,
                    help="profiling aid: truncate the model to this many layers so that a profiler capture stays "
                         "small; the printed line is then marked and is not a benchmark value")
    ap.add_argument("--micro", choices=["gemv", "attn", "gemm", "prefill"], default=None,
                    help="secondary measurements instead of the decode benchmark: the vector-matrix sweep or "
                         "decode attention over a static cache (one JSON line per case)")
    ap.add_argument("--batch", type=int, default=1,
                    help="independent sequences decoded per step (1 is the metric's configuration; larger batches run the "
                         "per-operator kernels: tensor-core GEMMs and the tiled attention kernel)")
    ap.add_argument("--prompt-len", type=int, default=32,
                    help="tokens of the (untimed) prefill; 32 is the metric's configuration, 512 configuration 4's")
    ap.add_argument("--repeats", type=int, default=0,
                    help="repetitions of the timed K-step region (0: as many as make the timed regions add up to ~0.5 s, 3..25)")
    ap.add_argument("--no-extra", action="store_true", help="N > 1: skip the short Llama-2-7B run reported beside the headline")
    ap.add_argument("--prefill-chunk", type=int, default=0,
                    help="prefill the prompt in slices of this many positions (0: one forward)")
    args = ap.parse_args()
    global PROMPT_LEN
    PROMPT_LEN = args.prompt_len
    args.warmup = max(args.warmup, 3)
    if args.dtype is None:
        args.dtype = WORKLOADS[args.workload][2]
    if args.micro:
        return run_micro(args)
    if args.impl == "reference":
        return run_reference(args)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torchrun (one rank per GPU)")
    import torch
    import torch.distributed as dist

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    import lumen_b200 as L
    from lumen_b200 import synth

    total = PROMPT_LEN + args.warmup + args.steps
    max_seq = 2048
    if total > max_seq:
        if args.workload == "tinyllama":
            raise SystemExit(f"prompt + warmup + steps = {total} exceeds max_seq_len {max_seq}")
        max_seq = (total + 1 + 255) // 256 * 256  # long prefixes (configuration 5: 4096 + 128 steps)
    cfg = tinyllama_cfg(args.dtype, max_seq, args.profile_layers, args.workload)
    big = args.workload != "tinyllama"

    nccl_id = None
    if world > 1:
        box = [L.Context.nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        nccl_id = box[0]
    ctx = L.Context(local_rank, rank, world, nccl_id)
    model = L.LlamaModel(L.LlamaConfig(**cfg, weight_dtype=args.dtype), ctx)
    B = max(1, args.batch)
    keep_params = (rank == 0 and not args.no_cpu_baseline and not big and B == 1 and not args.profile_layers)
    params = {}
    for name, w in gen_params(cfg, args.dtype, args.workload):
        model.set_param(name, w)
        if keep_params:
            params[name] = w
    # step-major ids [total + 1, B]: the B ids of one step are contiguous (B == 1: the plain stream)
    ids_all = synth.token_ids(1, (total + 1) * B, cfg["vocab_size"]).reshape(total + 1, B)
    ids = ids_all[:, 0].copy()
    weight_bytes = model.weight_bytes_per_step
    stream = torch.cuda.ExternalStream(ctx.stream, device=torch.device("cuda", local_rank))
    sampler = ClockSampler(local_rank)
    sampler.start()

    def barrier():
        ctx.synchronize()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    caches = model.init_kv_caches(B)
    d_ids = L.Tensor.from_array_no_grad(ids_all, ctx)
    d_logits = L.Tensor.from_array_no_grad(np.zeros(B * cfg["vocab_size"], np.float32), ctx)

    prefill_ms = []

    def prefill():
        # long prompts go through in slices of positions (each a prefill into the partly filled cache) so that
        # the activations of B x slice rows stay a few GB
        model.reset_kv_caches(caches)
        step = args.prefill_chunk if args.prefill_chunk > 0 else PROMPT_LEN
        ctx.synchronize()
        t0 = time.perf_counter()
        with L.no_grad():
            for c0 in range(0, PROMPT_LEN, step):
                model.forward(np.ascontiguousarray(ids_all[c0:min(PROMPT_LEN, c0 + step)].T), caches, 0, last_only=True)
        ctx.synchronize()
        prefill_ms.append((time.perf_counter() - t0) * 1000.0)

    # The timed region is exactly K steps; it is repeated R times (fresh prompt prefill and W untimed warm-up steps
    # before each repetition, so every repetition covers the same context lengths) and the median repetition is the
    # value.  R is chosen from the first repetition so that the timed regions add up to about half a second.
    def repeat_count(first_ms: float) -> int:
        if args.repeats > 0:
            return args.repeats
        r = int(np.ceil(500.0 / max(first_ms, 1e-3)))
        return max(3, min(25, r))

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches = 0

    def timed_device_steps() -> float:
        nonlocal launches
        prefill()
        pos = PROMPT_LEN
        for _ in range(args.warmup):
            model.forward_device(d_ids.data_ptr + 4 * B * pos, B, 1, caches, d_logits.data_ptr)
            pos += 1
        barrier()
        launches0 = ctx.launch_count
        sampler.active = True
        e0.record(stream)
        for _ in range(args.steps):
            model.forward_device(d_ids.data_ptr + 4 * B * pos, B, 1, caches, d_logits.data_ptr)
            pos += 1
        e1.record(stream)
        barrier()
        sampler.active = False
        launches = ctx.launch_count - launches0
        return max_over_ranks(e0.elapsed_time(e1))

    host_logits = []

    def timed_host_steps() -> float:
        # end to end through the host API: id in (pinned staging inside the library), logits out, every step
        prefill()
        pos = PROMPT_LEN
        for _ in range(args.warmup):
            model.forward(ids_all[pos][:, None], caches)
            pos += 1
        barrier()
        keep = not host_logits
        t0 = time.perf_counter()
        e0.record(stream)
        for _ in range(args.steps):
            lg = model.forward(ids_all[pos][:, None], caches)
            if keep and len(host_logits) < 4:
                host_logits.append(lg[0, 0].copy())
            pos += 1
        e1.record(stream)
        barrier()
        wall_ms = (time.perf_counter() - t0) * 1000.0
        return max_over_ranks(max(e0.elapsed_time(e1), wall_ms))

    with L.no_grad():
        dev_runs = [timed_device_steps()]
        for _ in range(repeat_count(dev_runs[0]) - 1):
            dev_runs.append(timed_device_steps())
        dev_ms = float(np.median(dev_runs))
        e2e_runs = [timed_host_steps()]
        for _ in range(min(len(dev_runs), repeat_count(e2e_runs[0])) - 1):
            e2e_runs.append(timed_host_steps())
        e2e_ms = float(np.median(e2e_runs))

        # ---- the same steps with the sampler on the device: only a token id comes back (single GPU) --------
        sampled_ms = None
        if world == 1 and B == 1:
            prefill()
            pos = PROMPT_LEN
            recent = [int(t) for t in ids[:PROMPT_LEN]]
            urand = np.random.default_rng(7).random(args.warmup + args.steps)
            for i in range(args.warmup):
                model.forward_sample(ids[None, pos:pos + 1], caches, 0.8, 0.9, 1.1, recent[-96:], float(urand[i]))
                pos += 1
            barrier()
            t0 = time.perf_counter()
            for i in range(args.steps):  # teacher-forced like the other loops: the sampled id is read but not fed back
                model.forward_sample(ids[None, pos:pos + 1], caches, 0.8, 0.9, 1.1, recent[-96:], float(urand[args.warmup + i]))
                pos += 1
            barrier()
            sampled_ms = (time.perf_counter() - t0) * 1000.0
    sampler.stop()

    tps = B * args.steps / (dev_ms / 1000.0)
    e2e_tps = B * args.steps / (e2e_ms / 1000.0)
    ctx_mean = PROMPT_LEN + args.warmup + (args.steps - 1) / 2.0
    bytes_step = algorithmic_bytes_per_step(cfg, weight_bytes, ctx_mean, world, B)
    peak, peak_kind = measured_hbm_peak()
    achieved = bytes_step / (dev_ms / args.steps / 1000.0) / 1e9
    mega = launches == args.steps
    # measured DRAM traffic exists for one case only: the persistent kernel, f32 weights, one GPU, the TinyLlama shape
    traffic = bytes_step * MEGA_TRAFFIC_RATIO if (mega and world == 1 and args.dtype == "f32" and args.workload == "tinyllama") else None
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": traffic,
                "peak_kind": f"of {peak_kind}", "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS,
                "kernel": ("decode_mega_kernel: one persistent launch runs the whole token" if mega else
                           "whole decode step (CUDA graph of %d kernels)" % (launches // max(args.steps, 1))),
                "algorithmic_bytes_per_step": bytes_step, "per": "GPU"}
    if traffic is not None:
        roofline["traffic_note"] = ("ncu dram bytes of a capture of the same kernel on a 4-layer truncation of the model, scaled by "
                                    "algorithmic bytes")
    line = {
        "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dev_ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": make_config(args, args.workload, args.dtype, B, max_seq, world, cfg),
        "repeats": {"n": len(dev_runs), "value": "median", "ms_per_step_min": min(dev_runs) / args.steps,
                    "ms_per_step_max": max(dev_runs) / args.steps, "timed_s": sum(dev_runs) / 1000.0,
                    "e2e_n": len(e2e_runs), "e2e_ms_per_step_min": min(e2e_runs) / args.steps,
                    "e2e_ms_per_step_max": max(e2e_runs) / args.steps},
        "e2e": {"value": e2e_tps, "unit": UNIT, "h2d_bytes_per_step": 4 * B, "d2h_bytes_per_step": 4 * B * cfg["vocab_size"],
                "ms_per_step": e2e_ms / args.steps},
        "e2e_sampled": (None if sampled_ms is None else
                        {"value": args.steps / (sampled_ms / 1000.0), "unit": UNIT, "h2d_bytes_per_step": 4 + 4 * 96,
                         "d2h_bytes_per_step": 4, "ms_per_step": sampled_ms / args.steps,
                         "note": "forward + top-p sampling on the device (temperature 0.8, top_p 0.9, repetition penalty 1.1 "
                                 "over 96 tokens): the reference samples on the host from the full logits"}),
        "gpu_launches": int(launches),
        # untimed part, for information: host wall clock of the last prefill (the first one pays the one-time set-up)
        "prefill": {"tokens": B * PROMPT_LEN, "ms": prefill_ms[-1], "tokens_per_s": B * PROMPT_LEN / (prefill_ms[-1] / 1000.0),
                    "slice": args.prefill_chunk if args.prefill_chunk > 0 else PROMPT_LEN},
        "clocks": sampler.summary(),
        "roofline": roofline,
    }
    if args.profile_layers:
        line["profile_only"] = f"model truncated to {args.profile_layers} layers: not a benchmark value"
        line["config"]["workload"] += f"_truncated_{args.profile_layers}_layers"
    if keep_params:
        # The CPU restatement on this box's host cores (rank 0).  N = 1: timed on a bounded sample, the reported baseline.
        # Every N: its logits at the first timed positions are compared with what the GPU arm returned there.
        n_cpu = max(4, min(args.steps, 256)) if world == 1 else 4
        tps_cpu, n, threads, cpu_logits = cpu_decode(cfg, params, ids, args.cpu_budget_s, n_cpu, args.warmup)
        if world == 1:
            line["cpu_baseline"] = {"value": tps_cpu, "unit": UNIT, "cores": threads, "kind": "port",
                                    "sample": f"{PROMPT_LEN}-token prefill and {args.warmup} warm-up steps (untimed) + {n} decode steps of "
                                              f"the same workload, <= {args.cpu_budget_s:.0f} s"}
        k = min(len(host_logits), n)
        if k > 0:
            errs = [float(np.abs(host_logits[i] - cpu_logits[args.warmup + i]).max() / np.abs(cpu_logits[args.warmup + i]).max())
                    for i in range(k)]
            line["parity_vs_cpu"] = {"steps_compared": k, "max_rel_err": max(errs), "tolerance": 1e-4 if args.dtype == "f32" else 1e-2,
                                     "cores": threads,
                                     "argmax_equal": all(int(host_logits[i].argmax()) == int(cpu_logits[args.warmup + i].argmax())
                                                         for i in range(k))}
    if world > 1 and not args.no_extra and args.workload == "tinyllama" and not args.profile_layers and B == 1:
        # the tensor-parallel shape the scaling claim is about, measured in the same process: Llama-2-7B, bf16 weights
        del model, caches
        extra = run_extra_7b(L, ctx, torch, dist, rank, world, local_rank)
        if extra:
            line["extra"] = extra
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


def run_extra_7b(L, ctx, torch, dist, rank, world, local_rank, prompt: int = 32, steps: int = 32, warmup: int = 4):
    """A short decode run at the Llama-2-7B shape (bf16 weights, tiled synthetic values), tensor-parallel over the
    same ranks: tokens/s, ms per step and the per-GPU fraction of the HBM peak (device-resident ids and logits)."""
    synth = load_synth()
    cfg = dict(synth.LLAMA2_7B)
    cfg["max_seq_len"] = 256
    model = L.LlamaModel(L.LlamaConfig(**cfg, weight_dtype="bf16"), ctx)
    for name, w in synth.iter_params_tiled(cfg, 0, std=0.02, round_bf16=True):
        model.set_param(name, w)
    ids = synth.token_ids(4, prompt + warmup + steps + 1, cfg["vocab_size"])
    caches = model.init_kv_caches(1)
    d_ids = L.Tensor.from_array_no_grad(ids, ctx)
    d_logits = L.Tensor.from_array_no_grad(np.zeros(cfg["vocab_size"], np.float32), ctx)
    stream = torch.cuda.ExternalStream(ctx.stream, device=torch.device("cuda", local_rank))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    runs = []
    with L.no_grad():
        for _ in range(3):
            model.reset_kv_caches(caches)
            model.forward(ids[None, :prompt], caches, 0, last_only=True)
            pos = prompt
            for _ in range(warmup):
                model.forward_device(d_ids.data_ptr + 4 * pos, 1, 1, caches, d_logits.data_ptr)
                pos += 1
            ctx.synchronize()
            dist.barrier()
            e0.record(stream)
            for _ in range(steps):
                model.forward_device(d_ids.data_ptr + 4 * pos, 1, 1, caches, d_logits.data_ptr)
                pos += 1
            e1.record(stream)
            ctx.synchronize()
            dist.barrier()
            t = torch.tensor([e0.elapsed_time(e1)], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            runs.append(float(t.item()))
    ms = float(np.median(runs))
    ctx_mean = prompt + warmup + (steps - 1) / 2.0
    bytes_step = algorithmic_bytes_per_step(cfg, model.weight_bytes_per_step, ctx_mean, world, 1)
    peak, peak_kind = measured_hbm_peak()
    gbs = bytes_step / (ms / steps / 1000.0) / 1e9
    return {"workload": f"llama2_7b_bf16_batch1_decode_tp{world}", "prompt_len": prompt, "steps": steps, "warmup": warmup,
            "value": steps / (ms / 1000.0), "unit": UNIT, "ms_per_step": ms / steps, "repeats": len(runs),
            "per_gpu_hbm_gbs": gbs, "per_gpu_frac": gbs / peak, "peak_kind": f"of {peak_kind}"}


if __name__ == "__main__":
    sys.exit(main())
