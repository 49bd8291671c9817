"""Bounded device-side waits: when an awaited activation never arrives, the persistent decode kernel gives up
after its limit (~0.2 s), records LUMEN_ERR_TIMEOUT in the device status word and returns; the host sees the
status at its next synchronising call and the context stays usable.  The missing activation is produced by a
debug switch of the kernel (a phase that publishes nothing): nothing faults, traps or hangs."""
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]

CHILD = textwrap.dedent("""
    import sys, time
    import numpy as np
    sys.path.insert(0, %r)
    sys.path.insert(0, %r)
    import lumen_b200 as L
    from helpers import small_cfg, make_params
    cfg = small_cfg()
    model = L.LlamaModel(L.LlamaConfig(**cfg))
    model.load_state(make_params(L, cfg, 5, std=0.08))
    ids = np.arange(8, dtype=np.float32)[None] %% cfg["vocab_size"]
    caches = model.init_kv_caches(1)
    with L.no_grad():
        model.forward(ids[:, :4], caches)                 # prefill: per-operator kernels, unaffected
        t0 = time.perf_counter()
        try:
            model.forward(ids[:, 4:5], caches)            # decode: persistent kernel, first phase stays silent
            print("NO_ERROR")
        except L.LumenError as e:
            print("ERROR", e.code, round(time.perf_counter() - t0, 2))
        # the step that gave up appended nothing: the cache length the host reports is the device's (4), not
        # the value the host had bumped when it enqueued the step
        print("LEN_AFTER", caches[0].len, caches[-1].len)
        # the context is still usable: operators and a fresh prefill run and give finite results
        a = L.Tensor.from_array_no_grad(np.ones((3, 16), np.float32))
        w = L.Tensor.from_array_no_grad(np.ones((5, 16), np.float32))
        print("MATMUL", float(L.matmul(a, w).data().sum()))
        model.reset_kv_caches(caches)
        print("PREFILL_FINITE", bool(np.isfinite(model.forward(ids[:, :4], caches)).all()))
""")


def test_unanswered_wait_times_out_and_context_survives():
    env = dict(os.environ, LUMEN_MEGA_DEBUG="8")
    code = CHILD % (str(ROOT), str(ROOT / "tests"))
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=180)
    assert r.returncode == 0, r.stdout + r.stderr
    lines = dict(l.split(" ", 1) for l in r.stdout.strip().splitlines() if " " in l)
    assert "ERROR" in lines, r.stdout
    code_s, secs = lines["ERROR"].split()
    assert int(code_s) == 9            # LUMEN_ERR_TIMEOUT
    assert float(secs) < 5.0           # a bounded wait, not a hang
    assert lines["LEN_AFTER"].split() == ["4", "4"]
    assert float(lines["MATMUL"]) == 3 * 5 * 16.0
    assert lines["PREFILL_FINITE"] == "True"
