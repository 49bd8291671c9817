"""Nucleus sampling: the oracle's restatement of `sample_top_p` (src/main.rs:74-137) on CPU, and the device
sampler against it on a GPU (same token for the same uniform draw)."""
import numpy as np
import pytest

from helpers import small_cfg, make_params


def test_oracle_sampler_properties(oracle):
    rng = np.random.default_rng(0)
    lg = (rng.standard_normal(500) * 3).astype(np.float32)
    top = int(lg.argmax())
    # a vanishing nucleus or temperature is greedy
    assert oracle.sample_top_p(lg, 1.0, 0.0, 1.0, [], 0.7) == top
    assert oracle.sample_top_p(lg, 1e-9, 0.9, 1.0, [], 0.3) == top
    # r = 0 always returns the most probable token, r -> 1 the last token of the nucleus
    assert oracle.sample_top_p(lg, 0.8, 0.9, 1.0, [], 0.0) == top
    p = np.exp((lg / np.float32(0.8)).astype(np.float64))
    p /= p.sum()
    order = np.argsort(-p, kind="stable")
    cut = int(np.searchsorted(np.cumsum(p[order]), 0.9) + 1)
    assert oracle.sample_top_p(lg, 0.8, 0.9, 1.0, [], 0.999999) in set(order[max(0, cut - 2):cut + 1].tolist())
    # a penalty > 1 divides once per occurrence: enough of them dethrone the top token
    assert oracle.sample_top_p(lg, 1.0, 0.0, 4.0, [top] * 6, 0.5) != top
    assert oracle.sample_top_p(lg, 1.0, 0.0, 1.0, [top] * 6, 0.5) == top   # penalty 1.0 is off
    # empirical frequencies follow the renormalised nucleus
    draws = [oracle.sample_top_p(lg, 0.8, 0.5, 1.0, [], float(u)) for u in rng.random(4000)]
    cut5 = int(np.searchsorted(np.cumsum(p[order]), 0.5) + 1)
    assert set(draws) <= set(order[:cut5].tolist())
    freq = np.bincount(draws, minlength=lg.size) / len(draws)
    want = np.zeros_like(p)
    want[order[:cut5]] = p[order[:cut5]] / p[order[:cut5]].sum()
    assert np.abs(freq - want).max() < 0.03


@pytest.mark.gpu
@pytest.mark.parametrize("vocab,scale", [(97, 3.0), (32000, 4.0), (32000, 0.05), (151936, 6.0)])
def test_device_sampler_matches_oracle(L, ctx, oracle, vocab, scale):
    rng = np.random.default_rng(vocab)
    lg = (rng.standard_normal(vocab) * scale).astype(np.float32)
    lg[5] = lg[6]  # a tie: the stable sort keeps index order
    t = L.Tensor.from_array_no_grad(lg)
    recent = rng.integers(0, vocab, size=40).tolist() + [int(lg.argmax())] * 3
    mismatches = 0
    cases = [(0.8, 0.9, 1.1, recent), (1.0, 0.5, 1.0, []), (0.3, 0.95, 1.3, recent[:7]), (1.0, 0.0, 1.0, []), (1.5, 1.0, 1.0, [])]
    for temp, top_p, pen, rec in cases:
        for u in rng.random(12).astype(np.float32):
            got = L.sample_top_p(ctx, t.data_ptr, vocab, temp, top_p, pen, rec, float(u))
            want = oracle.sample_top_p(lg, temp, top_p, pen, rec, float(u))
            mismatches += int(got != want)
    # the softmax denominator is a tree sum on the device and a sequential sum in the reference: a draw that sits
    # within an ulp of a boundary may fall on the other side
    assert mismatches <= 1, mismatches


@pytest.mark.gpu
def test_forward_sample_equals_forward_then_oracle_sampler(L, oracle):
    cfg = small_cfg()
    params = make_params(L, cfg, 17, std=0.3)
    m1, m2 = (L.LlamaModel(L.LlamaConfig(**cfg)) for _ in range(2))
    m1.load_state(params)
    m2.load_state(params)
    c1, c2 = m1.init_kv_caches(1), m2.init_kv_caches(1)
    rng = np.random.default_rng(3)
    toks = [3, 9, 27, 11]
    with L.no_grad():
        ids = np.asarray(toks, np.float32)[None]
        for step in range(10):
            u = float(rng.random())
            logits = m1.forward(ids, c1)[0, -1]
            want = oracle.sample_top_p(logits, 0.8, 0.9, 1.1, toks[-96:], u)
            got = m2.forward_sample(ids, c2, 0.8, 0.9, 1.1, toks[-96:], u)
            assert got == want, step
            toks.append(got)
            ids = np.asarray([[got]], np.float32)   # generated token fed back, as main.rs:367-372
    assert c1[0].len == c2[0].len == 4 + 9
