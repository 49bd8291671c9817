"""Chat-loop behaviours around the kept KV cache (src/main.rs:214-382): control flow on CPU with a stub model,
and on a GPU the device-sampling session against the reference's flow (host logits + the oracle's sampler)."""
import numpy as np
import pytest

from helpers import small_cfg, make_params


class _Cache:
    def __init__(self):
        self.len = 0


class _Cfg:
    max_seq_len = 40


class _StubModel:
    """Counts what is fed; emits a fixed token stream."""
    config = _Cfg()

    def __init__(self, stream):
        self.stream, self.calls = list(stream), []
        self.c = [_Cache()]

    def init_kv_caches(self, b):
        return self.c

    def reset_kv_caches(self, caches):
        self.calls.append(("reset",))
        caches[0].len = 0

    def forward(self, ids, caches, pos, last_only=False):
        caches[0].len += ids.shape[1]
        self.calls.append(("forward", ids.shape[1]))

    def forward_sample(self, ids, caches, t, p, rp, recent, u):
        caches[0].len += ids.shape[1]
        self.calls.append(("sample", ids.shape[1], len(recent)))
        return self.stream.pop(0)


def test_incremental_prefill_stop_tokens_and_auto_reset():
    from lumen_b200.chat import ChatSession
    m = _StubModel([5, 6, 99] + list(range(100, 200)))
    s = ChatSession(m, encode_first=lambda u: [1, 2, 3] + list(u), encode_next=lambda u: [4] + list(u), stop_ids=[99, 99, 2],
                    max_gen=50, recent_window=4)
    assert m.calls == [("reset",)]
    # turn 1: first-turn prompt (3 + 2 tokens) is prefilled, two tokens generated, 99 stops
    assert s.turn([40, 41]) == [5, 6]
    assert m.calls[1:] == [("sample", 5, 4), ("sample", 1, 4), ("sample", 1, 4)]
    assert m.c[0].len == 7 and s.all_tokens == [1, 2, 3, 40, 41, 5, 6]
    # turn 2: only the new chunk (1 + 1 tokens) goes through the model; the hard stop ends it at len + 2 >= 40
    m.calls.clear()
    out = s.turn([42])
    assert m.calls[0] == ("sample", 2, 4)
    assert m.c[0].len + 2 >= 40 and len(out) == 40 - 2 - 9
    # turn 3: the context cannot take the next chunk -> reset, rebuilt as a first turn, and no hard stop in that branch
    m.calls.clear()
    m.stream = [50, 99]
    assert s.turn([43]) == [50]
    assert m.calls[0] == ("reset",) and m.calls[1] == ("sample", 4, 4)
    assert s.all_tokens == [1, 2, 3, 43, 50] and s.first_turn is False
    # max_gen: the last step's logits are never sampled
    m.calls.clear()
    m.stream = [60, 61, 62, 63]
    s.max_gen = 3
    assert s.turn([44]) == [60, 61, 62]
    assert m.calls[-1] == ("forward", 1)
    # text markers stop generation after the token is kept (main.rs:301-305)
    s.reset()
    m.stream = [70, 71, 72]
    s.text_stop = lambda gen: gen[-1] == 71
    assert s.turn([45]) == [70, 71]


@pytest.mark.gpu
def test_session_matches_reference_flow(L, oracle):
    from lumen_b200.chat import ChatSession
    cfg = small_cfg(max_seq_len=64)
    params = make_params(L, cfg, 19, std=0.3)
    m1, m2 = (L.LlamaModel(L.LlamaConfig(**cfg)) for _ in range(2))
    m1.load_state(params)
    m2.load_state(params)
    enc_first = lambda u: [1, 2] + list(u)
    enc_next = lambda u: [3] + list(u)
    stop = [0]
    us = np.random.default_rng(5).random(400)
    it = iter(us)
    s = ChatSession(m1, enc_first, enc_next, stop_ids=stop, max_gen=12, uniform=lambda: next(it))
    got = [s.turn([10, 11]), s.turn([12]), s.turn([13, 14, 15])]

    # the reference's flow: logits to the host, sampler on the host (main.rs:324-376)
    it2 = iter(us)
    caches = m2.init_kv_caches(1)
    all_tokens, want, first = [], [], True
    with L.no_grad():
        for msg in ([10, 11], [12], [13, 14, 15]):
            new = (enc_first if first else enc_next)(msg)
            assert caches[0].len + len(new) + 8 < cfg["max_seq_len"]
            all_tokens += new
            start = len(all_tokens)
            logits = m2.forward(np.asarray(new, np.float32)[None], caches)[0, -1]
            for _ in range(12):
                nxt = oracle.sample_top_p(logits, 0.8, 0.9, 1.05, all_tokens[-96:], float(next(it2)))
                if nxt in stop:
                    break
                all_tokens.append(nxt)
                logits = m2.forward(np.asarray([[nxt]], np.float32), caches)[0, -1]
                if caches[0].len + 2 >= cfg["max_seq_len"]:
                    break
            want.append(all_tokens[start:])
            first = False
    assert got == want
    assert s.kv_caches[0].len == caches[0].len
