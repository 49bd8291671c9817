"""The cache-keeping behaviour of the reference's chat loop (src/main.rs:214-382) around `LlamaModel`,
without its terminal I/O and tokenizer: multi-turn generation where only the new chunk of each turn is
prefilled into the kept KV caches, automatic reset when the context is about to overflow, stop tokens, the
hard stop near `max_seq_len`, and the sliding window of recent tokens for the repetition penalty.  Sampling
runs on the device (`LlamaModel.forward_sample`), so one token id per step crosses PCIe.

The caller supplies what the tokenizer did there: `encode_first(user_msg)` and `encode_next(user_msg)` return
the token ids of a first-turn / follow-up prompt (main.rs:36-58 build the texts), and an optional
`text_stop(generated_ids)` reproduces the check for role markers in the decoded text (main.rs:301-305).
`LlamaTokenizer` (tokenizer.py, the mirror of src/tokenizer.rs) provides `encode` / `decode` / `eos_id` / `eot_id`
for these over a tokenizer.json.
"""
from __future__ import annotations

import numpy as np

from .tensor import no_grad


class ChatSession:
    def __init__(self, model, encode_first, encode_next, stop_ids=(), text_stop=None, temperature: float = 0.8,
                 top_p: float = 0.9, repetition_penalty: float = 1.05, recent_window: int = 96, max_gen: int = 200,
                 uniform=None):
        self.model = model
        self.encode_first, self.encode_next = encode_first, encode_next
        self.stop_ids = sorted(set(int(t) for t in stop_ids))                      # main.rs:200-211
        self.text_stop = text_stop
        self.temperature, self.top_p, self.repetition_penalty = temperature, top_p, repetition_penalty
        self.recent_window, self.max_gen = recent_window, max_gen
        self.uniform = uniform or np.random.default_rng().random                   # rand01(), main.rs:69-72
        self.all_tokens: list = []                                                  # main.rs:215
        self.first_turn = True
        self.kv_caches = model.init_kv_caches(1)                                    # main.rs:219-221
        model.reset_kv_caches(self.kv_caches)

    def reset(self) -> None:                                                        # "/reset", main.rs:243-249
        self.all_tokens.clear()
        self.model.reset_kv_caches(self.kv_caches)
        self.first_turn = True

    def _recent(self):
        return self.all_tokens[max(0, len(self.all_tokens) - self.recent_window):]

    def _step(self, ids, sample: bool = True):
        """forward on `ids` ([1,S]) and, unless this is the step whose logits nobody reads, the next token."""
        a = np.asarray(ids, dtype=np.float32)[None]
        if not sample:
            self.model.forward(a, self.kv_caches, 0, last_only=True)
            return None
        return self.model.forward_sample(a, self.kv_caches, self.temperature, self.top_p, self.repetition_penalty,
                                         self._recent(), float(self.uniform()))

    def turn(self, user_msg) -> list:
        """One exchange; returns the generated token ids (stop token excluded)."""
        max_seq = self.model.config.max_seq_len
        with no_grad():
            new_tokens = list(self.encode_first(user_msg) if self.first_turn else self.encode_next(user_msg))
            cur_len = self.kv_caches[0].len
            hard_stop = True
            if cur_len + len(new_tokens) + 8 >= max_seq:                            # main.rs:270-276: auto reset
                self.reset()
                new_tokens = list(self.encode_first(user_msg))
                hard_stop = False                                                   # that branch has no hard stop
            self.all_tokens.extend(new_tokens)
            assistant_start = len(self.all_tokens)
            nxt = self._step(new_tokens)                                            # prefill of the new chunk only
            for it in range(self.max_gen):
                if nxt in self.stop_ids:                                            # main.rs:296-298
                    break
                self.all_tokens.append(nxt)
                if self.text_stop is not None and self.text_stop(self.all_tokens[assistant_start:]):
                    break
                nxt = self._step([nxt], sample=it + 1 < self.max_gen)               # decode: only the last token
                if hard_stop and self.kv_caches[0].len + 2 >= max_seq:              # main.rs:372-375
                    break
            self.first_turn = False
            return self.all_tokens[assistant_start:]
