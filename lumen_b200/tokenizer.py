"""`LlamaTokenizer` - host-side mirror of src/tokenizer.rs:5-70 of the reference over the Hugging Face
`tokenizers` package (the reference uses the crate of the same library): `from_file`, `encode`, `decode`,
`vocab_size`, `token_to_id` and the special-token look-ups by the names the reference tries.

The module imports nothing else from this package and needs no GPU.  `tokenizers` is imported on first use, so
that the rest of the package works without it.
"""
from __future__ import annotations

from pathlib import Path


class LlamaTokenizer:
    def __init__(self, inner):
        self.inner = inner

    @classmethod
    def from_file(cls, path) -> "LlamaTokenizer":
        """tokenizer.rs:10-14: a `tokenizer.json`; a missing or malformed file raises (the reference returns Err)."""
        from tokenizers import Tokenizer
        p = Path(path)
        if not p.is_file():
            raise FileNotFoundError(f"tokenizer file not found: {p}")
        return cls(Tokenizer.from_file(str(p)))

    @classmethod
    def from_str(cls, json_text: str) -> "LlamaTokenizer":
        from tokenizers import Tokenizer
        return cls(Tokenizer.from_str(json_text))

    def encode(self, text: str, with_special_tokens: bool) -> list:
        """tokenizer.rs:16-19"""
        return [int(i) for i in self.inner.encode(text, add_special_tokens=with_special_tokens).ids]

    def decode(self, ids, skip_special_tokens: bool) -> str:
        """tokenizer.rs:21-26: ids that cannot be decoded give the empty string."""
        try:
            return self.inner.decode([int(i) for i in ids], skip_special_tokens=skip_special_tokens)
        except Exception:
            return ""

    def vocab_size(self) -> int:
        """tokenizer.rs:28-30 (added tokens included)"""
        return int(self.inner.get_vocab_size(with_added_tokens=True))

    def token_to_id(self, token: str):
        """tokenizer.rs:32-34: None for an unknown token."""
        i = self.inner.token_to_id(token)
        return None if i is None else int(i)

    def _first_known(self, names):
        for t in names:
            i = self.token_to_id(t)
            if i is not None:
                return i
        return None

    def bos_id(self):
        """tokenizer.rs:36-44"""
        return self._first_known(("<s>", "<|begin_of_text|>"))

    def eos_id(self):
        """tokenizer.rs:46-54: Llama-2 style first, then Llama-3's end of text, then its end of turn."""
        return self._first_known(("</s>", "<|end_of_text|>", "<|eot_id|>"))

    def eot_id(self):
        """tokenizer.rs:56-59"""
        return self.token_to_id("<|eot_id|>")

    def pad_id(self):
        """tokenizer.rs:61-69"""
        return self._first_known(("<pad>", "<|pad|>"))
