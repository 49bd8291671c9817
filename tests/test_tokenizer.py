"""`LlamaTokenizer` (lumen_b200/tokenizer.py, the mirror of src/tokenizer.rs:5-70) over a tokenizer.json built in the
test: a word-level vocabulary with Llama-2 style or Llama-3 style special tokens.  Needs no GPU; the module is loaded
by file path, so the CUDA library is not needed either."""
import importlib.util
import json
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def _module():
    spec = importlib.util.spec_from_file_location("_lumen_tokenizer", ROOT / "lumen_b200" / "tokenizer.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _tokenizer_json(specials, words=("hello", "world", "the", "cat", "sat")):
    from tokenizers import Tokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import Whitespace
    from tokenizers.processors import TemplateProcessing
    vocab = {"<unk>": 0}
    for w in list(specials) + list(words):
        vocab[w] = len(vocab)
    tok = Tokenizer(WordLevel(vocab, unk_token="<unk>"))
    tok.pre_tokenizer = Whitespace()
    tok.add_special_tokens(list(specials))
    bos = specials[0]
    tok.post_processor = TemplateProcessing(single=f"{bos} $A", special_tokens=[(bos, vocab[bos])])
    return tok.to_str(), vocab


def test_llama2_style_tokenizer(tmp_path):
    pytest.importorskip("tokenizers")
    text, vocab = _tokenizer_json(["<s>", "</s>", "<pad>"])
    path = tmp_path / "tokenizer.json"
    path.write_text(text)
    t = _module().LlamaTokenizer.from_file(path)
    assert t.vocab_size() == len(vocab)
    assert t.encode("hello world", False) == [vocab["hello"], vocab["world"]]
    assert t.encode("hello world", True) == [vocab["<s>"], vocab["hello"], vocab["world"]]   # with_special_tokens adds BOS
    assert t.encode("hello dog", False) == [vocab["hello"], vocab["<unk>"]]
    assert t.decode([vocab["<s>"], vocab["the"], vocab["cat"]], True) == "the cat"
    assert "<s>" in t.decode([vocab["<s>"], vocab["the"]], False)
    assert t.decode([10 ** 9], True) == ""                                                   # undecodable ids: empty string
    assert t.token_to_id("sat") == vocab["sat"] and t.token_to_id("dog") is None
    assert (t.bos_id(), t.eos_id(), t.pad_id(), t.eot_id()) == (vocab["<s>"], vocab["</s>"], vocab["<pad>"], None)


def test_llama3_style_special_tokens_and_errors(tmp_path):
    pytest.importorskip("tokenizers")
    text, vocab = _tokenizer_json(["<|begin_of_text|>", "<|end_of_text|>", "<|eot_id|>", "<|pad|>"])
    t = _module().LlamaTokenizer.from_str(text)
    assert t.bos_id() == vocab["<|begin_of_text|>"]
    assert t.eos_id() == vocab["<|end_of_text|>"]          # end of text is tried before end of turn
    assert t.eot_id() == vocab["<|eot_id|>"] and t.pad_id() == vocab["<|pad|>"]
    no_eos = json.loads(text)
    t2 = _module().LlamaTokenizer.from_str(_tokenizer_json(["<|begin_of_text|>", "<|eot_id|>"])[0])
    assert t2.eos_id() == t2.eot_id() is not None            # falls through to the end-of-turn token
    assert no_eos["model"]["type"] == "WordLevel"
    with pytest.raises(FileNotFoundError):
        _module().LlamaTokenizer.from_file(tmp_path / "missing.json")
    bad = tmp_path / "bad.json"
    bad.write_text("{not json")
    with pytest.raises(Exception):
        _module().LlamaTokenizer.from_file(bad)
