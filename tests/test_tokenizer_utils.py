"""The tokenizer layer of the entry points, without a device: the token-id stand-in for folders without a
tokenizer, a byte-level tokenizer read from ``tokenizer.json`` (built here, nothing is downloaded), end-of-sequence
ids from the caller, the configuration or ``tokenizer_config.json``, and the streaming detokenizer, which must give
the same text piece by piece as all at once and hold back half a character."""
import json
import os

import pytest

from mlx_lm_b200.tokenizer_utils import StreamingDetokenizer, TokenIdTokenizer, TokenizerWrapper, load_tokenizer


def test_token_ids_as_text():
    t = TokenIdTokenizer(100, [7])
    assert t.encode("5 17, 3") == [5, 17, 3] and t.decode([5, 17, 3]) == "5 17 3"
    assert t.vocab_size == 100 and t.eos_token_ids == {7} and t.bos_token is None
    with pytest.raises(ValueError, match="token ids"):
        t.encode("hello")
    with pytest.raises(ValueError, match="outside"):
        t.encode("5 100")
    t.add_eos_token("9")
    assert t.eos_token_ids == {7, 9}
    d = t.detokenizer
    pieces = []
    for tok in (12, 3, 45):
        d.add_token(tok)
        pieces.append(d.last_segment)
    d.finalize()
    pieces.append(d.last_segment)
    assert "".join(pieces).split() == ["12", "3", "45"] and pieces[0] == "12 " and pieces[-1] == ""


def byte_level_folder(path, eos_in_tokenizer_config=True):
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers

    alphabet = pre_tokenizers.ByteLevel.alphabet()
    vocab = {ch: i for i, ch in enumerate(sorted(alphabet))}
    vocab["<|end|>"] = len(vocab)
    tok = Tokenizer(models.BPE(vocab=vocab, merges=[]))
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    tok.add_special_tokens(["<|end|>"])
    tok.save(os.path.join(path, "tokenizer.json"))
    if eos_in_tokenizer_config:
        with open(os.path.join(path, "tokenizer_config.json"), "w") as f:
            json.dump({"bos_token": {"content": "<|end|>"}, "eos_token": "<|end|>"}, f)
    return vocab


def test_tokenizer_json_and_where_the_end_of_sequence_ids_come_from(tmp_path):
    vocab = byte_level_folder(str(tmp_path))
    end = vocab["<|end|>"]
    t = load_tokenizer(str(tmp_path), {"vocab_size": 300})
    assert isinstance(t, TokenizerWrapper) and not isinstance(t, TokenIdTokenizer)
    assert t.eos_token_ids == {end} and t.bos_token == "<|end|>" and t.vocab_size == len(vocab)
    ids = t.encode("héllo wörld", add_special_tokens=False)
    assert len(ids) == len("héllo wörld".encode()) and t.decode(ids) == "héllo wörld"
    # the configuration's ids win over tokenizer_config.json, the caller's over both
    assert load_tokenizer(str(tmp_path), {"vocab_size": 300, "eos_token_id": [3, 4]}).eos_token_ids == {3, 4}
    assert load_tokenizer(str(tmp_path), {"vocab_size": 300, "eos_token_id": 5}, eos_token_ids=[6]).eos_token_ids == {6}
    t.add_eos_token("a")
    assert t.eos_token_ids == {end, vocab["a"]}
    with pytest.raises(ValueError, match="not a token"):
        t.add_eos_token("no such token")
    # no tokenizer.json: the stand-in, with the configuration's id
    empty = tmp_path / "bare"
    empty.mkdir()
    s = load_tokenizer(str(empty), {"vocab_size": 50, "eos_token_id": 2})
    assert isinstance(s, TokenIdTokenizer) and s.eos_token_ids == {2} and s.vocab_size == 50


def test_streaming_detokenizer_holds_back_half_a_character(tmp_path):
    byte_level_folder(str(tmp_path), eos_in_tokenizer_config=False)
    t = load_tokenizer(str(tmp_path), {"vocab_size": 300})
    assert t.eos_token_ids == set() and t.bos_token is None
    text = "naïve café ✓ done"
    ids = t.encode(text, add_special_tokens=False)
    d = t.detokenizer
    pieces = []
    for tok in ids:
        d.add_token(tok)
        seg = d.last_segment
        assert "�" not in seg          # never half of a multi-byte character
        pieces.append(seg)
    d.finalize()
    pieces.append(d.last_segment)
    assert "".join(pieces) == text == d.text
    assert any(p == "" for p in pieces[:-1])   # the first bytes of "ï", "é" and "✓" gave nothing yet
    d.reset()
    assert d.text == "" and d.tokens == [] and d.last_segment == ""
    # a detokenizer is a fresh object per request
    assert t.detokenizer is not t.detokenizer and isinstance(t.detokenizer, StreamingDetokenizer)


def test_streaming_detokenizer_decodes_only_what_is_new(tmp_path):
    """A token costs a decode of the few tokens not flushed yet (and one before them), not of the whole sequence
    (mlx-lm streams byte-level BPE token by token as well, mlx_lm/tokenizer_utils.py:157-250)."""
    byte_level_folder(str(tmp_path), eos_in_tokenizer_config=False)
    t = load_tokenizer(str(tmp_path), {"vocab_size": 300})
    text = "streaming ✓ text, a few hundred bytes of it: " * 8
    ids = t.encode(text, add_special_tokens=False)
    seen = []

    def counting(tokens):
        seen.append(len(tokens))
        return t.decode(tokens)

    d = StreamingDetokenizer(counting)
    out = ""
    for tok in ids:
        d.add_token(tok)
        out += d.last_segment
    d.finalize()
    out += d.last_segment
    assert out == text and len(ids) > 300
    assert max(seen) <= 4 and sum(seen) <= 4 * len(ids)      # "✓" is three tokens: at most they and one before


def test_streaming_detokenizer_keeps_a_blank_that_a_sequence_start_would_drop():
    """A decoder that drops a blank at the start of a sequence (as sentence-piece style decoders do): the pieces
    still add up to the decode of the whole."""
    words = {0: " a", 1: " b", 2: "c", 3: " d"}
    decode = lambda toks: "".join(words[t] for t in toks).lstrip(" ")
    d = StreamingDetokenizer(decode)
    pieces = []
    for tok in (0, 1, 2, 3, 1):
        d.add_token(tok)
        pieces.append(d.last_segment)
    d.finalize()
    assert "".join(pieces) + d.last_segment == decode([0, 1, 2, 3, 1]) == "a bc d b"
