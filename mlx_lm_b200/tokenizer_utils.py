"""Tokenizers for the entry points.

mlx-lm wraps a Hugging Face tokenizer in ``TokenizerWrapper`` with a set of
end-of-sequence ids and a streaming detokenizer with ``reset`` / ``add_token``
/ ``finalize`` / ``last_segment`` / ``text`` (mlx_lm/tokenizer_utils.py:11-58,
284-474).  Here the wrapped object is a ``tokenizers.Tokenizer`` read from the
folder's ``tokenizer.json``; a folder without one (the random-weights mode
writes none) gets ``TokenIdTokenizer``, whose "text" is token ids in decimal
separated by blanks.
"""

from __future__ import annotations

import json
import os
from typing import Iterable, List, Optional, Sequence, Set


class StreamingDetokenizer:
    """Text grows as tokens are added; ``last_segment`` is what the last ``add_token`` or
    ``finalize`` made ready.

    Incremental: a token costs one decode of the few tokens that are not flushed yet, not of the whole
    sequence (mlx-lm streams byte-level BPE the same way, by hand over the vocabulary's byte table:
    mlx_lm/tokenizer_utils.py:157-250).  The tokens since the last flush are decoded together with the one
    token before them, and the text of that one token alone is cut off the front: a tokenizer that treats the
    start of a sequence specially (a dropped leading blank) then sees the same left context as in a decode of
    the whole sequence.  A tail that ends in the replacement character is an unfinished multi-byte character:
    it is held back until later tokens complete it (mlx_lm/tokenizer_utils.py:61-106 holds it back likewise)."""

    def __init__(self, decode):
        self._decode = decode
        self.reset()

    def reset(self) -> None:
        self.tokens: List[int] = []
        self.text = ""
        self._offset = 0          # characters of ``text`` handed out by last_segment
        self._flushed = 0         # tokens whose text is in ``text``

    def _pending_text(self) -> str:
        left = self.tokens[self._flushed - 1:self._flushed] if self._flushed else []
        text = self._decode(left + self.tokens[self._flushed:])
        if not left:
            return text
        head = self._decode(left)
        if text.startswith(head):
            return text[len(head):]
        # the left token's text changes with what follows it: fall back to the whole sequence
        return self._decode(self.tokens)[len(self.text):]

    def add_token(self, token: int) -> None:
        self.tokens.append(int(token))
        new = self._pending_text()
        if new.endswith("\ufffd"):
            return
        self.text += new
        self._flushed = len(self.tokens)

    def finalize(self) -> None:
        if self._flushed < len(self.tokens):
            self.text += self._pending_text()
            self._flushed = len(self.tokens)

    @property
    def last_segment(self) -> str:
        seg = self.text[self._offset:]
        self._offset = len(self.text)
        return seg


class TokenizerWrapper:
    def __init__(self, tokenizer, eos_token_ids: Optional[Iterable[int]] = None, bos_token: Optional[str] = None):
        self._tokenizer = tokenizer
        self.eos_token_ids: Set[int] = set(eos_token_ids or [])
        self.bos_token = bos_token
        self.has_chat_template = False

    def encode(self, text: str, add_special_tokens: bool = True) -> List[int]:
        return list(self._tokenizer.encode(text, add_special_tokens=add_special_tokens).ids)

    def decode(self, tokens: Sequence[int]) -> str:
        return self._tokenizer.decode(list(tokens), skip_special_tokens=False)

    def add_eos_token(self, token) -> None:
        if isinstance(token, int) or (isinstance(token, str) and token.isdigit()):
            self.eos_token_ids.add(int(token))
            return
        tid = self._tokenizer.token_to_id(token)
        if tid is None:
            raise ValueError(f"'{token}' is not a token for this tokenizer")
        self.eos_token_ids.add(tid)

    @property
    def detokenizer(self) -> StreamingDetokenizer:
        return StreamingDetokenizer(self.decode)

    @property
    def vocab_size(self) -> int:
        return self._tokenizer.get_vocab_size()


class TokenIdTokenizer(TokenizerWrapper):
    """Stands in where a model folder has no tokenizer: text is decimal token ids."""

    def __init__(self, vocab_size: int, eos_token_ids: Optional[Iterable[int]] = None):
        self._vocab_size = vocab_size
        self.eos_token_ids = set(eos_token_ids or [])
        self.bos_token = None
        self.has_chat_template = False

    def encode(self, text: str, add_special_tokens: bool = True) -> List[int]:
        try:
            ids = [int(t) for t in text.replace(",", " ").split()]
        except ValueError:
            raise ValueError("this model folder has no tokenizer.json: give the prompt as token ids, "
                             "e.g. --prompt '5 17 3'") from None
        if any(not 0 <= t < self._vocab_size for t in ids):
            raise ValueError(f"token id outside 0..{self._vocab_size - 1}")
        return ids

    def decode(self, tokens: Sequence[int]) -> str:
        return " ".join(str(int(t)) for t in tokens)

    def add_eos_token(self, token) -> None:
        self.eos_token_ids.add(int(token))

    @property
    def detokenizer(self) -> StreamingDetokenizer:
        return StreamingDetokenizer(lambda toks: "".join(f"{t} " for t in toks))

    @property
    def vocab_size(self) -> int:
        return self._vocab_size


def load_tokenizer(model_path: str, config: dict, eos_token_ids=None) -> TokenizerWrapper:
    """``tokenizer.json`` of the folder, else the token-id stand-in.  End-of-sequence ids come from
    the caller, else from the config (``eos_token_id`` may be a list), as in mlx_lm/utils.py:459-480."""
    eos = eos_token_ids if eos_token_ids is not None else config.get("eos_token_id")
    if eos is None:
        eos = []
    elif isinstance(eos, int):
        eos = [eos]
    path = os.path.join(model_path, "tokenizer.json")
    if not os.path.exists(path):
        return TokenIdTokenizer(int(config["vocab_size"]), eos)
    from tokenizers import Tokenizer

    tok = Tokenizer.from_file(path)
    bos = None
    cfg_path = os.path.join(model_path, "tokenizer_config.json")
    if os.path.exists(cfg_path):
        with open(cfg_path) as f:
            tc = json.load(f)
        b = tc.get("bos_token")
        bos = b.get("content") if isinstance(b, dict) else b
        if not eos:
            e = tc.get("eos_token")
            e = e.get("content") if isinstance(e, dict) else e
            if e is not None and tok.token_to_id(e) is not None:
                eos = [tok.token_to_id(e)]
    return TokenizerWrapper(tok, eos, bos)
