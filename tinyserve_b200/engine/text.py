"""Text at the edge of the engine: tokenizer loading, incremental detokenisation and stop
strings.  The engine itself works on token ids; a model folder without tokenizer files
is served by ids alone.  Behaviour follows serve.py:2309-2379."""
from __future__ import annotations

import os

_TOKENIZER_FILES = ("tokenizer.json", "tokenizer.model", "vocab.json", "tokenizer_config.json")


def load_tokenizer(model_dir: str):
    """The folder's tokenizer through ``transformers.AutoTokenizer``, or None if the folder
    has no tokenizer files (serve.py:2392)."""
    if not model_dir or not any(os.path.isfile(os.path.join(model_dir, f)) for f in _TOKENIZER_FILES):
        return None
    from transformers import AutoTokenizer
    return AutoTokenizer.from_pretrained(model_dir)


class Detokenizer:
    """Turns a growing list of generated ids into text piece by piece.

    Every call decodes the request's whole output again and hands out what is new beyond the
    text already given (a tokenizer may join or space a token differently once its neighbour is
    known, so only the whole sequence decodes reliably; the cost is linear in the output so far).
    Text that ends in U+FFFD is held back unless the request is over: the bytes of one character
    may be spread over several tokens.  tinyserve decodes a sliding window instead
    (serve.py:2309-2341); the pieces are the same."""

    def __init__(self, tok):
        self.tok = tok
        self.text = ""
        self.released = 0      # characters already handed out when stop strings hold text back

    def update(self, ids, final: bool) -> str:
        if self.tok is None:
            return ""
        whole = self.tok.decode(list(ids), skip_special_tokens=True)
        if not final and whole.endswith("\ufffd"):
            return ""
        if not whole.startswith(self.text):
            # the tokenizer rewrote earlier text (rare): keep what was given, add only what is longer
            whole = self.text + whole[len(self.text):]
        piece = whole[len(self.text):]
        self.text = whole
        return piece


def apply_stop_strings(text: str, stop: list) -> tuple:
    """(text safe to show, whether a stop string was reached).  Text from the first complete
    stop string on is cut; otherwise the longest tail that could still grow into a stop
    string is held back (serve.py:2343-2379)."""
    found = [text.find(s) for s in stop if s]
    found = [i for i in found if i >= 0]
    if found:
        return text[:min(found)], True
    held = 0
    for s in stop:
        for k in range(min(len(s) - 1, len(text)), 0, -1):
            if text.endswith(s[:k]):
                held = max(held, k)
                break
    return text[:len(text) - held], False
