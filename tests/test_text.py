"""Incremental detokenisation and stop strings (no GPU), with a byte-level toy tokenizer."""
from tinyserve_b200.engine.text import Detokenizer, apply_stop_strings


class ByteTokenizer:
    """Token i is byte i; decoding joins the bytes (errors become U+FFFD, as tokenizers do)."""

    def decode(self, ids, skip_special_tokens=True):
        return bytes(ids).decode("utf-8", errors="replace")


def test_pieces_add_up_and_split_characters_are_held_back():
    text = "naïve café 日本"
    ids = list(text.encode("utf-8"))
    d = Detokenizer(ByteTokenizer())
    pieces = []
    for n in range(1, len(ids) + 1):
        pieces.append(d.update(ids[:n], final=n == len(ids)))
    assert "".join(pieces) == text == d.text
    assert "�" not in "".join(pieces)
    assert "" in pieces                       # the first byte of a two-byte character gives nothing yet
    # a request that ends in the middle of a character hands out what it has
    d = Detokenizer(ByteTokenizer())
    assert d.update(ids[:3], final=True).endswith("�")
    assert Detokenizer(None).update([1, 2], True) == ""


def test_stop_strings():
    assert apply_stop_strings("hello world", ["wor"]) == ("hello ", True)
    assert apply_stop_strings("hello wo", ["world"]) == ("hello ", False)     # could still grow into it
    assert apply_stop_strings("hello", ["xyz"]) == ("hello", False)
    assert apply_stop_strings("abc END def END", ["END", "def"]) == ("abc ", True)
