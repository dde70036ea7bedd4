"""Text deltas and stop strings, with a toy tokenizer whose tokens are byte strings."""

from __future__ import annotations

import random

from acvram_b200.engine.text import cut_at_stop, text_delta


class ByteTokenizer:
    """Token i is a fixed byte string; some characters of several bytes are spread over two tokens."""

    def __init__(self):
        words = [b" the", b" cat", b"s", b" sat", b".", b"\n", b" caf", "é".encode(), " naïve".encode(), b" STOP", b"!", b" end"]
        e = "€".encode()
        self.pieces = words + [e[:1], e[1:2], e[2:], "ü".encode()[:1], "ü".encode()[1:]]

    def decode(self, ids):
        return b"".join(self.pieces[i] for i in ids).decode("utf-8", errors="replace")


def stream(tok, ids):
    out, delivered, shown = [], 0, 0
    for n in range(1, len(ids) + 1):
        d, delivered = text_delta(tok, ids[:n], delivered)
        out.append(d)
    return out


def test_deltas_add_up_to_the_whole_text_and_never_split_a_character():
    tok = ByteTokenizer()
    ids = [0, 1, 2, 3, 12, 13, 14, 4, 6, 7, 15, 16, 8, 5, 0, 1]
    deltas = stream(tok, ids)
    assert "".join(deltas) == tok.decode(ids) == " the cats sat€. caféü naïve\n the cat"
    assert all("�" not in d for d in deltas)
    assert deltas[4] == "" and deltas[5] == "" and deltas[6] == "€", "the three bytes of one character come out together"
    rng = random.Random(0)
    for _ in range(200):
        ids = [rng.randrange(12) for _ in range(rng.randrange(1, 40))]
        assert "".join(stream(tok, ids)) == tok.decode(ids)


def test_bytes_that_never_become_a_character_are_not_held_for_ever():
    tok = ByteTokenizer()
    ids = [0, 12] + [1] * 12                         # a lone first byte of a character, then ordinary tokens
    assert "".join(stream(tok, ids)) == tok.decode(ids)


def test_cut_at_the_first_stop_string_even_across_two_deltas():
    text, delta = " the cat sat", " sat"
    assert cut_at_stop(text, delta, ["dog"]) == (" sat", False)
    assert cut_at_stop(text, delta, [" sat"]) == ("", True)
    assert cut_at_stop(text, delta, ["sa", "at"]) == (" ", True), "the earliest begin wins"
    assert cut_at_stop(" the cat sat", "t sat", ["cat s"]) == ("", True), "it began in text already delivered"
    assert cut_at_stop("ab STOP", " STOP", ["STOP"]) == (" ", True)
    assert cut_at_stop("abc", "c", ["", "zz"]) == ("c", False)
    # an occurrence wholly inside text delivered earlier was judged then, not now
    assert cut_at_stop("xx STOP yy", " yy", ["STOP"]) == (" yy", False)
