"""Text of generated tokens: what each step adds, and the cut at a stop string.

A tokenizer is anything with ``decode(list of token ids) -> str``.  Tokens do not map to
characters one by one (a character of several bytes may be spread over tokens, a token may
begin with a space that only shows after another token), so the text that a step adds is the
difference between two decodings of a short window of the latest tokens, with and without the
new ones, as the reference does it (acvram/engine/runner.py:2640-2657).  A delta that would
end inside a character (the decoder's replacement mark at its end) is held back until the
character is whole.

Stop strings follow the reference's contract (acvram/engine/runner.py:396-415): the request
ends where the first stop string begins, the string itself is not delivered, and only text
that has not been delivered yet can be taken back.  Here the text so far is kept on the
request, so a step searches only the part that the new delta can have completed.
"""

from __future__ import annotations

from typing import Sequence

WINDOW = 8                 # tokens decoded again beside the new ones
REPLACEMENT = "�"     # what decoders put for bytes that are no whole character yet


def text_delta(tokenizer, output_ids: Sequence[int], delivered: int, final: bool = False) -> tuple[str, int]:
    """(text that the tokens output_ids[delivered:] add, how many of the tokens it covers).

    The second value is len(output_ids) unless the text ends inside a character: then nothing is
    added now and the tokens are decoded again, with their successors, at the next call
    (``final``: there is no next call, what is there is given out)."""
    n = len(output_ids)
    if delivered >= n:
        return "", n
    lo = max(0, delivered - WINDOW)
    try:
        head = tokenizer.decode(list(output_ids[lo:delivered])) if delivered > lo else ""
        full = tokenizer.decode(list(output_ids[lo:n]))
    except Exception:  # noqa: BLE001  (a tokenizer that cannot decode gives no text, as in the reference)
        return "", n
    delta = full[len(head):] if full.startswith(head) else full
    if delta.endswith(REPLACEMENT) and n - delivered < WINDOW and not final:
        return "", delivered
    return delta, n


def cut_at_stop(text: str, delta: str, stops: Sequence[str]) -> tuple[str, bool]:
    """``text`` already ends with ``delta``.  If a stop string occurs in the part of ``text`` that
    ``delta`` can have completed, return (the delta up to where the first one begins, True)."""
    longest = max((len(s) for s in stops if s), default=0)
    if not longest:
        return delta, False
    begin = len(text) - len(delta)                       # text[:begin] went out in earlier steps
    search_from = max(0, begin - longest + 1)
    cut = -1
    for s in stops:
        if s:
            at = text.find(s, search_from)
            if at >= 0 and (cut < 0 or at < cut):
                cut = at
    if cut < 0:
        return delta, False
    return (text[begin:cut] if cut > begin else ""), True
