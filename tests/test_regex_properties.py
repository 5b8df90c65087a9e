"""The guided-decoding regex recogniser against Python's ``re`` on generated patterns and strings: full-match agreement,
and the prefix rule the token mask relies on (a prefix the recogniser refuses cannot be completed into a match)."""
import re

from hypothesis import assume, given, settings
from hypothesis import strategies as st

from cuteafd_b200.serve.regex import RegexRecognizer

ATOMS = st.sampled_from(["a", "b", "c", "\\d", "[ab]", "[^a]", ".", "x", "\\w", "(ab|c)", "(?:a|b)"])
QUANT = st.sampled_from(["", "", "*", "+", "?", "{2}", "{1,3}", "{0,2}"])
PIECE = st.tuples(ATOMS, QUANT).map(lambda t: t[0] + t[1])
BRANCH = st.lists(PIECE, min_size=1, max_size=4).map("".join)
PATTERN = st.lists(BRANCH, min_size=1, max_size=3).map("|".join)
TEXT = st.text(alphabet=st.sampled_from(list("abcx019_ ")), max_size=7)


def _run(rec: RegexRecognizer, text: str):
    """(every byte accepted, complete at the end)"""
    r = rec.clone()
    for b in text.encode():
        if not r.feed(b):
            return False, False
    return True, r.complete()


@settings(max_examples=400, deadline=None)
@given(pat=PATTERN, text=TEXT)
def test_full_match_agrees_with_re(pat, text):
    rec = RegexRecognizer(pat)
    alive, complete = _run(rec, text)
    assert (alive and complete) == bool(re.fullmatch(pat, text)), (pat, text)


@settings(max_examples=200, deadline=None)
@given(pat=PATTERN, text=TEXT, tail=TEXT)
def test_a_refused_prefix_has_no_completion(pat, text, tail):
    rec = RegexRecognizer(pat)
    alive, _ = _run(rec, text)
    assume(not alive)
    assert re.fullmatch(pat, text + tail) is None, (pat, text, tail)
