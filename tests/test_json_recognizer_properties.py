"""The byte-level JSON recogniser behind ``response_format: json_object`` against Python's own parser: any document
``json`` writes is accepted in every prefix, and a text the recogniser accepts in full is a document ``json`` reads."""
import json

from hypothesis import given, settings
from hypothesis import strategies as st

from cuteafd_b200.serve.constraints import JsonRecognizer

LEAF = st.one_of(st.none(), st.booleans(), st.integers(-10 ** 9, 10 ** 9), st.sampled_from([0.5, -2.25, 1e-7, 3e20]),
                 st.text(alphabet=st.sampled_from(list("ab \"\\/\n\té漢{}[]:,")), max_size=6))
VALUE = st.recursive(LEAF, lambda kids: st.one_of(st.lists(kids, max_size=3), st.dictionaries(st.text("abc", max_size=3), kids, max_size=3)),
                     max_leaves=12)
NOISE = st.text(alphabet=st.sampled_from(list("{}[]\":,0123456789.-+eE truefalsn\\ab")), max_size=24)


def _run(text: str, object_only: bool):
    r = JsonRecognizer(object_only=object_only)
    for b in text.encode():
        if not r.feed(b):
            return False, False
    return True, r.complete()


@settings(max_examples=300)
@given(v=VALUE, pretty=st.booleans())
def test_documents_python_writes_are_accepted_prefix_by_prefix(v, pretty):
    text = json.dumps(v, ensure_ascii=False) if pretty else json.dumps(v, separators=(",", ":"), ensure_ascii=False)
    alive, done = _run(text, object_only=False)
    assert alive and done, text
    if isinstance(v, dict):
        assert _run(text, object_only=True) == (True, True)
    elif not isinstance(v, dict):
        assert _run(text, object_only=True)[1] is False


@settings(max_examples=500)
@given(text=NOISE)
def test_what_the_recogniser_accepts_python_reads(text):
    alive, done = _run(text, object_only=False)
    if alive and done:
        json.loads(text)                             # raises if the recogniser let through something that is not JSON
