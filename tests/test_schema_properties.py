"""Guided decoding as a property: for schemas drawn from the supported subset, every document that conforms is accepted
in its compact form, every prefix of it keeps the recogniser alive (so the token mask never paints the model into a
corner on the way), and nothing may follow a finished document."""
import json

from hypothesis import given, settings
from hypothesis import strategies as st

from cuteafd_b200.serve.schema import SchemaRecognizer

TEXT = st.text(alphabet=st.sampled_from(list("abc XYZ09_-\"\\\n\t/é")), max_size=8)
NUMS = st.one_of(st.integers(-10 ** 6, 10 ** 6), st.sampled_from([0.5, -1.25, 3.0, 1e-5, 2.5e10, -0.0]))


def pairs(depth: int = 0):
    """Strategy of (schema, conforming value)."""
    scalars = [
        TEXT.map(lambda s: ({"type": "string"}, s)),
        st.integers(-10 ** 9, 10 ** 9).map(lambda n: ({"type": "integer"}, n)),
        NUMS.map(lambda n: ({"type": "number"}, n)),
        st.booleans().map(lambda b: ({"type": "boolean"}, b)),
        st.just(({"type": "null"}, None)),
        st.lists(st.one_of(TEXT, st.integers(0, 9)), min_size=1, max_size=3, unique_by=repr).flatmap(
            lambda opts: st.sampled_from(opts).map(lambda v: ({"enum": opts}, v))),
        st.one_of(TEXT, st.integers(0, 99)).map(lambda v: ({"const": v}, v)),
    ]
    if depth >= 2:
        return st.one_of(scalars)

    def arr_of(item):
        s, v = item
        return st.integers(0, 3).map(lambda n: ({"type": "array", "items": s, "minItems": min(n, 1), "maxItems": 3}, [v] * n if n else []))

    def obj_of(members):
        props = {f"k{i}": s for i, (s, _) in enumerate(members)}
        return st.lists(st.booleans(), min_size=len(members), max_size=len(members)).map(
            lambda req: ({"type": "object", "properties": props, "required": [k for k, r in zip(props, req) if r] or list(props)},
                         {k: v for (k, r), (_, v) in zip(zip(props, req), members) if r} or {k: v for k, (_, v) in zip(props, members)}))

    def any_of(ps):
        return st.sampled_from(ps).map(lambda p: ({"anyOf": [s for s, _ in ps]}, p[1]))

    sub = pairs(depth + 1)
    return st.one_of(scalars + [sub.flatmap(arr_of), st.lists(sub, min_size=1, max_size=3).flatmap(obj_of),
                                st.lists(sub, min_size=1, max_size=3).flatmap(any_of)])


@settings(max_examples=250, deadline=None)
@given(p=pairs())
def test_conforming_documents_are_accepted_prefix_by_prefix(p):
    schema, value = p
    if schema.get("type") == "array" and len(value) < schema.get("minItems", 0):
        return
    text = json.dumps(value, separators=(",", ":"), ensure_ascii=False).encode()
    r = SchemaRecognizer(schema)
    for i, b in enumerate(text):
        assert r.feed(b), (schema, text, i)
    assert r.complete(), (schema, text)
    assert not r.feed(ord("x")) and not SchemaRecognizer(schema).feed(ord("}"))
