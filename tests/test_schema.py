"""JSON-schema guided decoding: the recogniser accepts exactly the compact documents of a schema, and a served request
with ``response_format: json_schema`` returns a document that validates."""
import json

import pytest

from cuteafd_b200.serve.schema import SchemaRecognizer

SCHEMA = {"type": "object", "required": ["name", "age", "tags", "kind"], "properties": {
    "name": {"type": "string"}, "age": {"type": "integer"}, "score": {"type": "number"},
    "tags": {"type": "array", "items": {"type": "string"}, "maxItems": 2},
    "kind": {"enum": ["cat", "dog", 7]},
    "extra": {"type": ["null", "boolean"]}}}


def accepts(schema, text: str) -> bool:
    r = SchemaRecognizer(schema)
    return all(r.feed(b) for b in text.encode()) and r.complete()


def prefix_ok(schema, text: str) -> bool:
    r = SchemaRecognizer(schema)
    return all(r.feed(b) for b in text.encode())


def test_objects_follow_property_order_and_types():
    assert accepts(SCHEMA, '{"name":"a\\"b","age":-12,"tags":[],"kind":"dog"}')
    assert accepts(SCHEMA, '{"name":"","age":0,"tags":["x","y"],"kind":7}')
    assert not accepts(SCHEMA, '{"name":"a","age":1.5,"tags":[],"kind":"dog"}')          # integer
    assert not accepts(SCHEMA, '{"name":"a","age":1,"tags":["x","y","z"],"kind":"dog"}')  # maxItems
    assert not accepts(SCHEMA, '{"age":1,"name":"a","tags":[],"kind":"dog"}')             # member order is fixed
    assert not accepts(SCHEMA, '{"name":"a","age":1,"tags":[],"kind":"cow"}')
    assert not accepts(SCHEMA, '{"name":"a","age":01,"tags":[],"kind":"cat"}')
    assert prefix_ok(SCHEMA, '{"name":"a","age":1') and not accepts(SCHEMA, '{"name":"a","age":1')
    assert not prefix_ok(SCHEMA, '{ "name"')                                                  # compact output only


def test_scalars_arrays_alternatives_and_any():
    assert accepts({"type": "number"}, "-1.5e+3") and not accepts({"type": "number"}, "1.") and not accepts({"type": "number"}, "--1")
    assert accepts({"type": "array", "items": {"type": "integer"}, "minItems": 1}, "[1,22,-3]")
    assert not accepts({"type": "array", "items": {"type": "integer"}, "minItems": 1}, "[]")
    assert accepts({"type": ["null", "boolean"]}, "null") and accepts({"type": ["null", "boolean"]}, "false")
    assert accepts({"anyOf": [{"type": "integer"}, {"type": "string"}]}, '"x"') and accepts({"anyOf": [{"type": "integer"}, {"type": "string"}]}, "42")
    assert accepts({"const": {"a": 1}}, '{"a":1}')
    # an alternative that is complete does not end the value while another can still grow
    both = {"anyOf": [{"enum": ["", 5]}, {"type": "integer"}]}
    assert accepts(both, "5") and accepts(both, "50") and accepts(both, '""') and not accepts(both, "5x")
    assert accepts({"type": "array", "items": both}, "[5,50,5]")
    nested = {"type": "object", "properties": {"p": {"type": "object", "properties": {"q": {"type": "array", "items": {}}}}}}
    assert accepts(nested, '{"p":{"q":[1,"x",{"k":[true,null]},[2]]}}')
    assert accepts({}, '{"free":[1,2]}') and accepts({}, "3") and accepts({"type": "object"}, '{"a": 1}')
    with pytest.raises(ValueError):
        SchemaRecognizer({"type": "string", "pattern": "a+"})
    with pytest.raises(ValueError):
        SchemaRecognizer({"$ref": "#/x"})


def test_clone_is_independent():
    r = SchemaRecognizer(SCHEMA)
    for b in b'{"name":"a","age":1':
        assert r.feed(b)
    c = r.clone()
    assert c.feed(ord("2")) and r.feed(ord(",")) and c.feed(ord(","))
    assert not r.feed(ord("2"))


def test_served_request_returns_a_valid_document():
    import http.client
    from cuteafd_b200 import tiny_moe
    from cuteafd_b200.ref.model import init_weights
    from cuteafd_b200.runtime.backends import OracleBackend
    from cuteafd_b200.runtime.scheduler import Scheduler
    from cuteafd_b200.serve import tokenizer
    from cuteafd_b200.serve.server import Server, ServerState
    cfg = tiny_moe()
    tok = tokenizer.ByteTokenizer(cfg.vocab_size)
    srv = Server(ServerState(Scheduler(OracleBackend(cfg, init_weights(cfg, seed=0)), eos_ids=tok.eos_ids), tok, cfg.name), port=0).start()
    schema = {"type": "object", "properties": {"ok": {"type": "boolean"}, "n": {"type": "integer"}, "k": {"enum": ["a", "b"]}}}
    try:
        c = http.client.HTTPConnection("127.0.0.1", srv.port, timeout=300)
        body = {"messages": [{"role": "user", "content": "json please"}], "max_tokens": 60, "temperature": 0.8, "seed": 1,
                "response_format": {"type": "json_schema", "json_schema": {"name": "t", "schema": schema}}}
        c.request("POST", "/v1/chat/completions", json.dumps(body), {"Content-Type": "application/json"})
        r = c.getresponse()
        out = json.loads(r.read())
        assert r.status == 200
        text = out["choices"][0]["message"]["content"]
        assert text.startswith('{"ok":')
        if out["choices"][0]["finish_reason"] == "stop":
            doc = json.loads(text)
            assert isinstance(doc["ok"], bool) and isinstance(doc["n"], int) and doc["k"] in ("a", "b")
        c.request("POST", "/v1/chat/completions", json.dumps(dict(body, response_format={"type": "json_schema", "json_schema": {
            "schema": {"type": "string", "pattern": "x"}}})), {"Content-Type": "application/json"})
        bad = c.getresponse()
        bad.read()
        assert bad.status == 400
        c.close()
    finally:
        srv.stop()


# ---- regular expressions and structural tags ------------------------------------------------------------
def _accepts(rec, text: str) -> bool:
    r = rec.clone()
    return all(r.feed(b) for b in text.encode()) and r.complete()


def _prefix_ok(rec, text: str) -> bool:
    r = rec.clone()
    return all(r.feed(b) for b in text.encode())


def test_regex_recognizer_agrees_with_re_on_full_matches():
    import itertools
    import re
    from cuteafd_b200.serve.regex import RegexRecognizer
    cases = {
        r"\d{3}-\d{4}": ["555-1234", "55-1234", "555-12345", ""],
        r"(yes|no|maybe)!?": ["yes", "no!", "maybe!!", "y", "nope"],
        r"[A-Z][a-z]+( [A-Z][a-z]+)*": ["Ada Lovelace", "ada", "Ada  Lovelace", "Ada L"],
        r"[^,\s]+(,[^,\s]+){0,2}": ["a,b,c", "a,b,c,d", "a,,b", "abc"],
        r"-?(0|[1-9]\d*)(\.\d+)?": ["0", "-12.50", "01", "3.", "-"],
        r"a{2,}b?": ["a", "aa", "aaaab", "aabb"],
        r"\w+@\w+\.(com|org)": ["me@site.org", "me@site.net", "@site.com"],
        r"(?:ab)*c": ["c", "ababc", "abac"],
        r"\[x\]\.\*": ["[x].*", "x.*"],
        r"café|naïve": ["café", "naïve", "cafe"],
    }
    for pat, texts in cases.items():
        rec = RegexRecognizer(pat)
        for t in texts:
            assert _accepts(rec, t) == bool(re.fullmatch(pat, t)), (pat, t)
    # prefix property: every prefix of a match is accepted byte by byte, and a dead byte is refused at once
    rec = RegexRecognizer(r"\d{3}-\d{4}")
    assert all(_prefix_ok(rec, "555-1234"[:n]) for n in range(9)) and not _prefix_ok(rec, "55a")
    # exhaustive agreement on short strings over a small alphabet
    pat = r"(a|bc)*d?"
    rec = RegexRecognizer(pat)
    for n in range(6):
        for tup in itertools.product("abcd", repeat=n):
            t = "".join(tup)
            assert _accepts(rec, t) == bool(re.fullmatch(pat, t)), t
    r = RegexRecognizer(r"ab")
    assert not r.done and r.feed(ord("a")) and not r.done and r.feed(ord("b")) and r.done
    r = RegexRecognizer(r"ab*")
    r.feed(ord("a"))
    assert r.complete() and not r.done                          # more may follow: the reply ends with end-of-sequence
    for bad in (r"(a", r"a**?", r"a{5,2}", r"(?=a)b", r"a\1", r"[a", r"*a", r"a{999}", r"[[:alpha:]]"):
        with pytest.raises(ValueError):
            RegexRecognizer(bad)


def test_structural_tag_recognizer():
    from cuteafd_b200.serve.regex import StructuralTagRecognizer
    tags = [{"begin": "<tool_call>", "end": "</tool_call>",
             "schema": {"type": "object", "properties": {"name": {"enum": ["get_time", "search"]}, "n": {"type": "integer"}},
                        "required": ["name", "n"]}},
            {"begin": "<n>", "end": "</n>", "schema": {"type": "integer"}}]
    rec = StructuralTagRecognizer(tags)
    assert _accepts(rec, "plain text with < and > signs")
    assert _accepts(rec, 'Let me check. <tool_call>{"name":"search","n":3}</tool_call> done')
    assert not _prefix_ok(rec, '<tool_call>{"name":"delete"')                 # not in the enum
    assert not _prefix_ok(rec, '<tool_call>{"name":"search","n":3} </tool_call>')   # the end string must follow at once
    assert _prefix_ok(rec, '<tool_call>{"name":"search"') and not _accepts(rec, '<tool_call>{"name":"search"')
    assert _accepts(rec, "value <n>42</n> and <n>-7</n>")                     # a number ends at the end string's first byte
    assert not _prefix_ok(rec, "<n>4x")
    r = rec.clone()
    for b in b'<n>1</n><tool_call>{"name":"get_time","n":0}</tool_call>':
        assert r.feed(b)
    assert r.complete() and r.blocks == 2
    with pytest.raises(ValueError):
        StructuralTagRecognizer([])


def test_regex_and_structural_tag_through_response_format():
    from cuteafd_b200.serve import constraints
    from cuteafd_b200.serve.tokenizer import ByteTokenizer
    tok = ByteTokenizer(300)
    c = constraints.from_response_format({"type": "regex", "pattern": r"[ab]{2}"}, tok, 300)
    m = c.mask()
    allowed = {t for t in range(300) if m[t]}
    assert {tok.encode("a")[0], tok.encode("b")[0]} <= allowed and tok.encode("c")[0] not in allowed
    assert c.advance(tok.encode("a")[0]) and not c.finished() and c.advance(tok.encode("b")[0]) and c.finished()
    c = constraints.from_response_format({"type": "structural_tag", "structures": [{"begin": "<v>", "schema": {"type": "boolean"}, "end": "</v>"}]}, tok, 300)
    for t in tok.encode("<v>"):
        assert c.advance(t)
    m = c.mask()
    assert m[tok.encode("t")[0]] and m[tok.encode("f")[0]] and not m[tok.encode("x")[0]]
    with pytest.raises(ValueError):
        constraints.from_response_format({"type": "regex", "pattern": "(a"}, tok, 300)
