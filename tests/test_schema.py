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
