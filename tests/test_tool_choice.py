"""Tool choice: required / named / auto-with-strict-tools compile to a structural tag around the template's inline call
form; the three protocols' spellings agree; an oracle server's forced call parses as a tool call with valid arguments."""
import json

import pytest

from cuteafd_b200.serve import api, constraints as C
from cuteafd_b200.serve.gateway import to_chat_body
from cuteafd_b200.serve.regex import StructuralTagRecognizer
from cuteafd_b200.serve.tokenizer import load_tokenizer, parse_tool_calls

LOOKUP = {"type": "function", "function": {"name": "lookup", "strict": True, "parameters": {
    "type": "object", "properties": {"x": {"const": "a"}}, "required": ["x"], "additionalProperties": False}}}
LOOSE = {"type": "function", "function": {"name": "loose", "parameters": {"type": "object"}}}


def accepts(fmt, text):
    r = StructuralTagRecognizer(fmt["structures"], fmt["at_least_one"], fmt["stop_after_first"])
    return all(r.feed(b) for b in text.encode()) and r.complete()


def call(name, args):
    return "<tool_call>" + json.dumps({"name": name, "arguments": args}, separators=(",", ":")) + "</tool_call>"


def test_choice_spellings_of_the_three_protocols():
    assert C.tool_choice_of({}) == ("auto", None, True)
    assert C.tool_choice_of({"tool_choice": "required", "parallel_tool_calls": False}) == ("required", None, False)
    assert C.tool_choice_of({"tool_choice": {"type": "function", "function": {"name": "f"}}}) == ("named", "f", True)
    assert C.tool_choice_of({"tool_choice": {"type": "function", "name": "f"}}, "responses") == ("named", "f", True)
    assert C.tool_choice_of({"tool_choice": {"type": "any", "disable_parallel_tool_use": True}}, "anthropic") == ("required", None, False)
    assert C.tool_choice_of({"tool_choice": {"type": "tool", "name": "f"}}, "anthropic") == ("named", "f", True)
    assert C.tool_choice_of({"tool_choice": {"type": "none"}}, "anthropic")[0] == "none"
    for bad in ("sometimes", 3, {"type": "function"}, {"type": "weird"}):
        with pytest.raises(ValueError):
            C.tool_choice_of({"tool_choice": bad})


def test_required_opens_with_a_call_and_checks_strict_arguments():
    f = C.tool_call_format([LOOKUP, LOOSE], "required", None, True)
    assert accepts(f, call("lookup", {"x": "a"}))
    assert accepts(f, call("loose", {"q": [1, {"z": None}]}) + " then " + call("lookup", {"x": "a"}))
    assert not accepts(f, "")                                                   # a call is owed
    assert not accepts(f, "Sure. " + call("lookup", {"x": "a"}))                # nothing before the first call
    assert not accepts(f, call("lookup", {"x": "b"})) and not accepts(f, call("lookup", {}))
    assert not accepts(f, call("lookup", {"x": "a", "extra": True})) and not accepts(f, call("other", {}))
    assert not accepts(f, call("loose", [])) and not accepts(f, "<tool_call>null</tool_call>")


def test_named_and_single_call():
    f = C.tool_call_format([LOOKUP, LOOSE], "named", "loose", False)
    assert accepts(f, call("loose", {})) and not accepts(f, call("lookup", {"x": "a"}))
    assert not accepts(f, call("loose", {}) + "x") and not accepts(f, call("loose", {}) + call("loose", {}))
    r = StructuralTagRecognizer(f["structures"], True, True)
    assert all(r.feed(b) for b in call("loose", {}).encode()) and r.done      # the reply ends without an end token
    with pytest.raises(ValueError, match="not among"):
        C.tool_call_format([LOOKUP], "named", "loose", True)
    with pytest.raises(ValueError, match="needs tools"):
        C.tool_call_format([], "required", None, True)


def test_auto_constrains_only_strict_tools():
    assert C.tool_call_format([LOOSE], "auto", None, True) is None
    assert C.tool_call_format([LOOKUP], "none", None, True) is None
    f = C.tool_call_format([LOOKUP, LOOSE], "auto", None, True)
    assert accepts(f, "plain text") and accepts(f, "text " + call("lookup", {"x": "a"}) + " more")
    assert not accepts(f, "text " + call("lookup", {"x": 1}))


def test_build_request_binds_the_choice():
    tok = load_tokenizer(None, 512)
    body = {"messages": [{"role": "user", "content": "look it up"}], "tools": [LOOKUP, LOOSE]}
    assert api.build_request(body, tok, 512).constraint is not None             # strict tool under auto
    assert api.build_request(dict(body, tools=[LOOSE]), tok, 512).constraint is None
    req = api.build_request(dict(body, tool_choice="required"), tok, 512)
    assert req.constraint.rec.at_least_one and not req.constraint.rec.stop_after_first
    # a forced call outranks a response_format; strict tools under auto yield to it
    both = api.build_request(dict(body, tool_choice="required", response_format={"type": "json_object"}), tok, 512)
    assert isinstance(both.constraint.rec, StructuralTagRecognizer)
    auto = api.build_request(dict(body, response_format={"type": "json_object"}), tok, 512)
    assert not isinstance(auto.constraint.rec, StructuralTagRecognizer)
    shown = tok.decode(api.build_request(dict(body, tool_choice="auto"), tok, 512).prompt)
    hidden = tok.decode(api.build_request(dict(body, tool_choice="none"), tok, 512).prompt)
    assert "lookup" in shown and "lookup" not in hidden and api.build_request(dict(body, tool_choice="none"), tok, 512).constraint is None
    for bad in ({"tool_choice": "always"}, {"tool_choice": {"type": "function", "function": {"name": "nope"}}}):
        with pytest.raises(api.BadRequest):
            api.build_request(dict(body, **bad), tok, 512)
    with pytest.raises(api.BadRequest):
        api.build_request({"messages": body["messages"], "tool_choice": "required"}, tok, 512)
    # Anthropic declarations and choice
    ant = {"messages": body["messages"], "max_tokens": 32, "tool_choice": {"type": "tool", "name": "lookup"},
           "tools": [{"name": "lookup", "input_schema": LOOKUP["function"]["parameters"], "strict": True}]}
    assert api.build_request(ant, tok, 512, flavor="anthropic").constraint.rec.at_least_one


def test_gateway_forwards_the_choice_in_chat_spelling():
    ant = {"model": "m", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 8,
           "tools": [{"name": "lookup", "input_schema": {"type": "object"}}],
           "tool_choice": {"type": "tool", "name": "lookup", "disable_parallel_tool_use": True}}
    out = to_chat_body(ant, "anthropic", {})
    assert out["tool_choice"] == {"type": "function", "function": {"name": "lookup"}} and out["parallel_tool_calls"] is False
    assert "tool_choice" not in to_chat_body(dict(ant, tool_choice={"type": "auto"}), "anthropic", {})
    assert to_chat_body(dict(ant, tool_choice={"type": "any"}), "anthropic", {})["tool_choice"] == "required"


def test_a_forced_call_through_the_oracle_server():
    """A random-weight model under ``tool_choice=required`` still answers with one parsable call whose arguments
    satisfy the strict schema: the constraint, not the model, writes the structure."""
    from cuteafd_b200.config import tiny_moe
    from cuteafd_b200.ref.model import init_weights
    from cuteafd_b200.runtime.backends import OracleBackend
    from cuteafd_b200.runtime.scheduler import Scheduler, collect
    cfg = tiny_moe()
    tok = load_tokenizer(None, cfg.vocab_size)
    s = Scheduler(OracleBackend(cfg, init_weights(cfg, seed=0)))
    body = {"messages": [{"role": "user", "content": "go"}], "tools": [LOOKUP], "tool_choice": "required",
            "parallel_tool_calls": False, "max_tokens": 120, "temperature": 0}
    req = api.build_request(body, tok, cfg.vocab_size)
    s.submit(req)
    for _ in range(2000):
        if not s.step() and not s.decoding and not s.prefilling and not s.pending and s.waiting.empty():
            break
    out = collect(req, timeout=1.0)
    text = tok.decode(out["tokens"])
    content, calls = parse_tool_calls(text)
    assert out.get("error") is None and out["finish"] == "stop", (out.get("error"), out["finish"], text)
    assert content == "" and len(calls) == 1 and calls[0]["function"]["name"] == "lookup"
    assert json.loads(calls[0]["function"]["arguments"]) == {"x": "a"}
