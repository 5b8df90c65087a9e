"""Constrained decoding: incremental byte-level recognisers turned into allowed-token masks.

``JsonConstraint`` accepts exactly the prefixes of one JSON value (an object when
``object_only``); ``ChoiceConstraint`` accepts one of a fixed set of strings.  A mask is computed
by running each candidate token's bytes through a copy of the recogniser, so any tokenizer whose
tokens map to byte strings works; end-of-sequence is allowed only once the value is complete.
The mask is applied first in the sampling chain, and a grammar that allows no token is a request
error, never a fallback to the unmasked distribution.

The reference delegates this to xgrammar (rust/crates/cuteafd-daemon/src/shared/constraints.rs,
native/shared/src/xgrammar_adapter.cc); that library is not part of this build, so the JSON and
choice grammars are implemented directly.
"""
from __future__ import annotations

import copy

import torch

_WS = b" \t\r\n"
_DIGITS = b"0123456789"


class JsonRecognizer:
    """Pushdown recogniser of JSON prefixes, one byte at a time."""

    def __init__(self, object_only: bool = True):
        self.stack: list[str] = []                # "obj" | "arr"
        self.mode = "value"
        self.object_only = object_only
        self.lit = b""                            # remaining bytes of true/false/null
        self.num = ""                             # number sub-state
        self.hex = 0
        self.after_string = ""                    # where a finished string returns to: "key" | "value"
        self.done = False
        self.started = False

    def clone(self) -> "JsonRecognizer":
        c = copy.copy(self)
        c.stack = list(self.stack)
        return c

    def complete(self) -> bool:
        return self.done or (self.mode == "number" and not self.stack and self.num in ("int", "zero", "frac", "exp"))

    def _end_value(self) -> None:
        if not self.stack:
            self.mode, self.done = "done", True
        else:
            self.mode = "obj_comma" if self.stack[-1] == "obj" else "arr_comma"

    def feed(self, b: int) -> bool:
        ch = bytes([b])
        m = self.mode
        if m == "done":
            return ch in _WS
        if m == "number":
            if self._feed_number(ch):
                return True
            if self.num not in ("int", "zero", "frac", "exp"):
                return False
            self._end_value()
            return self.feed(b)
        if m == "string":
            if ch == b'"':
                if self.after_string == "key":
                    self.mode = "obj_colon"
                else:
                    self._end_value()
                return True
            if ch == b"\\":
                self.mode = "string_esc"
                return True
            return b >= 0x20
        if m == "string_esc":
            if ch in b'"\\/bfnrt':
                self.mode = "string"
                return True
            if ch == b"u":
                self.mode, self.hex = "string_hex", 4
                return True
            return False
        if m == "string_hex":
            if ch in b"0123456789abcdefABCDEF":
                self.hex -= 1
                if self.hex == 0:
                    self.mode = "string"
                return True
            return False
        if m == "literal":
            if self.lit[:1] == ch:
                self.lit = self.lit[1:]
                if not self.lit:
                    self._end_value()
                return True
            return False
        if ch in _WS:
            return True
        if m in ("value", "arr_value"):
            if m == "arr_value" and ch == b"]":
                self.stack.pop()
                self._end_value()
                return True
            if self.object_only and not self.started and ch != b"{":
                return False
            self.started = True
            if ch == b"{":
                self.stack.append("obj"); self.mode = "obj_key_or_end"; return True
            if ch == b"[":
                self.stack.append("arr"); self.mode = "arr_value"; return True
            if ch == b'"':
                self.mode, self.after_string = "string", "value"; return True
            if ch == b"-":
                self.mode, self.num = "number", "minus"; return True
            if ch == b"0":
                self.mode, self.num = "number", "zero"; return True
            if ch in _DIGITS:
                self.mode, self.num = "number", "int"; return True
            for lit in (b"true", b"false", b"null"):
                if lit[:1] == ch:
                    self.mode, self.lit = "literal", lit[1:]; return True
            return False
        if m in ("obj_key_or_end", "obj_key"):
            if ch == b'"':
                self.mode, self.after_string = "string", "key"; return True
            if ch == b"}" and m == "obj_key_or_end":
                self.stack.pop(); self._end_value(); return True
            return False
        if m == "obj_colon":
            if ch == b":":
                self.mode = "value"; return True
            return False
        if m == "obj_comma":
            if ch == b",":
                self.mode = "obj_key"; return True
            if ch == b"}":
                self.stack.pop(); self._end_value(); return True
            return False
        if m == "arr_comma":
            if ch == b",":
                self.mode = "value"; return True
            if ch == b"]":
                self.stack.pop(); self._end_value(); return True
            return False
        return False

    def _feed_number(self, ch: bytes) -> bool:
        n = self.num
        if n == "minus":
            if ch == b"0": self.num = "zero"; return True
            if ch in _DIGITS: self.num = "int"; return True
            return False
        if n in ("int", "zero"):
            if n == "int" and ch in _DIGITS: return True
            if ch == b".": self.num = "dot"; return True
            if ch in b"eE": self.num = "e"; return True
            return False
        if n == "dot":
            if ch in _DIGITS: self.num = "frac"; return True
            return False
        if n == "frac":
            if ch in _DIGITS: return True
            if ch in b"eE": self.num = "e"; return True
            return False
        if n == "e":
            if ch in b"+-": self.num = "esign"; return True
            if ch in _DIGITS: self.num = "exp"; return True
            return False
        if n == "esign":
            if ch in _DIGITS: self.num = "exp"; return True
            return False
        if n == "exp":
            return ch in _DIGITS
        return False


class ChoiceRecognizer:
    def __init__(self, options: list[str]):
        self.options = [o.encode() for o in options]
        self.pos = 0

    def clone(self) -> "ChoiceRecognizer":
        c = ChoiceRecognizer.__new__(ChoiceRecognizer)
        c.options, c.pos = list(self.options), self.pos
        return c

    def feed(self, b: int) -> bool:
        keep = [o for o in self.options if len(o) > self.pos and o[self.pos] == b]
        if not keep:
            return False
        self.options, self.pos = keep, self.pos + 1
        return True

    def complete(self) -> bool:
        return any(len(o) == self.pos for o in self.options)


class TokenConstraint:
    """Binds a recogniser to a tokenizer: ``mask()`` before each selection, ``advance()`` after."""

    def __init__(self, recognizer, tokenizer, vocab_size: int):
        self.rec, self.tok, self.vocab = recognizer, tokenizer, vocab_size
        self._bytes = [tokenizer.token_bytes(t) if t < tokenizer.vocab_size else b"" for t in range(vocab_size)]
        self.eos = set(getattr(tokenizer, "eos_ids", ()))

    def mask(self) -> torch.Tensor:
        m = torch.zeros(self.vocab, dtype=torch.bool)
        complete = self.rec.complete()
        for t, bs in enumerate(self._bytes):
            if t in self.eos:
                m[t] = complete
                continue
            if not bs:
                continue
            r = self.rec.clone()
            m[t] = all(r.feed(b) for b in bs)
        return m

    def advance(self, token: int) -> bool:
        if token in self.eos:
            return self.rec.complete()
        return all(self.rec.feed(b) for b in self._bytes[token])

    def finished(self) -> bool:
        return self.rec.complete() and getattr(self.rec, "done", True)


def from_response_format(fmt: dict | None, tokenizer, vocab_size: int) -> TokenConstraint | None:
    """OpenAI ``response_format`` / ``guided_choice`` -> constraint (None = unconstrained)."""
    if not fmt:
        return None
    t = fmt.get("type")
    if t == "json_schema":
        spec = fmt.get("json_schema") or {}
        schema = spec.get("schema") if isinstance(spec, dict) and "schema" in spec else fmt.get("schema")
        if isinstance(schema, dict) and schema:
            from .schema import SchemaRecognizer
            return TokenConstraint(SchemaRecognizer(schema), tokenizer, vocab_size)      # ValueError: unsupported keyword
    if t in ("json_object", "json_schema"):
        return TokenConstraint(JsonRecognizer(object_only=True), tokenizer, vocab_size)
    if t == "choice":
        return TokenConstraint(ChoiceRecognizer(list(fmt.get("choices", []))), tokenizer, vocab_size)
    if t == "regex":
        from .regex import RegexRecognizer
        return TokenConstraint(RegexRecognizer(str(fmt.get("pattern") or fmt.get("regex") or "")), tokenizer, vocab_size)
    if t == "structural_tag":
        from .regex import StructuralTagRecognizer
        return TokenConstraint(StructuralTagRecognizer(list(fmt.get("structures") or fmt.get("tags") or []),
                                                       at_least_one=bool(fmt.get("at_least_one")),
                                                       stop_after_first=bool(fmt.get("stop_after_first"))), tokenizer, vocab_size)
    if t in (None, "text"):
        return None
    raise ValueError(f"unsupported response_format type {t!r}")


TOOL_BEGIN, TOOL_END = "<tool_call>", "</tool_call>"


def tool_choice_of(body: dict, flavor: str = "openai") -> tuple[str, str | None, bool]:
    """A request's tool choice in any of the three protocols -> ``(mode, tool name, parallel calls allowed)`` with mode
    one of ``none | auto | required | named``.  OpenAI chat: ``"none" | "auto" | "required"`` or
    ``{"type": "function", "function": {"name": N}}`` plus ``parallel_tool_calls``; Responses: the same strings or
    ``{"type": "function", "name": N}``; Anthropic: ``{"type": "auto" | "any" | "tool" | "none", "name": N,
    "disable_parallel_tool_use": bool}``."""
    tc = body.get("tool_choice")
    parallel = body.get("parallel_tool_calls", True) is not False
    if tc is None:
        return "auto", None, parallel
    if isinstance(tc, str):
        mode = {"any": "required"}.get(tc, tc)
        if mode not in ("none", "auto", "required"):
            raise ValueError(f"tool_choice {tc!r} is not one of none, auto, required")
        return mode, None, parallel
    if not isinstance(tc, dict):
        raise ValueError("tool_choice must be a string or an object")
    if tc.get("disable_parallel_tool_use"):
        parallel = False
    t = tc.get("type")
    if t in ("function", "tool"):
        name = (tc.get("function") or {}).get("name") if isinstance(tc.get("function"), dict) else tc.get("name")
        if not isinstance(name, str) or not name:
            raise ValueError("tool_choice names no function")
        return "named", name, parallel
    if t in ("auto", "none"):
        return t, None, parallel
    if t in ("any", "required"):
        return "required", None, parallel
    raise ValueError(f"tool_choice type {t!r} is not supported")


def tool_call_format(tools: list[dict] | None, mode: str, name: str | None, parallel: bool) -> dict | None:
    """The ``structural_tag`` format that holds a reply to the request's tool choice, or None when nothing has to be
    constrained.  ``tools`` are OpenAI function tools.  A call is ``<tool_call>{"name": N, "arguments": {...}}</tool_call>``
    (the template's inline form); the arguments of a ``strict`` tool follow its ``parameters`` schema, those of other
    tools are any JSON object.  ``required`` / ``named``: the reply opens with a call; ``auto``: free text, constrained
    only inside a call and only when some tool is strict.  Without ``parallel`` the reply ends after its first call.

    Counterpart: rust/crates/cuteafd-daemon/src/shared/constraints.rs:290-330,590-620 (tool_choice required / auto with
    strict parameters compiled to a structural tag; invalid arguments refused token by token)."""
    fns = [t.get("function", t) for t in tools or [] if isinstance(t, dict)]
    if mode == "none":
        return None
    if mode in ("required", "named") and not fns:
        raise ValueError(f"tool_choice {mode} needs tools")
    if mode == "named":
        fns = [f for f in fns if f.get("name") == name]
        if not fns:
            raise ValueError(f"tool_choice names {name!r}, which is not among the tools")
    if mode == "auto" and not any(f.get("strict") for f in fns):
        return None
    calls = []
    for f in fns:
        params = f.get("parameters") if f.get("strict") and isinstance(f.get("parameters"), dict) else {"type": "object"}
        calls.append({"type": "object", "properties": {"name": {"const": f.get("name", "")}, "arguments": params},
                      "required": ["name", "arguments"], "additionalProperties": False})
    schema = calls[0] if len(calls) == 1 else {"anyOf": calls}
    return {"type": "structural_tag", "structures": [{"begin": TOOL_BEGIN, "schema": schema, "end": TOOL_END}],
            "at_least_one": mode in ("required", "named"), "stop_after_first": not parallel}

