"""JSON-schema guided decoding: a byte-level recogniser that accepts exactly the prefixes of compact JSON documents
matching a schema, with the interface ``TokenConstraint`` expects (``clone`` / ``feed`` / ``complete``).

Supported: ``type`` object / array / string / number / integer / boolean / null (also as a list of types), ``enum``,
``const``, ``anyOf`` / ``oneOf``, ``properties`` + ``required`` (members are written in the order of ``properties``;
optional members are left out), ``items``, ``minItems`` / ``maxItems``, nested to any depth; a schema without a type is
any JSON value.  Output is compact (no whitespace), which keeps the mask small and the result deterministic.
Not supported (raises ``ValueError`` when the constraint is built): ``$ref``, ``pattern``, numeric ranges,
``additionalProperties`` schemas.

The recogniser is a stack of small frames.  A frame's ``feed`` returns MORE (byte taken, not finished), DONE (byte
taken, finished), PASS (finished before this byte: the parent must look at it; numbers end this way) or NO.

The reference delegates structured outputs to xgrammar (native/shared/src/xgrammar_adapter.cc); that library is
not part of this build.
"""
from __future__ import annotations

import copy
import json

MORE, DONE, PASS, NO = 0, 1, 2, 3
_DIG = b"0123456789"
_ESC = b"\"\\/bfnrt"
_HEX = b"0123456789abcdefABCDEF"


class Lit:
    def __init__(self, data: bytes):
        self.d, self.i = data, 0

    def feed(self, b: int) -> int:
        if self.i < len(self.d) and self.d[self.i] == b:
            self.i += 1
            return DONE if self.i == len(self.d) else MORE
        return NO

    def can_end(self) -> bool:
        return self.i == len(self.d)


class Str:
    """A JSON string including its quotes."""

    def __init__(self):
        self.s = 0            # 0 expect opening quote, 1 body, 2 after backslash, 3..6 hex digits, 7 closed

    def feed(self, b: int) -> int:
        s = self.s
        if s == 0:
            if b == 0x22:
                self.s = 1
                return MORE
            return NO
        if s == 1:
            if b == 0x22:
                self.s = 7
                return DONE
            if b == 0x5C:
                self.s = 2
                return MORE
            return MORE if b >= 0x20 else NO
        if s == 2:
            if b == 0x75:
                self.s = 3
                return MORE
            if b in _ESC:
                self.s = 1
                return MORE
            return NO
        if 3 <= s <= 6:
            if b in _HEX:
                self.s = 1 if s == 6 else s + 1
                return MORE
            return NO
        return NO

    def can_end(self) -> bool:
        return self.s == 7


class Num:
    """JSON number; ends at the first byte that cannot extend it (PASS)."""

    def __init__(self, integer: bool):
        self.integer, self.s = integer, 0     # 0 start, 1 after '-', 2 zero, 3 int digits, 4 after '.', 5 frac, 6 after e, 7 after sign, 8 exp

    def can_end(self) -> bool:
        return self.s in (2, 3, 5, 8)

    def feed(self, b: int) -> int:
        s, d = self.s, b in _DIG
        nxt = None
        if s == 0:
            nxt = 1 if b == 0x2D else 2 if b == 0x30 else 3 if d else None
        elif s == 1:
            nxt = 2 if b == 0x30 else 3 if d else None
        elif s in (2, 3):
            if s == 3 and d:
                nxt = 3
            elif not self.integer and b == 0x2E:
                nxt = 4
            elif not self.integer and b in b"eE":
                nxt = 6
        elif s == 4:
            nxt = 5 if d else None
        elif s == 5:
            nxt = 5 if d else 6 if b in b"eE" else None
        elif s == 6:
            nxt = 7 if b in b"+-" else 8 if d else None
        elif s == 7:
            nxt = 8 if d else None
        elif s == 8:
            nxt = 8 if d else None
        if nxt is None:
            return PASS if self.can_end() else NO
        self.s = nxt
        return MORE


class Enum:
    """One of several literal JSON encodings."""

    def __init__(self, options: list[bytes]):
        self.o, self.i = list(options), 0

    def can_end(self) -> bool:
        return any(len(o) == self.i for o in self.o)

    def feed(self, b: int) -> int:
        keep = [o for o in self.o if len(o) > self.i and o[self.i] == b]
        if not keep:
            return PASS if self.can_end() else NO
        self.o, self.i = keep, self.i + 1
        if len(keep) == 1 and len(keep[0]) == self.i:
            return DONE
        return MORE


class Seq:
    """Frames one after the other (an object with its fixed member order)."""

    def __init__(self, parts: list):
        self.parts, self.k = parts, 0

    def can_end(self) -> bool:
        return self.k == len(self.parts) or (self.k == len(self.parts) - 1 and self.parts[self.k].can_end())

    def feed(self, b: int) -> int:
        while self.k < len(self.parts):
            r = self.parts[self.k].feed(b)
            if r == MORE:
                return MORE
            if r == DONE:
                self.k += 1
                return DONE if self.k == len(self.parts) else MORE
            if r == PASS:
                self.k += 1
                continue                      # the same byte goes to the next part
            return NO
        return PASS


class Arr:
    def __init__(self, make_item, lo: int, hi: int | None):
        self.make, self.lo, self.hi = make_item, lo, hi
        self.s, self.n, self.item = 0, 0, None      # 0 expect '[', 1 after '[', 2 in item, 3 after item, 4 closed

    def can_end(self) -> bool:
        return self.s == 4

    def _start_item(self, b: int) -> int:
        if self.hi is not None and self.n >= self.hi:
            return NO
        self.item = self.make()
        self.s = 2
        return self.feed(b)

    def feed(self, b: int) -> int:
        if self.s == 0:
            if b == 0x5B:
                self.s = 1
                return MORE
            return NO
        if self.s == 1:
            if b == 0x5D:
                if self.lo > 0:
                    return NO
                self.s = 4
                return DONE
            return self._start_item(b)
        if self.s == 2:
            r = self.item.feed(b)
            if r == MORE:
                return MORE
            if r == NO:
                return NO
            self.n += 1
            self.s = 3
            return MORE if r == DONE else self.feed(b)
        if self.s == 3:
            if b == 0x2C:
                if self.hi is not None and self.n >= self.hi:
                    return NO
                self.item = self.make()
                self.s = 2
                return MORE
            if b == 0x5D and self.n >= self.lo:
                self.s = 4
                return DONE
            return NO
        return NO


class _Finished:
    """Stands in for an alternative that has matched completely while others can still grow (5 of an enum against
    the integer 50): the value may end here, and any further byte is not this frame's."""

    def can_end(self) -> bool:
        return True

    def feed(self, b: int) -> int:
        return PASS


class Alt:
    """Several alternatives in parallel; the ones that reject a byte drop out."""

    def __init__(self, frames: list):
        self.f = frames

    def can_end(self) -> bool:
        return any(x.can_end() for x in self.f)

    def feed(self, b: int) -> int:
        res = [(x, x.feed(b)) for x in self.f]
        live = [(x, r) for x, r in res if r != NO]
        if not live:
            return NO
        done = any(r == DONE for _, r in live)
        more = [x for x, r in live if r == MORE]
        if more:                                  # finished for good only when nothing can grow any further
            self.f = more + ([_Finished()] if done else [])
            return MORE
        return DONE if done else PASS


class AnyJson:
    """Any JSON value: containers and strings through the generic recogniser, scalars directly."""

    def __init__(self):
        self.inner = None

    def can_end(self) -> bool:
        return self.inner is not None and self.inner.can_end()

    def feed(self, b: int) -> int:
        if self.inner is None:
            if b in b"{[":
                from .constraints import JsonRecognizer
                self.inner = _Generic(JsonRecognizer(object_only=False))
            elif b == 0x22:
                self.inner = Str()
            elif b in b"-0123456789":
                self.inner = Num(False)
            else:
                self.inner = Enum([b"true", b"false", b"null"])
        return self.inner.feed(b)


class _Generic:
    def __init__(self, rec):
        self.r = rec

    def can_end(self) -> bool:
        return self.r.complete()

    def feed(self, b: int) -> int:
        if not self.r.feed(b):
            return NO
        return DONE if self.r.complete() else MORE


def _literal(v) -> bytes:
    return json.dumps(v, separators=(",", ":"), ensure_ascii=False).encode()


def compile_schema(schema: dict):
    """Schema -> a factory of fresh frames (arrays need one frame per item)."""
    if not isinstance(schema, dict):
        raise ValueError("a schema must be an object")
    for k in ("$ref", "pattern", "minimum", "maximum", "exclusiveMinimum", "exclusiveMaximum", "patternProperties"):
        if k in schema:
            raise ValueError(f"schema keyword {k!r} is not supported")
    if isinstance(schema.get("additionalProperties"), dict):
        raise ValueError("additionalProperties with a schema is not supported")
    if "const" in schema:
        lit = _literal(schema["const"])
        return lambda: Lit(lit)
    if "enum" in schema:
        opts = [_literal(v) for v in schema["enum"]]
        if not opts:
            raise ValueError("empty enum")
        return lambda: Enum(opts)
    for key in ("anyOf", "oneOf"):
        if key in schema:
            subs = [compile_schema(s) for s in schema[key]]
            return lambda: Alt([m() for m in subs])
    t = schema.get("type")
    if isinstance(t, list):
        subs = [compile_schema(dict(schema, type=x)) for x in t]
        return lambda: Alt([m() for m in subs])
    if t is None:
        return AnyJson
    if t == "string":
        return Str
    if t == "integer":
        return lambda: Num(True)
    if t == "number":
        return lambda: Num(False)
    if t == "boolean":
        return lambda: Enum([b"true", b"false"])
    if t == "null":
        return lambda: Lit(b"null")
    if t == "array":
        item = compile_schema(schema.get("items", {}))
        lo, hi = int(schema.get("minItems", 0)), schema.get("maxItems")
        return lambda: Arr(item, lo, None if hi is None else int(hi))
    if t == "object":
        props = schema.get("properties")
        if not props:
            from .constraints import JsonRecognizer
            return lambda: _Generic(JsonRecognizer(object_only=True))
        req = schema.get("required")
        keys = [k for k in props if req is None or k in req]
        members = [(_literal(k) + b":", compile_schema(props[k])) for k in keys]

        def make():
            parts = [Lit(b"{")]
            for i, (head, sub) in enumerate(members):
                parts.append(Lit((b"," if i else b"") + head))
                parts.append(sub())
            parts.append(Lit(b"}"))
            return Seq(parts)
        return make
    raise ValueError(f"unsupported schema type {t!r}")


class SchemaRecognizer:
    """Top-level recogniser for ``TokenConstraint``."""

    def __init__(self, schema: dict):
        self.root = compile_schema(schema)()
        self.done = False

    def clone(self) -> "SchemaRecognizer":
        c = SchemaRecognizer.__new__(SchemaRecognizer)
        c.root, c.done = copy.deepcopy(self.root), self.done
        return c

    def feed(self, b: int) -> bool:
        if self.done:
            return False
        r = self.root.feed(b)
        if r == DONE:
            self.done = True
            return True
        return r == MORE

    def complete(self) -> bool:
        return self.done or self.root.can_end()
