"""Regular-expression and structural-tag guided decoding: byte-level recognisers with the interface ``TokenConstraint``
expects (``clone`` / ``feed`` / ``complete`` / ``done``).

``RegexRecognizer(pattern)`` accepts exactly the prefixes of strings the pattern matches as a whole (anchors are
implied).  The pattern is compiled to a Thompson NFA over bytes and simulated with state sets, so cloning is copying a
frozenset and a step is a loop over a handful of states.  Supported syntax: literals, ``.``, escapes ``\\d \\D \\w \\W \\s
\\S \\n \\t \\r \\\\`` and escaped metacharacters, classes ``[a-z0-9_]`` / ``[^...]``, groups ``( )`` and ``(?: )``,
alternation ``|``, quantifiers ``* + ? {m} {m,} {m,n}`` (counted repeats are unrolled; ``n`` is capped at 256).
Non-ASCII literals are matched as their UTF-8 bytes; ``.`` and negated classes accept any byte except a newline, so
multi-byte characters pass through them.  Not supported (``ValueError``): back-references, look-around, lazy
quantifiers, named classes.

``StructuralTagRecognizer(tags)`` lets the model write free text until it has written one of the ``begin`` strings;
from there the content must match that tag's JSON schema, then the tag's ``end`` string must follow, and free text
resumes.  That is the shape of tool-call blocks (``<tool_call>{...}</tool_call>``).

The reference delegates these to xgrammar (native/shared/src/xgrammar_adapter.cc: JSON schema, regex, structural
tags); that library is not part of this build.
"""
from __future__ import annotations

import copy

_DIGIT = frozenset(range(0x30, 0x3A))
_WORD = frozenset(list(range(0x30, 0x3A)) + list(range(0x41, 0x5B)) + list(range(0x61, 0x7B)) + [0x5F])
_SPACE = frozenset(b" \t\n\r\f\v")
_ALL = frozenset(range(256))
_DOT = _ALL - {0x0A}
_MAX_REPEAT = 256
_MAX_STATES = 20000


class _Nfa:
    def __init__(self):
        self.eps: list[list[int]] = []
        self.edges: list[list[tuple[frozenset, int]]] = []

    def state(self) -> int:
        if len(self.eps) >= _MAX_STATES:
            raise ValueError("pattern is too large")
        self.eps.append([])
        self.edges.append([])
        return len(self.eps) - 1


class _Parser:
    """Pattern -> syntax tree: ("lit", byteset) | ("cat", [..]) | ("alt", [..]) | ("rep", node, lo, hi|None) | ("eps",)."""

    def __init__(self, pattern: str):
        self.p, self.i = pattern, 0

    def parse(self):
        node = self.alt()
        if self.i != len(self.p):
            raise ValueError(f"unexpected {self.p[self.i]!r} at {self.i}")
        return node

    def alt(self):
        parts = [self.cat()]
        while self.i < len(self.p) and self.p[self.i] == "|":
            self.i += 1
            parts.append(self.cat())
        return parts[0] if len(parts) == 1 else ("alt", parts)

    def cat(self):
        items = []
        while self.i < len(self.p) and self.p[self.i] not in "|)":
            items.append(self.repeat())
        return ("cat", items) if items else ("eps",)

    def repeat(self):
        node = self.atom()
        while self.i < len(self.p) and self.p[self.i] in "*+?{":
            c = self.p[self.i]
            if c == "{":
                j = self.p.find("}", self.i)
                body = self.p[self.i + 1:j] if j > 0 else ""
                lo_s, comma, hi_s = body.partition(",")
                if j < 0 or not lo_s.strip().isdigit() or (hi_s.strip() and not hi_s.strip().isdigit()):
                    raise ValueError(f"bad repeat at {self.i}")
                lo = int(lo_s)
                hi = lo if not comma else (int(hi_s) if hi_s.strip() else None)
                if lo > _MAX_REPEAT or (hi is not None and (hi > _MAX_REPEAT or hi < lo)):
                    raise ValueError(f"repeat bound above {_MAX_REPEAT} or reversed")
                self.i = j + 1
            else:
                lo, hi = {"*": (0, None), "+": (1, None), "?": (0, 1)}[c]
                self.i += 1
            if self.i < len(self.p) and self.p[self.i] in "?+":
                raise ValueError("lazy and possessive quantifiers are not supported")
            node = ("rep", node, lo, hi)
        return node

    def atom(self):
        c = self.p[self.i]
        if c == "(":
            self.i += 1
            if self.p.startswith("?:", self.i):
                self.i += 2
            elif self.i < len(self.p) and self.p[self.i] == "?":
                raise ValueError("look-around and named groups are not supported")
            node = self.alt()
            if self.i >= len(self.p) or self.p[self.i] != ")":
                raise ValueError("unbalanced parenthesis")
            self.i += 1
            return node
        if c == "[":
            return ("lit", self.klass())
        if c == ".":
            self.i += 1
            return ("lit", _DOT)
        if c in "^$":
            self.i += 1                                      # the whole string is matched anyway
            return ("eps",)
        if c == "\\":
            return self.escape_atom()
        if c in "*+?{":
            raise ValueError(f"nothing to repeat at {self.i}")
        self.i += 1
        raw = c.encode("utf-8")
        return ("lit", frozenset([raw[0]])) if len(raw) == 1 else ("cat", [("lit", frozenset([b])) for b in raw])

    def _escape_set(self) -> frozenset:
        if self.i + 1 >= len(self.p):
            raise ValueError("pattern ends in a backslash")
        c = self.p[self.i + 1]
        self.i += 2
        table = {"d": _DIGIT, "D": _ALL - _DIGIT, "w": _WORD, "W": _ALL - _WORD, "s": _SPACE, "S": _ALL - _SPACE,
                 "n": frozenset([0x0A]), "t": frozenset([0x09]), "r": frozenset([0x0D]), "f": frozenset([0x0C]), "v": frozenset([0x0B])}
        if c in table:
            return table[c]
        if c.isdigit() or c in "bBAZzkpP":
            raise ValueError(f"escape \\{c} is not supported")
        raw = c.encode("utf-8")
        if len(raw) != 1:
            raise ValueError("escaped non-ASCII character")
        return frozenset([raw[0]])

    def escape_atom(self):
        return ("lit", self._escape_set())

    def klass(self) -> frozenset:
        self.i += 1
        neg = self.i < len(self.p) and self.p[self.i] == "^"
        if neg:
            self.i += 1
        members: set[int] = set()
        first = True
        while True:
            if self.i >= len(self.p):
                raise ValueError("unterminated character class")
            c = self.p[self.i]
            if c == "]" and not first:
                self.i += 1
                break
            first = False
            if c == "[" and self.p.startswith("[:", self.i):
                raise ValueError("named classes are not supported")
            if c == "\\":
                got = self._escape_set()
                if len(got) != 1:
                    members |= got
                    continue
                lo = next(iter(got))
            else:
                raw = c.encode("utf-8")
                if len(raw) != 1:
                    raise ValueError("non-ASCII characters inside a class are not supported")
                lo = raw[0]
                self.i += 1
            if self.i + 1 < len(self.p) and self.p[self.i] == "-" and self.p[self.i + 1] != "]":
                self.i += 1
                hc = self.p[self.i]
                if hc == "\\":
                    hs = self._escape_set()
                    if len(hs) != 1:
                        raise ValueError("bad range end")
                    hi = next(iter(hs))
                else:
                    hraw = hc.encode("utf-8")
                    if len(hraw) != 1:
                        raise ValueError("non-ASCII range end")
                    hi = hraw[0]
                    self.i += 1
                if hi < lo:
                    raise ValueError("reversed range")
                members |= set(range(lo, hi + 1))
            else:
                members.add(lo)
        return frozenset(_ALL - members - {0x0A}) if neg else frozenset(members)


def _build(nfa: _Nfa, node, start: int) -> int:
    """Wire ``node`` from ``start``; returns its end state."""
    kind = node[0]
    if kind == "eps":
        return start
    if kind == "lit":
        end = nfa.state()
        nfa.edges[start].append((node[1], end))
        return end
    if kind == "cat":
        cur = start
        for item in node[1]:
            cur = _build(nfa, item, cur)
        return cur
    if kind == "alt":
        end = nfa.state()
        for item in node[1]:
            s = nfa.state()
            nfa.eps[start].append(s)
            nfa.eps[_build(nfa, item, s)].append(end)
        return end
    _, sub, lo, hi = node
    cur = start
    for _ in range(lo):
        cur = _build(nfa, sub, cur)
    if hi is None:
        loop = nfa.state()
        nfa.eps[cur].append(loop)
        body_end = _build(nfa, sub, loop)
        nfa.eps[body_end].append(loop)
        return loop
    end = nfa.state()
    nfa.eps[cur].append(end)
    for _ in range(hi - lo):
        cur = _build(nfa, sub, cur)
        nfa.eps[cur].append(end)
    return end


class RegexRecognizer:
    def __init__(self, pattern: str):
        self.nfa = _Nfa()
        start = self.nfa.state()
        self.accept = _build(self.nfa, _Parser(pattern).parse(), start)
        self.cur = self._closure({start})

    def _closure(self, states: set[int]) -> frozenset:
        stack, seen = list(states), set(states)
        while stack:
            for t in self.nfa.eps[stack.pop()]:
                if t not in seen:
                    seen.add(t)
                    stack.append(t)
        return frozenset(seen)

    def clone(self) -> "RegexRecognizer":
        c = RegexRecognizer.__new__(RegexRecognizer)
        c.nfa, c.accept, c.cur = self.nfa, self.accept, self.cur          # the automaton is shared, the state set copied
        return c

    def feed(self, b: int) -> bool:
        nxt = {t for s in self.cur for chars, t in self.nfa.edges[s] if b in chars}
        if not nxt:
            return False
        self.cur = self._closure(nxt)
        return True

    def complete(self) -> bool:
        return self.accept in self.cur

    @property
    def done(self) -> bool:
        """Accepting and nothing can follow: the reply ends here without waiting for an end-of-sequence token."""
        return self.complete() and not any(self.nfa.edges[s] for s in self.cur)


class StructuralTagRecognizer:
    """Free text; after a ``begin`` string, schema-constrained JSON, then the ``end`` string.

    ``at_least_one``: the reply opens with a tag (no free text before the first one) and is not complete until one
    block has closed.  ``stop_after_first``: nothing follows the first block; the reply ends there."""

    def __init__(self, tags: list[dict], at_least_one: bool = False, stop_after_first: bool = False):
        from .schema import compile_schema
        if not tags:
            raise ValueError("structural_tag needs at least one tag")
        self.tags = []
        for t in tags:
            begin, end = str(t.get("begin", "")).encode(), str(t.get("end", "")).encode()
            if not begin:
                raise ValueError("a structural tag needs a begin string")
            self.tags.append((begin, compile_schema(t.get("schema") or {}), end))
        self.mode = "free"                    # free | body | end
        self.tail = b""                       # last bytes of free text (longest begin - 1)
        self.keep = max(len(b) for b, _, _ in self.tags)
        self.body = None
        self.end = b""
        self.end_at = 0
        self.blocks = 0
        self.at_least_one, self.stop_after_first = bool(at_least_one), bool(stop_after_first)

    def clone(self) -> "StructuralTagRecognizer":
        c = copy.copy(self)
        c.body = copy.deepcopy(self.body)
        return c

    def feed(self, b: int) -> bool:
        from .schema import DONE, MORE, PASS
        if self.mode == "free":
            if self.stop_after_first and self.blocks:
                return False
            if self.at_least_one and not self.blocks and not any(t[0].startswith(self.tail + bytes([b])) for t in self.tags):
                return False                  # the first tag opens the reply
            self.tail = (self.tail + bytes([b]))[-self.keep:]
            for begin, make, end in self.tags:
                if self.tail.endswith(begin):
                    self.mode, self.body, self.end, self.end_at, self.tail = "body", make(), end, 0, b""
                    break
            return True
        if self.mode == "body":
            r = self.body.feed(b)
            if r == MORE:
                return True
            if r == DONE:
                self._body_over()
                return True
            if r == PASS:                     # a number ended at this byte: it belongs to the end string
                self._body_over()
                return self.feed(b) if self.mode == "end" else False
            return False
        if self.end_at < len(self.end) and self.end[self.end_at] == b:
            self.end_at += 1
            if self.end_at == len(self.end):
                self.mode, self.blocks = "free", self.blocks + 1
            return True
        return False

    def _body_over(self) -> None:
        self.body = None
        if self.end:
            self.mode, self.end_at = "end", 0
        else:
            self.mode, self.blocks = "free", self.blocks + 1

    def complete(self) -> bool:
        return self.mode == "free" and (self.blocks > 0 or not self.at_least_one)

    @property
    def done(self) -> bool:
        """Free text may always continue (the reply ends with end-of-sequence) unless the first block ends it."""
        return self.stop_after_first and self.blocks > 0 and self.mode == "free"
