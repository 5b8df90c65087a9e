"""Tokenizer, chat template and streaming detokenizer.

A snapshot with ``tokenizer.json`` is served through the Hugging Face ``tokenizers`` runtime; a
snapshot without one (every synthetic checkpoint here) falls back to a byte-level tokenizer whose
ids are byte values plus a few control tokens, so text round-trips exactly at any vocabulary of at
least 260.  Counterpart: rust/crates/cuteafd-loader/src/tokenizer.rs (+ tokenizer/: literal spans,
streaming decoder), per-family chat encoders in rust/crates/cuteafd-api/src/openai/chat/.
"""
from __future__ import annotations

import json
import os

BOS, EOS, IM_START, IM_END = 256, 257, 258, 259
SPECIAL = {"<|bos|>": BOS, "<|eos|>": EOS, "<|im_start|>": IM_START, "<|im_end|>": IM_END}


class ByteTokenizer:
    vocab_floor = 260

    def __init__(self, vocab_size: int):
        if vocab_size < self.vocab_floor:
            raise ValueError("byte tokenizer needs a vocabulary of at least 260")
        self.vocab_size = vocab_size
        self.eos_ids = (EOS, IM_END)

    def encode(self, text: str, specials: bool = True) -> list[int]:
        out: list[int] = []
        i = 0
        while i < len(text):
            if specials and text[i] == "<":
                hit = next((s for s in SPECIAL if text.startswith(s, i)), None)
                if hit:
                    out.append(SPECIAL[hit])
                    i += len(hit)
                    continue
            out.extend(text[i].encode("utf-8"))
            i += 1
        return out

    def decode(self, ids: list[int]) -> str:
        return self.token_bytes_seq(ids).decode("utf-8", errors="replace")

    def token_bytes(self, tid: int) -> bytes:
        return bytes([tid]) if tid < 256 else b""

    def token_bytes_seq(self, ids: list[int]) -> bytes:
        return b"".join(self.token_bytes(t) for t in ids)


class HfTokenizer:
    def __init__(self, path: str):
        from tokenizers import Tokenizer
        self.tk = Tokenizer.from_file(path)
        self.vocab_size = self.tk.get_vocab_size()
        cfg = {}
        cfg_path = os.path.join(os.path.dirname(path), "tokenizer_config.json")
        if os.path.exists(cfg_path):
            cfg = json.load(open(cfg_path))
        eos = cfg.get("eos_token")
        eos = eos.get("content") if isinstance(eos, dict) else eos
        self.eos_ids = tuple(i for i in (self.tk.token_to_id(eos) if eos else None, self.tk.token_to_id("<|im_end|>")) if i is not None)

    def encode(self, text: str, specials: bool = True) -> list[int]:
        return self.tk.encode(text, add_special_tokens=False).ids

    def decode(self, ids: list[int]) -> str:
        return self.tk.decode(ids, skip_special_tokens=True)

    def token_bytes(self, tid: int) -> bytes:
        return self.tk.decode([tid]).encode()


def load_tokenizer(snapshot: str | None, vocab_size: int):
    if snapshot:
        p = os.path.join(snapshot, "tokenizer.json")
        if os.path.exists(p):
            return HfTokenizer(p)
    return ByteTokenizer(vocab_size)


MEDIA_MARK = "\x00media:{}\x00"      # stands for media item i of the request inside the rendered text


def split_media(rendered: str, items: list) -> list:
    """Rendered chat text with ``MEDIA_MARK`` markers -> [text, item, text, ...] in prompt order."""
    out, rest = [], rendered
    for i, item in enumerate(items):
        head, mark, rest = rest.partition(MEDIA_MARK.format(i))
        out.append(head)
        if mark:
            out.append(item)
    out.append(rest)
    return out


def render_chat(messages: list[dict], add_generation_prompt: bool = True, tools: list[dict] | None = None,
                media: list | None = None) -> str:
    """ChatML-style template.  Tool definitions ride in a system block; tool results are turns of
    role ``tool``; content parts of type text are concatenated.  With ``media`` (a list to fill), image / audio parts
    are appended to it as (kind, payload) and a ``MEDIA_MARK`` marker takes their place in the text."""
    parts = []
    if tools:
        parts.append("<|im_start|>system\nYou may call these tools by emitting a JSON object "
                     '{"name": ..., "arguments": {...}} between <tool_call> tags.\n' + json.dumps(tools) + "<|im_end|>\n")
    for m in messages:
        c = m.get("content")
        if isinstance(c, list):
            pieces = []
            for p in c:
                if not isinstance(p, dict):
                    continue
                t = p.get("type")
                if t in ("text", "input_text", "output_text"):
                    pieces.append(str(p.get("text", "")).replace("\x00", ""))
                elif media is not None and t in ("image_url", "input_image", "image"):
                    url = p.get("image_url")
                    url = url.get("url") if isinstance(url, dict) else url
                    if url is None and isinstance(p.get("source"), dict):            # Anthropic: {"type": "base64", "media_type", "data"}
                        src = p["source"]
                        url = f"data:{src.get('media_type', 'image/png')};base64,{src.get('data', '')}"
                    pieces.append(MEDIA_MARK.format(len(media)))
                    media.append(("image", url))
                elif media is not None and t in ("input_audio", "audio"):
                    a = p.get("input_audio") or p.get("audio") or {}
                    pieces.append(MEDIA_MARK.format(len(media)))
                    media.append(("audio", f"data:audio/{a.get('format', 'wav')};base64,{a.get('data', '')}"))
            c = "".join(pieces)
        elif isinstance(c, str):
            c = c.replace("\x00", "")
        if c is None:
            c = ""
        if m.get("tool_calls"):
            c += "".join(f"<tool_call>{json.dumps(tc.get('function', tc))}</tool_call>" for tc in m["tool_calls"])
        parts.append(f"<|im_start|>{m.get('role', 'user')}\n{c}<|im_end|>\n")
    if add_generation_prompt:
        parts.append("<|im_start|>assistant\n")
    return "".join(parts)


def parse_tool_calls(text: str) -> tuple[str, list[dict]]:
    """Split generated text into plain content and tool calls."""
    calls, out, i = [], [], 0
    while True:
        a = text.find("<tool_call>", i)
        if a < 0:
            out.append(text[i:])
            break
        b = text.find("</tool_call>", a)
        if b < 0:
            out.append(text[i:])
            break
        out.append(text[i:a])
        try:
            obj = json.loads(text[a + 11:b])
            calls.append({"id": f"call_{len(calls)}", "type": "function",
                          "function": {"name": obj.get("name", ""), "arguments": json.dumps(obj.get("arguments", {}))}})
        except json.JSONDecodeError:
            out.append(text[a:b + 12])
        i = b + 12
    return "".join(out), calls


class StopStream:
    """Stop strings that are not single tokens: the reply ends before the first occurrence of any of them.  Text is
    passed on as it arrives except for a tail that could still grow into a stop string."""

    def __init__(self, stops):
        self.stops = [s for s in stops if s]
        self.buf = ""
        self.hit: str | None = None

    def push(self, text: str) -> str:
        if self.hit is not None or not self.stops:
            return "" if self.hit is not None else text
        self.buf += text
        first = min(((self.buf.find(s), s) for s in self.stops if s in self.buf), default=None)
        if first is not None:
            self.hit = first[1]
            out, self.buf = self.buf[:first[0]], ""
            return out
        keep = 0
        for s in self.stops:
            for k in range(min(len(s) - 1, len(self.buf)), keep, -1):
                if s.startswith(self.buf[-k:]):
                    keep = k
                    break
        out = self.buf[:len(self.buf) - keep]
        self.buf = self.buf[len(self.buf) - keep:]
        return out

    def flush(self) -> str:
        out, self.buf = ("" if self.hit is not None else self.buf), ""
        return out


class ToolCallStream:
    """Splits a streamed reply into visible text and completed tool calls.  Text is passed through as it arrives except
    for what could still turn out to be the opening tag; everything between ``<tool_call>`` and ``</tool_call>`` is held
    back and comes out as one call (or, when it does not parse, as the text it was)."""
    OPEN, CLOSE = "<tool_call>", "</tool_call>"

    def __init__(self):
        self.buf = ""
        self.inside = False
        self.calls = 0

    def push(self, text: str) -> tuple[str, list[dict]]:
        self.buf += text
        out, calls = [], []
        while True:
            if not self.inside:
                a = self.buf.find(self.OPEN)
                if a >= 0:
                    out.append(self.buf[:a])
                    self.buf, self.inside = self.buf[a + len(self.OPEN):], True
                    continue
                # keep back the longest tail that is a prefix of the opening tag
                keep = next((k for k in range(min(len(self.OPEN) - 1, len(self.buf)), 0, -1) if self.OPEN.startswith(self.buf[-k:])), 0)
                out.append(self.buf[:len(self.buf) - keep])
                self.buf = self.buf[len(self.buf) - keep:]
                break
            b = self.buf.find(self.CLOSE)
            if b < 0:
                break
            body, self.buf, self.inside = self.buf[:b], self.buf[b + len(self.CLOSE):], False
            try:
                obj = json.loads(body)
                calls.append({"id": f"call_{self.calls}", "type": "function",
                              "function": {"name": obj.get("name", ""), "arguments": json.dumps(obj.get("arguments", {}))}})
                self.calls += 1
            except json.JSONDecodeError:
                out.append(self.OPEN + body + self.CLOSE)
        return "".join(out), calls

    def flush(self) -> str:
        """What is still held when the reply ends (an unfinished tag is text)."""
        rest = (self.OPEN if self.inside else "") + self.buf
        self.buf, self.inside = "", False
        return rest


class StreamDecoder:
    """Incremental detokenizer: emits only complete UTF-8 text, holding back partial sequences."""

    def __init__(self, tok):
        self.tok, self.buf = tok, b""

    def push(self, ids: list[int]) -> str:
        self.buf += b"".join(self.tok.token_bytes(t) for t in ids)
        cut = len(self.buf)
        # hold back an incomplete trailing multi-byte sequence
        for back in range(1, min(4, len(self.buf)) + 1):
            b = self.buf[-back]
            if b & 0xC0 == 0x80:
                continue
            need = 2 if b & 0xE0 == 0xC0 else 3 if b & 0xF0 == 0xE0 else 4 if b & 0xF8 == 0xF0 else 1
            if need > back:
                cut = len(self.buf) - back
            break
        text, self.buf = self.buf[:cut].decode("utf-8", errors="replace"), self.buf[cut:]
        return text

    def flush(self) -> str:
        text, self.buf = self.buf.decode("utf-8", errors="replace"), b""
        return text
