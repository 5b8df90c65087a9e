"""Streaming helpers under arbitrary chunking: however the text (or its bytes) is cut into pieces, the client sees what
it would have seen had the reply arrived at once: whole UTF-8 characters only, everything before the first stop string
and nothing after it, tool calls lifted out and the text around them intact."""
import json

from hypothesis import given
from hypothesis import strategies as st

from cuteafd_b200.serve.tokenizer import ByteTokenizer, StopStream, StreamDecoder, ToolCallStream

TEXT = st.text(alphabet=st.sampled_from(list("ab<>/_tolcé漢🙂 \n{}\":END")), max_size=40)


def _cut(s, cuts):
    pts = sorted({c % (len(s) + 1) for c in cuts})
    out, lo = [], 0
    for p in pts + [len(s)]:
        out.append(s[lo:p])
        lo = p
    return out


@given(text=TEXT, cuts=st.lists(st.integers(0, 200), max_size=8))
def test_stream_decoder_emits_whole_characters_whatever_the_token_boundaries(text, cuts):
    tok = ByteTokenizer(512)
    ids = tok.encode(text, specials=False)
    dec, out = StreamDecoder(tok), []
    for piece in _cut(ids, cuts):
        got = dec.push(piece)
        assert "�" not in got                      # never half a character
        out.append(got)
    out.append(dec.flush())
    assert "".join(out) == text


@given(text=TEXT, stops=st.lists(st.sampled_from(["END", "</s>", "\n\n", "ab", "é漢"]), min_size=1, max_size=3, unique=True),
       cuts=st.lists(st.integers(0, 200), max_size=8))
def test_stop_stream_ends_before_the_first_stop_string(text, stops, cuts):
    s, out = StopStream(stops), []
    for piece in _cut(text, cuts):
        out.append(s.push(piece))
    out.append(s.flush())
    hits = [text.find(x) for x in stops if x in text]
    want = text[:min(hits)] if hits else text
    assert "".join(out) == want and (s.hit is not None) == bool(hits)


@given(before=TEXT.filter(lambda t: "<tool_call>" not in t), after=TEXT.filter(lambda t: "<tool_call>" not in t),
       args=st.dictionaries(st.sampled_from(["a", "b", "q"]), st.integers(0, 9), max_size=2), cuts=st.lists(st.integers(0, 300), max_size=10))
def test_tool_call_stream_lifts_the_call_out_whatever_the_chunking(before, after, args, cuts):
    call = "<tool_call>" + json.dumps({"name": "f", "arguments": args}) + "</tool_call>"
    whole = before + call + after
    s, text, calls = ToolCallStream(), [], []
    for piece in _cut(whole, cuts):
        t, c = s.push(piece)
        text.append(t)
        calls += c
    text.append(s.flush())
    assert "".join(text) == before + after
    assert len(calls) == 1 and calls[0]["function"]["name"] == "f" and json.loads(calls[0]["function"]["arguments"]) == args
