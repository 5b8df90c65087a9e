"""HTTP surface over the oracle engine: OpenAI chat (JSON + SSE), Anthropic messages, Responses,
models / health / stats, auth, failure classes, probes, constraints, usage log, gateway, CLI."""
import http.client
import json

import pytest
import torch

from cuteafd_b200 import tiny_moe
from cuteafd_b200.ref.model import init_weights
from cuteafd_b200.runtime.backends import OracleBackend
from cuteafd_b200.runtime.scheduler import Scheduler
from cuteafd_b200.runtime.speculation import NgramDrafter
from cuteafd_b200.serve import constraints, tokenizer
from cuteafd_b200.serve.gateway import Gateway
from cuteafd_b200.serve.server import Server, ServerState
from cuteafd_b200.serve.usage import UsageLog


@pytest.fixture(scope="module")
def server():
    cfg = tiny_moe()
    be = OracleBackend(cfg, init_weights(cfg, seed=0))
    tok = tokenizer.ByteTokenizer(cfg.vocab_size)
    sched = Scheduler(be, max_active=4, queue_depth=8, drafter=NgramDrafter(block=3), eos_ids=tok.eos_ids)
    usage = UsageLog()
    srv = Server(ServerState(sched, tok, cfg.name, api_key="sekret", usage=usage), port=0).start()
    yield srv
    srv.stop()


def call(srv, method, path, body=None, headers=None, key="sekret"):
    c = http.client.HTTPConnection("127.0.0.1", srv.port, timeout=120)
    h = {"Content-Type": "application/json"}
    if key:
        h["Authorization"] = f"Bearer {key}"
    h.update(headers or {})
    c.request(method, path, json.dumps(body).encode() if body is not None else None, h)
    r = c.getresponse()
    raw = r.read()
    c.close()
    return r.status, dict(r.getheaders()), raw


def test_health_models_stats_auth(server):
    st, _, raw = call(server, "GET", "/health", key="")
    assert st == 200 and json.loads(raw)["status"] == "ok"
    assert call(server, "GET", "/v1/models", key="wrong")[0] == 401
    st, _, raw = call(server, "GET", "/v1/models")
    assert st == 200 and json.loads(raw)["data"][0]["id"] == "tiny-moe"
    st, _, raw = call(server, "GET", "/v1/stats")
    s = json.loads(raw)
    assert st == 200 and "prefix" in s and "draft_policy" in s and "kv" in s
    assert call(server, "GET", "/nope")[0] == 404
    assert call(server, "GET", "/", key="")[0] == 200


def test_chat_completion_json_and_probe(server):
    body = {"model": "tiny-moe", "messages": [{"role": "user", "content": "hello"}], "max_tokens": 12}
    st, _, raw = call(server, "POST", "/v1/chat/completions", body)
    out = json.loads(raw)
    assert st == 200 and out["object"] == "chat.completion"
    assert out["usage"]["completion_tokens"] <= 12 and out["choices"][0]["finish_reason"] in ("length", "stop")
    assert set(out["usage"]["speculation"]) >= {"request_id", "proposed", "accepted", "cycles"}
    # synthetic token-id prompt through the probe header; greedy decode is reproducible and hashes rows
    probe = {"prompt_ids": list(range(5, 90)), "record_rows": True, "no_speculation": True}
    a = json.loads(call(server, "POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "x"}], "max_tokens": 6},
                        {"x-cuteafd-probe": json.dumps(probe)})[2])
    b = json.loads(call(server, "POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "x"}], "max_tokens": 6},
                        {"x-cuteafd-probe": json.dumps(probe)})[2])
    assert a["probe"]["row_hashes"] == b["probe"]["row_hashes"] and len(a["probe"]["row_hashes"]) == 6
    assert b["usage"]["prompt_tokens_details"]["cached_tokens"] >= 64        # second run hits the prefix cache


def test_streaming_sse(server):
    body = {"messages": [{"role": "user", "content": "stream"}], "max_tokens": 8, "stream": True}
    st, hd, raw = call(server, "POST", "/v1/chat/completions", body)
    assert st == 200 and hd["Content-Type"] == "text/event-stream"
    events = [l[6:] for l in raw.decode().split("\n") if l.startswith("data: ")]
    assert events[-1] == "[DONE]"
    chunks = [json.loads(e) for e in events[:-1]]
    assert chunks[0]["choices"][0]["delta"].get("role") == "assistant"
    assert chunks[-1]["choices"][0]["finish_reason"] in ("length", "stop") and "usage" in chunks[-1]


def test_anthropic_and_responses(server):
    body = {"model": "tiny-moe", "system": "be brief", "messages": [{"role": "user", "content": [{"type": "text", "text": "hi"}]}], "max_tokens": 5}
    st, _, raw = call(server, "POST", "/v1/messages", body)
    m = json.loads(raw)
    assert st == 200 and m["type"] == "message" and m["stop_reason"] in ("max_tokens", "end_turn") and m["usage"]["output_tokens"] <= 5
    st, _, raw = call(server, "POST", "/v1/messages/count_tokens", body)
    assert st == 200 and json.loads(raw)["input_tokens"] > 0
    st, _, raw = call(server, "POST", "/v1/messages", dict(body, stream=True))
    names = [l[7:] for l in raw.decode().split("\n") if l.startswith("event: ")]
    assert names[0] == "message_start" and names[-1] == "message_stop" and "content_block_stop" in names
    st, _, raw = call(server, "POST", "/v1/responses", {"model": "tiny-moe", "input": "hello", "max_output_tokens": 4})
    r = json.loads(raw)
    assert st == 200 and r["object"] == "response" and r["status"] == "completed"
    assert call(server, "GET", f"/v1/responses/{r['id']}")[0] == 200
    assert call(server, "DELETE", f"/v1/responses/{r['id']}")[0] == 200
    assert call(server, "GET", f"/v1/responses/{r['id']}")[0] == 404


def test_failure_classes(server):
    assert call(server, "POST", "/v1/chat/completions", {"messages": []})[0] == 400
    assert call(server, "POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "x"}], "temperature": 9})[0] == 400
    st, _, raw = call(server, "POST", "/v1/messages", {"messages": [], "max_tokens": 3})
    assert st == 400 and json.loads(raw)["type"] == "error"
    # a prompt that cannot fit the KV pool is refused with the retry class: 429 + Retry-After
    probe = {"prompt_ids": [7] * 40000}
    st, hd, raw = call(server, "POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "x"}], "max_tokens": 4,
                                                                 "cuteafd_probe": probe})
    assert st == 429 and hd.get("Retry-After") == "1"


def test_json_constraint_and_usage(server):
    body = {"messages": [{"role": "user", "content": "give json"}], "max_tokens": 40, "response_format": {"type": "json_object"},
            "temperature": 0.7, "seed": 3}
    st, _, raw = call(server, "POST", "/v1/chat/completions", body)
    out = json.loads(raw)
    text = out["choices"][0]["message"]["content"]
    assert st == 200 and text.lstrip().startswith("{")
    if out["choices"][0]["finish_reason"] == "stop":
        json.loads(text)                                             # a finished constrained reply parses
    body = {"messages": [{"role": "user", "content": "pick"}], "max_tokens": 10, "response_format": {"type": "choice", "choices": ["yes", "no"]}}
    out = json.loads(call(server, "POST", "/v1/chat/completions", body)[2])
    assert out["choices"][0]["message"]["content"] in ("yes", "no")
    u = json.loads(call(server, "GET", "/console/usage/summary")[2])
    assert u["requests"] >= 2 and u["completion_tokens"] > 0


def test_gateway_translates(server):
    gw = Gateway(f"http://127.0.0.1:{server.port}", model_map={"claude-x": "tiny-moe"}).start()
    try:
        c = http.client.HTTPConnection("127.0.0.1", gw.port, timeout=120)
        c.request("POST", "/v1/messages", json.dumps({"model": "claude-x", "messages": [{"role": "user", "content": "hey"}], "max_tokens": 4}),
                  {"Content-Type": "application/json", "Authorization": "Bearer sekret"})
        r = c.getresponse()
        m = json.loads(r.read())
        assert r.status == 200 and m["type"] == "message" and m["role"] == "assistant"
    finally:
        gw.stop()


def test_gateway_record_and_replay(server, tmp_path):
    from cuteafd_b200.serve.gateway import Tape
    path = str(tmp_path / "tape.jsonl")
    body = {"model": "claude-x", "messages": [{"role": "user", "content": "hey"}], "max_tokens": 4, "temperature": 0}
    hdr = {"Content-Type": "application/json", "Authorization": "Bearer sekret"}

    def ask(gw, b):
        c = http.client.HTTPConnection("127.0.0.1", gw.port, timeout=120)
        c.request("POST", "/v1/messages", json.dumps(b), hdr)
        r = c.getresponse()
        return r.status, json.loads(r.read())
    gw = Gateway(f"http://127.0.0.1:{server.port}", model_map={"claude-x": "tiny-moe"}, tape=Tape(path, "record")).start()
    try:
        st, live = ask(gw, body)
        assert st == 200
    finally:
        gw.stop()
    assert len(open(path).read().splitlines()) == 1
    gw2 = Gateway("http://127.0.0.1:9", model_map={"claude-x": "tiny-moe"}, tape=Tape(path, "replay")).start()    # dead upstream
    try:
        st, again = ask(gw2, body)
        assert st == 200 and again["content"] == live["content"] and again["usage"] == live["usage"]
        st, miss = ask(gw2, dict(body, max_tokens=5))
        assert st == 404 and miss["error"]["type"] == "replay_miss"
    finally:
        gw2.stop()


def test_recognizers_and_tokenizer():
    r = constraints.JsonRecognizer()
    for b in b'{"a": [1, 2.5e3, true, null, "x\\n\\u00e9"], "b": {"c": -0}}':
        assert r.feed(b)
    assert r.complete() and not r.clone().feed(ord("x"))
    bad = constraints.JsonRecognizer()
    assert not bad.feed(ord("["))                                    # object_only
    assert not all(constraints.JsonRecognizer().feed(b) for b in b'{"a" 1}')
    tok = tokenizer.ByteTokenizer(300)
    ids = tok.encode("<|im_start|>user\nhé<|im_end|>")
    assert ids[0] == tokenizer.IM_START and ids[-1] == tokenizer.IM_END and tok.decode(ids) == "user\nhé"
    d = tokenizer.StreamDecoder(tok)
    e = "é".encode()
    assert d.push([e[0]]) == "" and d.push([e[1]]) == "é"
    text, calls = tokenizer.parse_tool_calls('ok <tool_call>{"name": "f", "arguments": {"x": 1}}</tool_call> done')
    assert calls[0]["function"]["name"] == "f" and "tool_call" not in text
    assert "<|im_start|>assistant" in tokenizer.render_chat([{"role": "user", "content": "q"}])


# ---- WebSocket endpoints --------------------------------------------------------------------------------
def _ws(server, path, key="sekret"):
    from websockets.sync.client import connect
    return connect(f"ws://127.0.0.1:{server.port}{path}", additional_headers={"Authorization": f"Bearer {key}"},
                   open_timeout=30, close_timeout=5)


def _until(ws, kind, limit=400):
    seen = []
    for _ in range(limit):
        ev = json.loads(ws.recv(timeout=120))
        seen.append(ev)
        if ev["type"] == kind:
            return seen
    raise AssertionError(f"no {kind} in {[e['type'] for e in seen]}")


def test_realtime_text_session(server):
    with _ws(server, "/v1/realtime?model=tiny") as ws:
        first = json.loads(ws.recv(timeout=30))
        assert first["type"] == "session.created" and first["session"]["modalities"] == ["text"]
        assert first["session"]["model"] == "tiny"
        ws.send(json.dumps({"type": "session.update", "session": {"instructions": "be brief", "temperature": 0.0,
                                                                    "max_response_output_tokens": 6}}))
        assert _until(ws, "session.updated")[-1]["session"]["instructions"] == "be brief"
        ws.send(json.dumps({"type": "conversation.item.create",
                            "item": {"type": "message", "role": "user", "content": [{"type": "input_text", "text": "hello"}]}}))
        assert _until(ws, "conversation.item.created")[-1]["item"]["content"][0]["text"] == "hello"
        ws.send(json.dumps({"type": "response.create"}))
        evs = _until(ws, "response.done")
        kinds = [e["type"] for e in evs]
        assert kinds[0] == "response.created" and "response.output_item.added" in kinds and "response.text.done" in kinds
        done = evs[-1]["response"]
        assert done["status"] == "completed" and 1 <= done["usage"]["output_tokens"] <= 6
        text = "".join(e["delta"] for e in evs if e["type"] == "response.text.delta")
        assert text == done["output"][0]["content"][0]["text"]
        # the reply is part of the conversation: a second turn sees a longer prompt
        ws.send(json.dumps({"type": "response.create", "response": {"max_output_tokens": 3}}))
        second = _until(ws, "response.done")[-1]["response"]
        assert second["usage"]["input_tokens"] > done["usage"]["input_tokens"]
        # audio and unknown events are errors, not disconnects
        ws.send(json.dumps({"type": "input_audio_buffer.append", "audio": "AAAA"}))
        assert _until(ws, "error")[-1]["error"]["type"] == "unsupported_modality"
        ws.send("not json")
        assert _until(ws, "error")[-1]["error"]["type"] == "invalid_request_error"
        ws.ping().wait(10)


def test_responses_over_websocket_and_cancel(server):
    with _ws(server, "/v1/responses") as ws:
        ws.send(json.dumps({"type": "response.create", "response": {"input": "count", "max_output_tokens": 5}}))
        evs = _until(ws, "response.completed")
        assert evs[0]["type"] == "response.created"
        rid = evs[-1]["response"]["id"]
        st, _, raw = call(server, "GET", f"/v1/responses/{rid}")
        assert st == 200 and json.loads(raw)["id"] == rid
        # a long response is cancelled from the client
        ws.send(json.dumps({"type": "response.create", "input": "go on", "max_output_tokens": 4000}))
        _until(ws, "response.created")
        ws.send(json.dumps({"type": "response.cancel"}))
        assert _until(ws, "response.cancelled", limit=5000)[-1]["response"]["status"] == "cancelled"
        ws.send(json.dumps({"type": "bogus"}))
        assert _until(ws, "error")[-1]["error"]["type"] == "invalid_request_error"


def test_websocket_needs_the_key(server):
    from websockets.exceptions import InvalidStatus
    with pytest.raises(InvalidStatus):
        _ws(server, "/v1/realtime", key="wrong").__enter__()


def test_responses_sessions(server):
    """previous_response_id continues the stored conversation; input_items lists it; cancel and delete behave."""
    st, _, raw = call(server, "POST", "/v1/responses", {"input": "first turn", "instructions": "be brief", "max_output_tokens": 4})
    a = json.loads(raw)
    assert st == 200
    st, _, raw = call(server, "POST", "/v1/responses", {"input": "second turn", "previous_response_id": a["id"], "max_output_tokens": 4})
    b = json.loads(raw)
    assert st == 200 and b["usage"]["input_tokens"] > a["usage"]["input_tokens"] + a["usage"]["output_tokens"]
    st, _, raw = call(server, "GET", f"/v1/responses/{b['id']}/input_items")
    items = json.loads(raw)["data"]
    assert st == 200 and [i["role"] for i in items] == ["system", "user", "assistant", "user"]
    assert items[1]["content"][0]["text"] == "first turn" and items[3]["content"][0]["text"] == "second turn"
    st, _, raw = call(server, "POST", f"/v1/responses/{b['id']}/cancel", {})
    assert st == 200 and json.loads(raw)["id"] == b["id"]
    assert call(server, "POST", "/v1/responses", {"input": "x", "previous_response_id": "resp_nope"})[0] == 400
    assert call(server, "DELETE", f"/v1/responses/{a['id']}")[0] == 200
    assert call(server, "GET", f"/v1/responses/{a['id']}/input_items")[0] == 404
    assert call(server, "POST", "/v1/responses", {"input": "x", "previous_response_id": a["id"]})[0] == 400


def test_console_state_and_usage_log(server):
    """The console document carries the live sections, and streamed replies are accounted like plain ones."""
    st, hd, raw = call(server, "GET", "/")
    assert st == 200 and b"/v1/console/state" in raw
    body = {"messages": [{"role": "user", "content": "count to three"}], "max_tokens": 6, "stream": True}
    st, _, raw = call(server, "POST", "/v1/chat/completions", body)
    assert st == 200 and b"[DONE]" in raw
    doc = json.loads(call(server, "GET", "/v1/console/state")[2])
    assert {"lanes", "pipeline", "drafts", "memory", "thermal", "usage"} <= set(doc) and doc["ready"] is True
    assert doc["pipeline"]["finished"] >= 1 and doc["pipeline"]["kv"]["total_pages"] > 0 and isinstance(doc["lanes"], list)
    rows = json.loads(call(server, "GET", "/console/usage/requests?limit=3")[2])["requests"]
    assert rows and rows[0]["api"] == "openai" and rows[0]["completion_tokens"] >= 1 and rows[0]["ttft"] is not None
    one = json.loads(call(server, "GET", f"/console/usage/request/{rows[0]['id']}")[2])
    assert one["logged"] and "count to three" in one["request"] and isinstance(one["reply"], str)
    hourly = json.loads(call(server, "GET", "/console/usage/hourly?hours=2")[2])["hourly"]
    assert len(hourly) == 2 and hourly[-1]["requests"] >= 1
    assert call(server, "GET", "/console/usage/request/999999")[0] == 404
    assert json.loads(call(server, "GET", "/console/memory")[2])["tracked_bytes"] >= 0


def test_usage_log_prunes_bodies_after_a_day(tmp_path):
    from cuteafd_b200.serve.usage import UsageLog
    now = [1_000_000.0]
    log = UsageLog(str(tmp_path / "u.sqlite"), clock=lambda: now[0])
    a = log.record("m", "openai", {"prompt_tokens": 10, "completion_tokens": 4, "cached_tokens": 5,
                                   "speculation": {"proposed": 8, "accepted": 6}}, 0.5, "stop", request={"x": 1}, reply="hi", ttft=0.1)
    now[0] += 25 * 3600
    b = log.record("m", "anthropic", {"prompt_tokens": 20, "completion_tokens": 2, "finish_detail": "repetition"}, 0.2, "length",
                   request="raw body", reply="yo")
    log.prune()
    assert log.request(a)["logged"] is False and log.request(b)["reply"] == "yo"       # accounting rows stay, bodies go
    s = log.summary(48)
    assert s["requests"] == 2 and s["draft_acceptance"] == 0.75 and s["loop_aborts"] == 1 and s["by_api"] == {"openai": 1, "anthropic": 1}
    assert log.summary(1)["requests"] == 1 and log.summary(1)["cached_share"] == 0.0
    assert [r["id"] for r in log.requests(10)] == [b, a] and [r["id"] for r in log.requests(10, before_id=b)] == [a]
    # a second handle on the same file sees the rows (the command-line report reads while the server writes)
    assert UsageLog(str(tmp_path / "u.sqlite"), clock=lambda: now[0]).summary(48)["requests"] == 2


def test_model_catalog(server):
    st, _, raw = call(server, "GET", "/v1/codex/models.json")
    m = json.loads(raw)["models"][0]
    assert st == 200 and m["slug"] == "tiny-moe" and m["context_window"] >= 1024 and m["max_output_tokens"] <= m["context_window"]


def test_http_panels_on_the_oracle_server(server):
    from cuteafd_b200.bench import panels
    out = panels.run(f"http://127.0.0.1:{server.port}", list(panels.QUICK) + ["speed", "sweep", "sustained"], "sekret",
                     {"max_tokens": 6, "levels": [1, 2], "seconds": 1.0, "concurrency": 2, "prefill_words": 96, "prompt_words": 120},
                     log=lambda *_: None)
    by = {p["panel"]: p for p in out["panels"]}
    assert by["smoke"]["ok"] and by["smoke"]["model"] == "tiny-moe"
    assert by["cache_exact"]["ok"] and by["cache_exact"]["cached_tokens"] >= 64 and by["cache_exact"]["rows_identical"]
    assert by["lossless"]["ok"] and by["template"]["ok"] and by["template"]["tokens_after_append"] > by["template"]["tokens"]
    assert by["tools"]["ok"] and by["tools"]["choice"] in ("get_time", "none")
    assert by["speed"]["ok"] and by["speed"]["prefill_tokens"] > 90 and by["speed"]["c1_ttft_s"] > 0
    assert by["sweep"]["ok"] and set(by["sweep"]["levels"]) == {"1", "2"}
    assert by["sustained"]["ok"] and by["sustained"]["requests"] >= 2 and by["sustained"]["failed"] == 0
    assert out["ok"]
    with pytest.raises(ValueError):
        panels.run(f"http://127.0.0.1:{server.port}", ["nope"], "sekret")


def test_context_load_and_fidelity_panels(server, tmp_path):
    """Sealed windows of the served weights score KL ~ 0 and full top-1 agreement through the probe; windows sealed from
    other weights miss the bars; prompts of growing length are all answered with their prefill rates."""
    from cuteafd_b200 import tiny_moe
    from cuteafd_b200.bench import fidelity as F
    from cuteafd_b200.bench import panels
    from cuteafd_b200.ref.model import init_weights
    cfg = tiny_moe()
    same, other = str(tmp_path / "same.safetensors"), str(tmp_path / "other.safetensors")
    wins = F.random_windows(cfg.vocab_size, 2, 24, seed=4)
    F.seal(F.logits_fn_for(cfg, init_weights(cfg, seed=0)), wins, same, meta={"model": cfg.name})
    F.seal(F.logits_fn_for(cfg, init_weights(cfg, seed=5)), wins, other, meta={"model": "other"})
    url = f"http://127.0.0.1:{server.port}"
    out = panels.run(url, ["fidelity", "context_load"], "sekret", {"windows": same, "lengths": [40, 100, 10 ** 7], "vocab": cfg.vocab_size},
                     log=lambda *_: None)
    by = {p["panel"]: p for p in out["panels"]}
    assert by["fidelity"]["ok"] and by["fidelity"]["kl_mean"] < 1e-4 and by["fidelity"]["top1"] == 1.0 and by["fidelity"]["positions"] == 2 * 23
    assert by["context_load"]["ok"] and set(by["context_load"]["lengths"]) == {"40", "100"}          # the third exceeds the window
    assert all(v["prefill_tok_s"] > 0 for v in by["context_load"]["lengths"].values())
    bad = panels.run(url, ["fidelity"], "sekret", {"windows": other}, log=lambda *_: None)["panels"][0]
    assert not bad["ok"] and bad["kl_mean"] > by["fidelity"]["kl_mean"]
    ag = panels.run(url, ["agentic"], "sekret", {"sessions": 2, "turns": 3, "max_tokens": 4, "prefix_words": 60}, log=lambda *_: None)["panels"][0]
    assert ag["ok"] and ag["failed"] == 0 and ag["emitted_tokens"] == 2 * 3 * 4 and ag["cache_share_after_first_turn"] > 0.5


def test_logprobs_and_probe_cold_top_k(server):
    body = {"messages": [{"role": "user", "content": "alpha beta gamma " * 30}], "max_tokens": 5, "temperature": 0,
            "logprobs": True, "top_logprobs": 3}
    st, _, raw = call(server, "POST", "/v1/chat/completions", body)
    out = json.loads(raw)
    lp = out["choices"][0]["logprobs"]["content"]
    assert st == 200 and len(lp) == out["usage"]["completion_tokens"] == 5
    for e in lp:
        tops = e["top_logprobs"]
        assert len(tops) == 3 and tops[0]["logprob"] >= tops[1]["logprob"] >= tops[2]["logprob"]
        assert e["logprob"] == tops[0]["logprob"] and e["bytes"] == tops[0]["bytes"] and e["logprob"] <= 0     # greedy: the top row
    # the same prompt again would hit the prefix cache; a cold probe computes it all, and top_k comes back as ids
    probe = {"x-cuteafd-probe": json.dumps({"cold": True, "top_k": 2})}
    st, _, raw = call(server, "POST", "/v1/chat/completions", dict(body, logprobs=False, top_logprobs=0), probe)
    cold = json.loads(raw)
    assert st == 200 and cold["usage"]["prompt_tokens_details"]["cached_tokens"] == 0 and "logprobs" not in cold["choices"][0]
    rows = cold["probe"]["top_rows"]
    assert len(rows) == 5 and all(len(r["top_ids"]) == 2 and r["token"] == r["top_ids"][0] for r in rows)
    assert [round(r["logprob"], 4) for r in rows] == [round(e["logprob"], 4) for e in lp]       # cold and warm agree
    warm = json.loads(call(server, "POST", "/v1/chat/completions", dict(body, logprobs=False, top_logprobs=0))[2])
    assert warm["usage"]["prompt_tokens_details"]["cached_tokens"] >= 64
    assert call(server, "POST", "/v1/chat/completions", dict(body, top_logprobs=50))[0] == 400


def test_probe_score_from_and_record_state(server):
    """Teacher-forced scoring through the probe header: one record per predicted prompt position from ``score_from`` on,
    nothing generated; the rows equal the oracle's own teacher-forced logits, and the width of the scoring steps does
    not change them.  ``record_state`` hashes the sequence state at the prompt and turn frontiers."""
    from cuteafd_b200.ref.model import KvState, RefDecoder
    cfg = tiny_moe()
    ids = [(7 * i + 3) % cfg.vocab_size for i in range(150)]
    msg = {"messages": [{"role": "user", "content": "x"}], "max_tokens": 4}

    def score(**kw):
        probe = dict({"prompt_ids": ids, "score_from": 100, "top_k": 2, "want": {"120": [1, 2, 3]}}, **kw)
        st, _, raw = call(server, "POST", "/v1/chat/completions", msg, {"x-cuteafd-probe": json.dumps(probe)})
        assert st == 200, raw
        return json.loads(raw)
    out = score(verify_rows=7)
    rows = out["probe"]["score_rows"]
    assert out["usage"]["completion_tokens"] == 0 and out["choices"][0]["message"]["content"] == ""
    assert [r["position"] for r in rows] == list(range(100, 150)) and [r["token"] for r in rows] == ids[100:]
    ref = RefDecoder(cfg, init_weights(cfg, seed=0))
    with torch.no_grad():
        lp = torch.log_softmax(ref.forward(torch.tensor(ids), KvState(cfg)).float(), -1)
    for r in rows:
        assert abs(r["logprob"] - float(lp[r["position"] - 1, r["token"]])) < 1e-3
        assert r["top_ids"][0] == int(lp[r["position"] - 1].argmax()) and len(r["top_ids"]) == 2
    assert set(rows[20]["want"]) == {"1", "2", "3"} and "want" not in rows[0]
    wide = score(verify_rows=64, score_positions=[101, 149])["probe"]["score_rows"]
    assert [r["position"] for r in wide] == [101, 149]
    assert abs(wide[1]["logprob"] - rows[-1]["logprob"]) < 1e-4
    assert call(server, "POST", "/v1/chat/completions", msg,
                {"x-cuteafd-probe": json.dumps({"prompt_ids": ids, "score_from": 999})})[0] == 400
    # state hashes: the same prompt gives the same prompt-frontier hash cold and through the prefix cache
    p2 = {"prompt_ids": ids, "record_state": True, "no_speculation": True}
    a = json.loads(call(server, "POST", "/v1/chat/completions", msg, {"x-cuteafd-probe": json.dumps(dict(p2, cold=True))})[2])
    b = json.loads(call(server, "POST", "/v1/chat/completions", msg, {"x-cuteafd-probe": json.dumps(p2)})[2])
    ha, hb = a["probe"]["state_hashes"], b["probe"]["state_hashes"]
    assert [h["frontier"] for h in ha] == ["prompt", "turn"] and ha[0]["kv_len"] == 150
    assert ha[0]["hash"] == hb[0]["hash"] and ha[0]["hash"] != ha[1]["hash"]


def test_console_events_and_fabric_phase(server):
    c = http.client.HTTPConnection("127.0.0.1", server.port, timeout=30)
    c.request("GET", "/v1/console/events?period=0.05&count=3", headers={"Authorization": "Bearer sekret"})
    r = c.getresponse()
    raw = r.read().decode()
    assert r.status == 200 and raw.count("event: snapshot") == 3
    first = json.loads(raw.split("data: ", 1)[1].split("\n\n", 1)[0])
    assert "pipeline" in first and "lanes" in first
    assert json.loads(call(server, "GET", "/v1/console/snapshot")[2])["model"] == "tiny-moe"
    st, _, raw = call(server, "POST", "/v1/fabric/phase", {"phase": "warm"})
    assert st == 200 and json.loads(raw) == {"phase": "warm", "closed": None} or json.loads(raw)["phase"] == "warm"
    call(server, "POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 3})
    closed = json.loads(call(server, "POST", "/v1/fabric/phase", {"phase": "timed"})[2])["closed"]
    assert closed["phase"] == "warm" and closed["delta"]["finished"] == 1 and closed["delta"]["emitted_tokens"] >= 1 and closed["seconds"] > 0


def test_tool_history_translation_across_flavours():
    from cuteafd_b200.serve import api
    from cuteafd_b200.serve.tokenizer import render_chat
    a_tools = [{"name": "get_time", "description": "now", "input_schema": {"type": "object", "properties": {"tz": {"type": "string"}}}},
               {"type": "web_search_20250305", "name": "web_search"}]
    norm = api.normalize_tools(a_tools, "anthropic")
    assert norm == [{"type": "function", "function": {"name": "get_time", "description": "now", "parameters": a_tools[0]["input_schema"]}}]
    r_tools = [{"type": "function", "name": "get_time", "parameters": {"type": "object", "properties": {}}}, {"type": "web_search"}]
    assert api.normalize_tools(r_tools, "responses")[0]["function"]["name"] == "get_time" and len(api.normalize_tools(r_tools, "responses")) == 1
    assert api.normalize_tools([], "openai") is None
    body = {"system": "be brief", "messages": [
        {"role": "user", "content": "time in Oslo?"},
        {"role": "assistant", "content": [{"type": "text", "text": "checking"}, {"type": "tool_use", "id": "tu_1", "name": "get_time", "input": {"tz": "Europe/Oslo"}}]},
        {"role": "user", "content": [{"type": "tool_result", "tool_use_id": "tu_1", "content": [{"type": "text", "text": "12:00"}]},
                                     {"type": "text", "text": "thanks, and Paris?"}]}]}
    msgs = api.anthropic_messages(body)
    assert [m["role"] for m in msgs] == ["system", "user", "assistant", "tool", "user"]
    assert msgs[2]["tool_calls"][0]["function"] == {"name": "get_time", "arguments": '{"tz": "Europe/Oslo"}'}
    assert msgs[3] == {"role": "tool", "tool_call_id": "tu_1", "content": "12:00"}
    text = render_chat(msgs, True, norm)
    assert '<tool_call>{"name": "get_time"' in text and "<|im_start|>tool\n12:00" in text and text.index("12:00") < text.index("Paris")
    items = [{"role": "user", "content": [{"type": "input_text", "text": "time?"}]},
             {"type": "reasoning", "summary": []},
             {"type": "function_call", "call_id": "c1", "name": "get_time", "arguments": "{}"},
             {"type": "function_call", "call_id": "c2", "name": "get_time", "arguments": '{"tz":"UTC"}'},
             {"type": "function_call_output", "call_id": "c1", "output": "12:00"},
             {"type": "function_call_output", "call_id": "c2", "output": {"t": "11:00"}}]
    rm = api.responses_items_to_messages(items)
    assert [m["role"] for m in rm] == ["user", "assistant", "tool", "tool"] and len(rm[1]["tool_calls"]) == 2
    assert rm[3]["content"] == '{"t": "11:00"}' and api.responses_items_to_messages(rm) == rm          # a stored conversation passes unchanged
    obj = api.responses_object("m", 'ok <tool_call>{"name": "get_time", "arguments": {"tz": "UTC"}}</tool_call>', "stop", {})
    kinds = [o["type"] for o in obj["output"]]
    assert kinds == ["message", "function_call"] and obj["output"][1]["name"] == "get_time" and json.loads(obj["output"][1]["arguments"]) == {"tz": "UTC"}
    assert obj["output_text"] == "ok "


def test_build_state_on_the_oracle_engine(tmp_path):
    """The command-line path that builds a server (flags -> engine, scheduler, trace, watchdog, loop abort)."""
    from cuteafd_b200.cli import build_parser
    from cuteafd_b200.serve.server import build_state
    args = build_parser().parse_args(["serve", "--fake-engine", "--preset", "tiny-moe", "--speculation-trace", str(tmp_path / "t.jsonl"),
                                      "--stall-dump-seconds", "30", "--loop-fast-span", "64", "--usage-db", str(tmp_path / "u.sqlite")])
    state = build_state(args)
    assert state.sched.trace is not None and state.sched.watchdog is not None and state.usage is not None
    assert state.sched.loop_abort.fast_span == 64 and state.model_id == "tiny-moe"
    state.sched.watchdog.stop()
    state.sched.trace.close()


def test_capacity_tables():
    from cuteafd_b200.config import qwen3_30b_a3b
    from cuteafd_b200.planner import capacity
    assert [capacity.prefill_unit_rows(k) for k in (1, 2, 3, 4, 8)] == [8192, 4096, 2688, 2048, 1024]
    assert capacity.prefill_waves(8192, 2048) == [2048] * 4 and capacity.prefill_waves(5000, 2048) == [2048, 2048, 960]
    keys = capacity.default_prewarm(8, draft_block=4)
    assert [1, 1, 1] in keys and [8, 8, 1] in keys and [8, 40, 5] in keys and [4, 8, 2] in keys and len(keys) == len({tuple(k) for k in keys})
    assert all(s <= 8 and t >= s and q * s >= t for s, t, q in keys)            # what EngineBackend.prewarm accepts
    assert capacity.default_prewarm(64, 0)[-1] == [64, 64, 1] and len(capacity.default_prewarm(64, 4, limit=10)) == 10
    cfg = qwen3_30b_a3b()
    assert 8 * capacity.workspace_bytes(cfg, 1024) == capacity.workspace_bytes(cfg, 8192) < 4 << 30


def test_expert_usage_counters(server):
    call(server, "POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "route some tokens"}], "max_tokens": 4})
    st, _, raw = call(server, "GET", "/experts")
    u = json.loads(raw)
    assert st == 200 and u["experts"] == 8 and u["top_k"] == 2 and u["layers"]
    for layer in u["layers"].values():
        assert len(layer["tokens"]) == 8 and layer["total"] == sum(layer["tokens"]) > 0 and layer["total"] % 2 == 0
        assert layer["imbalance"] >= 1.0
    assert json.loads(call(server, "GET", "/v1/console/state")[2])["experts"]["layers"].keys() == u["layers"].keys()


def test_responses_compact_round_trip(server):
    from cuteafd_b200.serve import api
    conv = [{"role": "user", "content": "plan a trip to Oslo"}, {"role": "assistant", "content": "sure: flights, hotel, museums"},
            {"role": "user", "content": "book the museums first"}]
    st, _, raw = call(server, "POST", "/v1/responses/compact", {"input": conv, "max_output_tokens": 12})
    out = json.loads(raw)
    assert st == 200 and out["object"] == "response.compaction" and out["output"][0]["type"] == "compaction"
    assert out["usage"]["output_tokens"] >= 1 and out["usage"]["input_tokens"] > 20
    item = out["output"][0]
    summary = api.decode_opaque(item["encrypted_content"], "compaction")
    assert isinstance(summary, str) and summary
    # the item stands for the turns it replaced in a later request
    msgs = api.responses_items_to_messages([item, {"role": "user", "content": "continue"}])
    assert msgs[0]["role"] == "user" and msgs[0]["content"] == api.COMPACT_PREFIX + summary and msgs[1]["content"] == "continue"
    st, _, raw = call(server, "POST", "/v1/responses", {"input": [item, {"role": "user", "content": "continue"}], "max_output_tokens": 4})
    assert st == 200 and json.loads(raw)["status"] in ("completed", "incomplete")
    bad = dict(item, encrypted_content="cafd1.not-base64!!")
    assert call(server, "POST", "/v1/responses", {"input": [bad], "max_output_tokens": 4})[0] == 400
    assert api.decode_opaque(api.encode_opaque("compaction", "héllo"), "compaction") == "héllo"
    with pytest.raises(api.BadRequest):
        api.decode_opaque(api.encode_opaque("other", "x"), "compaction")


def test_tool_call_stream_filter():
    from cuteafd_b200.serve.tokenizer import ToolCallStream, parse_tool_calls
    full = 'Let me look. <tool_call>{"name": "get_time", "arguments": {"tz": "UTC"}}</tool_call> and <tool_call>{"name": "x", "arguments": {}}</tool_call>done <tool'
    want_text, want_calls = parse_tool_calls(full)
    for step in (1, 3, 7, 1000):                                  # any chunking gives the same text and calls
        t = ToolCallStream()
        text, calls = [], []
        for i in range(0, len(full), step):
            v, c = t.push(full[i:i + step])
            assert "<tool_call>" not in v
            text.append(v)
            calls += c
        text.append(t.flush())
        assert "".join(text) == want_text and [c["function"] for c in calls] == [c["function"] for c in want_calls]
        assert [c["id"] for c in calls] == ["call_0", "call_1"]
    t = ToolCallStream()
    assert t.push("a < b and <to")[0] == "a < b and " and t.push("tal>")[0] == "<total>"      # a false start is released
    v, c = ToolCallStream().push("<tool_call>not json</tool_call>")
    assert v == "<tool_call>not json</tool_call>" and c == []
    t = ToolCallStream()
    t.push('x<tool_call>{"name"')
    assert t.flush() == '<tool_call>{"name"'                    # cut off mid-call: returned as text


def test_stop_stream_and_multi_token_stop(server):
    from cuteafd_b200.serve.tokenizer import StopStream
    for step in (1, 2, 5, 100):
        s, out = StopStream(["END", "\\n\\nUser:"]), []
        text = "line one\\nline two EN and then END never shown"
        for i in range(0, len(text), step):
            out.append(s.push(text[i:i + step]))
        out.append(s.flush())
        assert "".join(out) == "line one\\nline two EN and then " and s.hit == "END"
    s = StopStream(["xyz"])
    assert s.push("abcx") == "abc" and s.push("y") == "" and s.push("q") == "xyq" and s.flush() == "" and s.hit is None
    assert StopStream([]).push("anything") == "anything"
    # through the server: find a two-token string the greedy reply contains, then ask to stop at it
    body = {"messages": [{"role": "user", "content": "tell me something long"}], "max_tokens": 24, "temperature": 0}
    full = json.loads(call(server, "POST", "/v1/chat/completions", body)[2])
    text = full["choices"][0]["message"]["content"]
    assert len(text) >= 4
    stop = text[2:4]
    cut = json.loads(call(server, "POST", "/v1/chat/completions", dict(body, stop=[stop]))[2])
    got = cut["choices"][0]["message"]["content"]
    assert got == text[:text.index(stop)] and cut["choices"][0]["finish_reason"] == "stop"
    assert 0 < cut["usage"]["completion_tokens"] <= full["usage"]["completion_tokens"]
    assert call(server, "POST", "/v1/chat/completions", dict(body, stop=[1, 2]))[0] == 400


def test_prometheus_metrics(server):
    call(server, "POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "count"}], "max_tokens": 3})
    st, hd, raw = call(server, "GET", "/metrics")
    text = raw.decode()
    assert st == 200 and "text/plain" in hd.get("Content-Type", hd.get("content-type", ""))
    vals = {}
    for line in text.splitlines():
        assert line.startswith("#") or line.startswith("cuteafd_"), line
        if not line.startswith("#"):
            name, v = line.rsplit(" ", 1)
            vals[name] = float(v)
    assert vals["cuteafd_finished_total"] >= 1 and vals["cuteafd_emitted_tokens_total"] >= 1 and vals["cuteafd_ready"] == 1
    assert vals['cuteafd_kv_pages{kind="total"}'] > 0 and 'cuteafd_requests{state="decode"}' in vals
    assert text.count("# TYPE cuteafd_finished_total counter") == 1


def test_build_state_with_a_draft_model(tmp_path):
    from cuteafd_b200 import tiny_moe
    from cuteafd_b200.cli import build_parser
    from cuteafd_b200.loader import snapshot
    from cuteafd_b200.runtime.scheduler import Request, collect
    from cuteafd_b200.serve.server import build_state
    cfg = tiny_moe()
    tgt = snapshot.write_random_snapshot(cfg, str(tmp_path / "t"), fmt="bf16", seed=0)
    args = build_parser().parse_args(["serve", "--fake-engine", "--snapshot", tgt, "--speculator", "draft-model", "--draft-snapshot", tgt])
    state = build_state(args)
    assert type(state.sched.drafter).__name__ == "ModelDrafter"
    req = state.sched.submit(Request(list(range(1, 40)), max_tokens=12))
    for _ in range(400):
        if not state.sched.step() and not state.sched.decoding and not state.sched.prefilling and state.sched.waiting.empty() and not state.sched.pending:
            break
    out = collect(req, timeout=1.0)
    sp = out["usage"]["speculation"]
    assert len(out["tokens"]) == 12 and sp["accepted"] == sp["proposed"] > 0 and sp["cycles"] < 12     # the target drafting for itself


def test_gateway_streams(server):
    """Streaming clients of the translated flavours get their protocol's event sequence; a streamed request in the
    upstream's own protocol is passed through."""
    gw = Gateway(f"http://127.0.0.1:{server.port}", model_map={"claude-x": "tiny-moe"}).start()
    try:
        def post(path, body):
            c = http.client.HTTPConnection("127.0.0.1", gw.port, timeout=120)
            c.request("POST", path, json.dumps(body), {"Content-Type": "application/json", "Authorization": "Bearer sekret"})
            r = c.getresponse()
            return r.status, r.getheader("Content-Type"), r.read().decode()
        st, ct, raw = post("/v1/messages", {"model": "claude-x", "max_tokens": 5, "stream": True, "messages": [{"role": "user", "content": "hi"}]})
        names = [l[7:] for l in raw.splitlines() if l.startswith("event: ")]
        assert st == 200 and "event-stream" in ct
        assert names[0] == "message_start" and names[-2:] == ["message_delta", "message_stop"] and "content_block_delta" in names
        st, ct, raw = post("/v1/responses", {"model": "tiny-moe", "max_output_tokens": 5, "stream": True, "input": "hi"})
        names = [l[7:] for l in raw.splitlines() if l.startswith("event: ")]
        assert names[0] == "response.created" and names[-1] == "response.completed" and "response.output_text.delta" in names
        done = json.loads([l for l in raw.splitlines() if l.startswith("data: ")][-1][6:])
        assert done["response"]["status"] in ("completed", "incomplete") and done["response"]["usage"]["output_tokens"] >= 1
        st, ct, raw = post("/v1/chat/completions", {"model": "tiny-moe", "max_tokens": 4, "stream": True, "messages": [{"role": "user", "content": "hi"}]})
        assert st == 200 and "event-stream" in ct and raw.rstrip().endswith("data: [DONE]") and "chat.completion.chunk" in raw
    finally:
        gw.stop()


def test_gateway_get_carries_the_key(server):
    gw = Gateway(f"http://127.0.0.1:{server.port}").start()
    try:
        def get(path, key):
            c = http.client.HTTPConnection("127.0.0.1", gw.port, timeout=30)
            c.request("GET", path, headers={"Authorization": f"Bearer {key}"} if key else {})
            r = c.getresponse()
            return r.status, json.loads(r.read())
        st, models = get("/v1/models", "sekret")
        assert st == 200 and models["data"][0]["id"] == "tiny-moe"
        assert get("/v1/models", "wrong")[0] == 401 and get("/v1/models", "")[0] == 401
    finally:
        gw.stop()


def test_deployment_cap_on_output_tokens():
    """MAX_OUTPUT_TOKENS: the most a request may ask for, and what a request that names no limit gets."""
    from cuteafd_b200.serve import api
    from cuteafd_b200.serve.tokenizer import load_tokenizer
    tok = load_tokenizer(None, 512)
    body = {"messages": [{"role": "user", "content": "hi"}]}
    assert api.build_request(body, tok, 512).max_tokens == 256
    assert api.build_request(body, tok, 512, max_output_tokens=40).max_tokens == 40
    assert api.build_request(dict(body, max_tokens=1000), tok, 512, max_output_tokens=40).max_tokens == 40
    assert api.build_request(dict(body, max_tokens=7), tok, 512, max_output_tokens=40).max_tokens == 7
    with pytest.raises(api.BadRequest):
        api.build_request(dict(body, max_tokens=True), tok, 512)
