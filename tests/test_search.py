"""Hosted web search: providers against local stand-in services, the session cache, the gateway's tool loop."""
import http.client
import json
import threading
import urllib.parse
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

import pytest

from cuteafd_b200.serve import search
from cuteafd_b200.serve.gateway import Gateway
from cuteafd_b200.serve.search import Exa, SearchQuery, SearchSession, Searxng, alpha_search, domain_ok

PAGES = [
    {"url": "https://docs.example.org/tma", "title": "TMA notes", "text": "Bulk tensor copies need 16-byte aligned starts. " * 3,
     "publishedDate": "2025-03-01"},
    {"url": "https://blog.other.net/post", "title": "Other post", "text": "Unrelated text about gardening."},
    {"url": "https://sub.example.org/x", "title": "Sub page", "text": "More about tensor memory and alignment."},
]


class Service:
    """One listener that plays Exa, SearXNG and an OpenAI-compatible upstream."""

    def __init__(self):
        svc = self
        self.seen = []
        self.turns = 0

        class H(BaseHTTPRequestHandler):
            protocol_version = "HTTP/1.1"

            def log_message(self, *a): return

            def _send(self, st, obj):
                raw = json.dumps(obj).encode()
                self.send_response(st); self.send_header("Content-Length", str(len(raw))); self.end_headers(); self.wfile.write(raw)

            def do_GET(self):
                u = urllib.parse.urlparse(self.path)
                q = urllib.parse.parse_qs(u.query)
                svc.seen.append(("searxng", q))
                self._send(200, {"results": [{"url": p["url"], "title": p["title"], "content": p["text"][:40]} for p in PAGES]})

            def do_POST(self):
                body = json.loads(self.rfile.read(int(self.headers["Content-Length"])))
                if self.path == "/search":
                    if self.headers.get("x-api-key") != "k":
                        return self._send(401, {"error": "bad key"})
                    svc.seen.append(("exa", body))
                    res = [p for p in PAGES if not body.get("includeDomains") or any(d in p["url"] for d in body["includeDomains"])]
                    return self._send(200, {"results": res[: body["numResults"]]})
                # chat upstream: first turn asks for a search, second answers from the tool message
                svc.seen.append(("chat", body))
                svc.turns += 1
                tool_msgs = [m for m in body["messages"] if m["role"] == "tool"]
                if not tool_msgs and any(t["function"]["name"] == "get_time" for t in body.get("tools", [])):
                    msg = {"role": "assistant", "content": "one moment", "tool_calls": [
                        {"id": "c9", "type": "function", "function": {"name": "get_time", "arguments": '{"tz": "UTC"}'}}]}
                    fin = "tool_calls"
                elif not tool_msgs and any(t["function"]["name"] == "web_search" for t in body.get("tools", [])):
                    msg = {"role": "assistant", "content": "", "tool_calls": [
                        {"id": "c1", "type": "function", "function": {"name": "web_search", "arguments": json.dumps({"query": "tma alignment"})}}]}
                    fin = "tool_calls"
                else:
                    msg = {"role": "assistant", "content": "answer using " + (tool_msgs[-1]["content"][:30] if tool_msgs else "nothing")}
                    fin = "stop"
                self._send(200, {"choices": [{"index": 0, "message": msg, "finish_reason": fin}],
                                 "usage": {"prompt_tokens": 5, "completion_tokens": 3}})

        self.httpd = ThreadingHTTPServer(("127.0.0.1", 0), H)
        self.httpd.daemon_threads = True
        self.port = self.httpd.server_address[1]
        threading.Thread(target=self.httpd.serve_forever, daemon=True).start()

    def stop(self):
        self.httpd.shutdown(); self.httpd.server_close()


@pytest.fixture()
def svc():
    s = Service()
    yield s
    s.stop()


def test_domain_filter():
    q = SearchQuery("x", allowed_domains=["example.org"], blocked_domains=["sub.example.org"])
    assert domain_ok("https://docs.example.org/a", q) and not domain_ok("https://sub.example.org/a", q)
    assert not domain_ok("https://notexample.org/", q) and domain_ok("https://example.org", q)


def test_providers_speak_their_wire_formats(svc):
    base = f"http://127.0.0.1:{svc.port}"
    hits = Exa("k", base).search(SearchQuery("tma", allowed_domains=["example.org"], max_results=2))
    kind, sent = svc.seen[-1]
    assert kind == "exa" and sent["numResults"] == 2 and sent["includeDomains"] == ["example.org"] and "text" in sent["contents"]
    assert [h.url for h in hits] == [PAGES[0]["url"], PAGES[2]["url"]] and hits[0].published == "2025-03-01"
    with pytest.raises(search.SearchError, match="401"):
        Exa("wrong", base).search(SearchQuery("tma"))
    hits = Searxng(base).search(SearchQuery("tma", blocked_domains=["other.net"]), recency_days=3)
    kind, sent = svc.seen[-1]
    assert kind == "searxng" and sent["format"] == ["json"] and sent["time_range"] == ["week"]
    assert [h.url for h in hits] == [PAGES[0]["url"], PAGES[2]["url"]]
    with pytest.raises(search.SearchError, match="unavailable"):
        Searxng("http://127.0.0.1:9", timeout=0.5).search(SearchQuery("x"))


def test_session_cache_refs_find_and_expiry(svc):
    now = [0.0]
    ses = SearchSession(clock=lambda: now[0])
    prov = Exa("k", f"http://127.0.0.1:{svc.port}")
    out = alpha_search(prov, ses, {"command": "search", "query": "tma", "max_results": 3})
    assert out["ok"] and [r["ref"] for r in out["results"]] == ["ref_1", "ref_2", "ref_3"]
    again = alpha_search(prov, ses, {"query": "tma"})
    assert [r["ref"] for r in again["results"]] == ["ref_1", "ref_2", "ref_3"]            # the same page keeps its reference
    assert alpha_search(prov, ses, {"command": "open", "ref": "ref_1"})["page"]["title"] == "TMA notes"
    m = alpha_search(prov, ses, {"command": "find", "ref": "ref_1", "pattern": "16-BYTE"})
    assert m["ok"] and len(m["matches"]) == 3 and "aligned" in m["matches"][0]
    assert not alpha_search(prov, ses, {"command": "open", "url": "https://never.seen/"})["ok"]     # never fetched for the client
    assert alpha_search(prov, ses, {"command": "time"})["utc"].endswith("Z")
    assert "unsupported" in alpha_search(prov, ses, {"command": "screenshot"})["output"]
    assert "no search provider" in alpha_search(None, ses, {"query": "x"})["output"]
    now[0] = 3601.0
    assert not alpha_search(prov, ses, {"command": "open", "ref": "ref_1"})["ok"]


def test_gateway_runs_the_search_the_model_asks_for(svc):
    base = f"http://127.0.0.1:{svc.port}"
    gw = Gateway(base, provider=Exa("k", base)).start()
    try:
        def post(path, body):
            c = http.client.HTTPConnection("127.0.0.1", gw.port, timeout=30)
            c.request("POST", path, json.dumps(body), {"Content-Type": "application/json"})
            r = c.getresponse()
            return r.status, json.loads(r.read())
        st, out = post("/v1/messages", {"model": "m", "max_tokens": 64, "messages": [{"role": "user", "content": "how must TMA copies start?"}],
                                        "tools": [{"type": "web_search_20250305", "name": "web_search", "max_uses": 2,
                                                   "allowed_domains": ["example.org"]}]})
        assert st == 200 and svc.turns == 2
        kinds = [b["type"] for b in out["content"]]
        assert kinds[:2] == ["server_tool_use", "web_search_tool_result"] and kinds[-1] == "text"
        assert out["content"][0]["input"] == {"query": "tma alignment"}
        assert [r["url"] for r in out["content"][1]["content"]] == [PAGES[0]["url"], PAGES[2]["url"]]
        assert out["content"][-1]["text"].startswith("answer using [ref_1] TMA notes")
        assert out["usage"]["server_tool_use"] == {"web_search_requests": 1}
        # the second upstream turn carried the assistant's call and the tool result
        chat_bodies = [b for k, b in svc.seen if k == "chat"]
        assert [m["role"] for m in chat_bodies[-1]["messages"]][-2:] == ["assistant", "tool"]
        # Responses flavour gets web_search_call items; no declaration = no tool, one turn
        svc.turns = 0
        st, out = post("/v1/responses", {"model": "m", "input": "q", "tools": [{"type": "web_search"}]})
        assert st == 200 and out["output"][0]["type"] == "web_search_call" and out["output"][0]["action"]["query"] == "tma alignment"
        svc.turns = 0
        st, out = post("/v1/responses", {"model": "m", "input": "q"})
        assert st == 200 and svc.turns == 1 and all(o["type"] != "web_search_call" for o in out["output"])
        st, out = post("/v1/alpha/search", {"command": "search", "query": "tma"})
        assert st == 200 and out["ok"] and out["provider"] == "exa"
    finally:
        gw.stop()


def test_gateway_forwards_client_tools_and_returns_calls(svc):
    base = f"http://127.0.0.1:{svc.port}"
    gw = Gateway(base).start()
    try:
        c = http.client.HTTPConnection("127.0.0.1", gw.port, timeout=30)
        body = {"model": "m", "max_tokens": 32, "messages": [{"role": "user", "content": [{"type": "text", "text": "time?"}]}],
                "tools": [{"name": "get_time", "description": "now", "input_schema": {"type": "object", "properties": {"tz": {"type": "string"}}}}]}
        c.request("POST", "/v1/messages", json.dumps(body), {"Content-Type": "application/json"})
        out = json.loads(c.getresponse().read())
        sent = [b for k, b in svc.seen if k == "chat"][-1]
        assert sent["tools"][0]["function"]["name"] == "get_time" and sent["messages"][0]["content"] == "time?"
        kinds = [b["type"] for b in out["content"]]
        assert kinds == ["text", "tool_use"] and out["content"][1]["name"] == "get_time" and out["content"][1]["input"] == {"tz": "UTC"}
        assert out["stop_reason"] == "tool_use"
        # the client answers with a tool_result: the upstream sees an assistant call and a tool turn
        body["messages"] += [{"role": "assistant", "content": out["content"]},
                             {"role": "user", "content": [{"type": "tool_result", "tool_use_id": out["content"][1]["id"], "content": "12:00"}]}]
        c.request("POST", "/v1/messages", json.dumps(body), {"Content-Type": "application/json"})
        out2 = json.loads(c.getresponse().read())
        sent = [b for k, b in svc.seen if k == "chat"][-1]
        assert [m["role"] for m in sent["messages"]] == ["user", "assistant", "tool"] and sent["messages"][2]["content"] == "12:00"
        assert out2["content"][-1]["text"].startswith("answer using 12:00")
    finally:
        gw.stop()
