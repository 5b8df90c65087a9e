"""Standalone protocol gateway: accepts Anthropic Messages and OpenAI Responses requests and
forwards them as OpenAI Chat Completions to an upstream server, translating the reply back.
A model-name map renames client model ids.  Hosted web search (``serve/search.py``): when the client declares a
server-side search tool the gateway runs the searches the model asks for, and ``POST /v1/alpha/search`` serves the
search / open / find / time commands of client-executed search extensions.  (The in-process server already speaks all three
protocols; the gateway exists for fronting any OpenAI-compatible upstream.)

Counterpart: rust/crates/cuteafd-api/src/gateway/mod.rs:1-60,148,215-216 and
rust/crates/cuteafd-daemon/src/commands/gateway.rs.
"""
from __future__ import annotations

import json
import threading
import urllib.error
import urllib.request
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

from . import api, search


def _flatten(content):
    """Text parts of any flavour -> one string (an OpenAI-compatible upstream takes plain strings everywhere)."""
    if isinstance(content, list):
        return "".join(p.get("text", "") for p in content if isinstance(p, dict) and p.get("type") in ("text", "input_text", "output_text"))
    return content if content is not None else ""


def to_chat_body(body: dict, flavor: str, model_map: dict[str, str]) -> dict:
    if flavor == "anthropic":
        msgs = api.anthropic_messages(body)
    else:
        msgs = api.responses_messages(body)
    msgs = [dict(m, content=_flatten(m.get("content"))) for m in msgs]
    out = {"model": model_map.get(body.get("model", ""), body.get("model", "")), "messages": msgs,
           "max_tokens": body.get("max_tokens") or body.get("max_output_tokens") or 256}
    tools = api.normalize_tools(body.get("tools"), flavor)          # hosted tool types are handled by the gateway itself
    if tools:
        out["tools"] = tools
        from .constraints import tool_choice_of
        mode, name, parallel = tool_choice_of(body, flavor)        # any protocol's spelling -> the chat one
        if mode != "auto":
            out["tool_choice"] = {"type": "function", "function": {"name": name}} if mode == "named" else mode
        if not parallel:
            out["parallel_tool_calls"] = False
    for k in ("temperature", "top_p", "top_k", "seed", "stop"):
        if k in body:
            out[k] = body[k]
    if body.get("stop_sequences"):
        out["stop"] = body["stop_sequences"]
    return out


def from_chat_reply(reply: dict, flavor: str, model: str) -> dict:
    ch = reply["choices"][0]
    text = ch["message"].get("content") or ""
    for c in ch["message"].get("tool_calls") or []:                 # back into the inline form the reply builders parse
        fn = c.get("function", {})
        try:
            args = json.loads(fn.get("arguments") or "{}")
        except json.JSONDecodeError:
            args = {}
        text += "<tool_call>" + json.dumps({"name": fn.get("name", ""), "arguments": args}) + "</tool_call>"
    u = reply.get("usage", {})
    usage = {"prompt_tokens": u.get("prompt_tokens", 0), "completion_tokens": u.get("completion_tokens", 0),
             "cached_tokens": u.get("prompt_tokens_details", {}).get("cached_tokens", 0)}
    if flavor == "anthropic":
        return api.anthropic_message(model, text, ch.get("finish_reason", "stop"), usage)
    return api.responses_object(model, text, ch.get("finish_reason", "stop"), usage)


class Tape:
    """Record / replay of upstream exchanges.  ``record``: every forwarded request body and the reply it got are appended
    to a JSONL file.  ``replay``: replies come from the file, matched by the hash of the forwarded body, and the
    upstream is never contacted (client tests and demos without an engine).  Counterpart: the gateway's record/replay
    mode (rust/crates/cuteafd-api/src/gateway/mod.rs)."""

    def __init__(self, path: str, mode: str):
        assert mode in ("record", "replay")
        self.path, self.mode = path, mode
        self.lock = threading.Lock()
        self.replies: dict[str, list] = {}
        if mode == "replay":
            with open(path) as f:
                for line in f:
                    rec = json.loads(line)
                    self.replies.setdefault(rec["key"], []).append(rec)

    @staticmethod
    def key(path: str, body: dict) -> str:
        import hashlib
        return hashlib.sha256((path + "\n" + json.dumps(body, sort_keys=True)).encode()).hexdigest()

    def store(self, path: str, body: dict, status: int, reply: dict) -> None:
        with self.lock, open(self.path, "a") as f:
            f.write(json.dumps({"key": self.key(path, body), "path": path, "request": body, "status": status, "reply": reply}) + "\n")

    def fetch(self, path: str, body: dict):
        """(status, reply) of the recorded exchange; repeated identical requests walk their recordings in order and
        stay on the last one."""
        with self.lock:
            recs = self.replies.get(self.key(path, body))
            if not recs:
                return None
            rec = recs.pop(0) if len(recs) > 1 else recs[0]
        return rec["status"], rec["reply"]


class _UpstreamFailed(Exception):
    pass


def sse_events(out: dict, flavor: str) -> list[tuple[str, dict]]:
    """A finished reply as the event sequence a streaming client of that flavour expects.  The gateway asks its upstream
    for whole replies (so that it can run hosted tools between turns) and replays them as one-delta streams: the
    protocol is the streaming one, the text arrives in one piece."""
    ev: list[tuple[str, dict]] = []
    if flavor == "anthropic":
        head = dict(out, content=[], stop_reason=None)
        ev.append(("message_start", {"type": "message_start", "message": head}))
        for i, b in enumerate(out.get("content", [])):
            if b.get("type") == "text":
                ev.append(("content_block_start", {"type": "content_block_start", "index": i, "content_block": {"type": "text", "text": ""}}))
                ev.append(("content_block_delta", {"type": "content_block_delta", "index": i, "delta": {"type": "text_delta", "text": b.get("text", "")}}))
            elif b.get("type") == "tool_use":
                ev.append(("content_block_start", {"type": "content_block_start", "index": i, "content_block": dict(b, input={})}))
                ev.append(("content_block_delta", {"type": "content_block_delta", "index": i,
                                                   "delta": {"type": "input_json_delta", "partial_json": json.dumps(b.get("input", {}))}}))
            else:                                                   # server tool blocks travel whole
                ev.append(("content_block_start", {"type": "content_block_start", "index": i, "content_block": b}))
            ev.append(("content_block_stop", {"type": "content_block_stop", "index": i}))
        ev.append(("message_delta", {"type": "message_delta", "delta": {"stop_reason": out.get("stop_reason")},
                                     "usage": {"output_tokens": out.get("usage", {}).get("output_tokens", 0)}}))
        ev.append(("message_stop", {"type": "message_stop"}))
        return ev
    ev.append(("response.created", {"type": "response.created", "response": {"id": out["id"], "status": "in_progress"}}))
    for i, item in enumerate(out.get("output", [])):
        ev.append(("response.output_item.added", {"type": "response.output_item.added", "output_index": i, "item": item}))
        if item.get("type") == "message":
            for part in item.get("content", []):
                if part.get("type") == "output_text":
                    ev.append(("response.output_text.delta", {"type": "response.output_text.delta", "output_index": i, "delta": part.get("text", "")}))
        elif item.get("type") == "function_call":
            ev.append(("response.function_call_arguments.done", {"type": "response.function_call_arguments.done", "output_index": i,
                                                                 "name": item.get("name"), "arguments": item.get("arguments")}))
        ev.append(("response.output_item.done", {"type": "response.output_item.done", "output_index": i, "item": item}))
    ev.append(("response.completed", {"type": "response.completed", "response": out}))
    return ev


def attach_searches(out: dict, flavor: str, ran: list[dict]) -> None:
    """Show the client the searches the gateway ran for it, in its own protocol's block types."""
    if flavor == "anthropic":
        blocks = []
        for i, r in enumerate(ran):
            tid = f"srvtoolu_{i}"
            blocks.append({"type": "server_tool_use", "id": tid, "name": "web_search", "input": {"query": r["query"]}})
            blocks.append({"type": "web_search_tool_result", "tool_use_id": tid,
                           "content": [{"type": "web_search_result", "url": h["url"], "title": h["title"],
                                        "page_age": h.get("published")} for h in r["results"]]})
        out["content"] = blocks + out.get("content", [])
        out.setdefault("usage", {})["server_tool_use"] = {"web_search_requests": len(ran)}
    else:
        items = [{"type": "web_search_call", "id": f"ws_{i}", "status": "completed", "action": {"type": "search", "query": r["query"]}}
                 for i, r in enumerate(ran)]
        out["output"] = items + out.get("output", [])


def make_gateway(upstream: str, model_map: dict[str, str], tape: "Tape | None" = None, provider=None):
    sessions: dict = {}
    sessions_lock = threading.Lock()

    class H(BaseHTTPRequestHandler):
        protocol_version = "HTTP/1.1"

        def log_message(self, *a):
            return

        def _json(self, status, body, headers=None):
            raw = json.dumps(body).encode()
            self.send_response(status)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(raw)))
            for k, v in (headers or {}).items():
                self.send_header(k, v)
            self.end_headers()
            self.wfile.write(raw)

        def do_GET(self):
            try:
                req = urllib.request.Request(upstream + self.path, headers={"Authorization": self.headers.get("Authorization", "")})
                with urllib.request.urlopen(req, timeout=30) as r:
                    return self._json(r.status, json.loads(r.read()))
            except urllib.error.HTTPError as e:
                try:
                    return self._json(e.code, json.loads(e.read() or b"{}"))
                except json.JSONDecodeError:
                    return self._json(e.code, {"error": {"message": f"upstream answered {e.code}"}})
            except urllib.error.URLError as e:
                return self._json(503, {"error": {"message": f"upstream unavailable: {e}"}})

        def _sse_all(self, events: list) -> None:
            self.send_response(200)
            self.send_header("Content-Type", "text/event-stream")
            self.send_header("Cache-Control", "no-cache")
            self.send_header("Connection", "close")
            self.end_headers()
            for name, ev in events:
                self.wfile.write(f"event: {name}\ndata: {json.dumps(ev)}\n\n".encode())
            self.wfile.flush()
            self.close_connection = True

        def _proxy_stream(self, fpath: str, fwd: dict) -> None:
            """A streamed request in the upstream's own protocol: bytes are passed through as they arrive."""
            req = urllib.request.Request(upstream + fpath, json.dumps(fwd).encode(),
                                         {"Content-Type": "application/json", "Authorization": self.headers.get("Authorization", "")})
            try:
                r = urllib.request.urlopen(req, timeout=600)
            except urllib.error.HTTPError as e:
                return self._json(e.code, json.loads(e.read() or b"{}"))
            except urllib.error.URLError as e:
                return self._json(503, {"error": {"message": f"upstream unavailable: {e}"}})
            with r:
                self.send_response(r.status)
                self.send_header("Content-Type", r.headers.get("Content-Type", "text/event-stream"))
                self.send_header("Cache-Control", "no-cache")
                self.send_header("Connection", "close")
                self.end_headers()
                while True:
                    chunk = r.read1(65536) if hasattr(r, "read1") else r.read(65536)
                    if not chunk:
                        break
                    self.wfile.write(chunk)
                    self.wfile.flush()
            self.close_connection = True

        def _session(self, body: dict) -> "search.SearchSession":
            key = (self.headers.get("Authorization", ""), str(body.get("session_id") or body.get("previous_response_id") or ""))
            with sessions_lock:
                if len(sessions) > 1024:
                    sessions.clear()
                return sessions.setdefault(key, search.SearchSession())

        def _chat(self, fpath: str, fwd: dict) -> tuple[int, dict, dict]:
            """One upstream exchange (or its recording): (status, reply, headers to pass on)."""
            if tape is not None and tape.mode == "replay":
                hit = tape.fetch(fpath, fwd)
                if hit is None:
                    return 404, {"error": {"message": "no recorded exchange for this request", "type": "replay_miss"}}, {}
                return hit[0], hit[1], {}
            req = urllib.request.Request(upstream + fpath, json.dumps(fwd).encode(),
                                         {"Content-Type": "application/json", "Authorization": self.headers.get("Authorization", "")})
            try:
                with urllib.request.urlopen(req, timeout=600) as r:
                    reply = json.loads(r.read())
            except urllib.error.HTTPError as e:
                hd = {"Retry-After": e.headers["Retry-After"]} if e.headers.get("Retry-After") else {}
                return e.code, json.loads(e.read() or b"{}"), hd
            except urllib.error.URLError as e:
                return 503, {"error": {"message": f"upstream unavailable: {e}"}}, {}
            if tape is not None:
                tape.store(fpath, fwd, 200, reply)
            return 200, reply, {}

        def do_POST(self):
            path = self.path.split("?")[0]
            flavor = {"/v1/messages": "anthropic", "/v1/responses": "responses"}.get(path)
            n = int(self.headers.get("Content-Length", "0") or 0)
            try:
                body = json.loads(self.rfile.read(n) or b"{}")
            except json.JSONDecodeError:
                return self._json(400, {"error": {"message": "invalid JSON"}})
            if path == "/v1/alpha/search":
                return self._json(200, search.alpha_search(provider, self._session(body), body))
            fwd = to_chat_body(body, flavor, model_map) if flavor else body
            fpath = "/v1/chat/completions" if flavor else self.path
            if not flavor and body.get("stream") and not (tape is not None and tape.mode == "replay"):
                return self._proxy_stream(fpath, fwd)
            decl = search.wants_hosted_search(body) if flavor else None
            ran: list[dict] = []
            if decl is not None and provider is not None:
                failed: list = []

                def chat(b: dict) -> dict:
                    st, reply, hd = self._chat(fpath, b)
                    if st != 200:
                        failed.append((st, reply, hd))
                        raise _UpstreamFailed()
                    return reply
                try:
                    reply, ran = search.run_tool_loop(chat, fwd, decl, provider, self._session(body))
                except _UpstreamFailed:
                    st, reply, hd = failed[0]
                    return self._json(st, reply, hd)
            else:
                st, reply, hd = self._chat(fpath, fwd)
                if st != 200:
                    return self._json(st, reply, hd)
            if not flavor:
                return self._json(200, reply)
            out = from_chat_reply(reply, flavor, body.get("model", ""))
            if ran:
                attach_searches(out, flavor, ran)
            if body.get("stream"):
                return self._sse_all(sse_events(out, flavor))
            return self._json(200, out)

    return H


class Gateway:
    def __init__(self, upstream: str, host: str = "127.0.0.1", port: int = 0, model_map: dict[str, str] | None = None,
                 tape: Tape | None = None, provider=None):
        self.httpd = ThreadingHTTPServer((host, port), make_gateway(upstream.rstrip("/"), model_map or {}, tape, provider))
        self.httpd.daemon_threads = True
        self.port = self.httpd.server_address[1]
        self.thread = threading.Thread(target=self.httpd.serve_forever, daemon=True)

    def start(self) -> "Gateway":
        self.thread.start()
        return self

    def stop(self) -> None:
        self.httpd.shutdown()
        self.httpd.server_close()


def run_gateway(args) -> int:
    import time
    mm = dict(kv.split("=", 1) for kv in args.model_map.split(",") if "=" in kv)
    tape = None
    if getattr(args, "record", ""):
        tape = Tape(args.record, "record")
    elif getattr(args, "replay", ""):
        tape = Tape(args.replay, "replay")
    import os
    provider = search.provider_from_env(dict(os.environ))        # EXA_API_KEY / SEARXNG_URL
    gw = Gateway(args.upstream, args.host, args.port, mm, tape, provider).start()
    print(f"gateway on http://{args.host}:{gw.port} -> {args.upstream}", flush=True)
    try:
        while True:
            time.sleep(3600)
    except KeyboardInterrupt:
        gw.stop()
    return 0
