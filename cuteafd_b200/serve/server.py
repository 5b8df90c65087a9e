"""HTTP serving: OpenAI Chat Completions (JSON and SSE), Anthropic Messages, OpenAI Responses,
models, health, stats, thermal, fabric, memory, experts, usage, and a minimal console.

Routes mirror the reference's router (rust/crates/cuteafd-api/src/openai.rs:448-474;
api/gateway/anthropic.rs:25-26; api/gateway/responses.rs:38-45; usage/http.rs:53-66).  Requests are
handed to the scheduler thread through its queue; each handler thread drains its own event queue.
The server is plain ``http.server`` threads: the data plane is the GPU, not the HTTP layer.
"""
from __future__ import annotations

import hmac
import json
import os
import threading
import time
import uuid
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

from ..runtime.scheduler import FAIL_BAD_REQUEST, FAIL_UNAVAILABLE, Request, Scheduler
from . import api, ws
from .tokenizer import StopStream, StreamDecoder, ToolCallStream

class ServerState:
    def __init__(self, scheduler: Scheduler, tokenizer, model_id: str, api_key: str = "", usage=None, extras=None, media=None):
        self.sched, self.tok, self.model_id, self.api_key = scheduler, tokenizer, model_id, api_key
        self.media = media                  # MediaProcessor, or None for a text-only deployment
        self.usage = usage
        self.extras = extras or {}
        if "expert_usage" not in self.extras and hasattr(scheduler.be, "expert_usage"):
            self.extras["expert_usage"] = scheduler.be.expert_usage        # /experts and the console read the backend's counters
        self.started = time.time()
        self.responses: dict[str, dict] = {}
        self.sessions: dict[str, list] = {}      # response id -> the conversation that produced it, reply included
        self.lock = threading.Lock()


def make_handler(state: ServerState):
    class Handler(BaseHTTPRequestHandler):
        protocol_version = "HTTP/1.1"
        server_version = "cuteafd_b200"

        def log_message(self, fmt, *args):      # quiet
            return

        # ---- helpers ------------------------------------------------------------------------------
        def _json(self, status: int, body, headers: dict | None = None) -> None:
            raw = json.dumps(body).encode()
            self.send_response(status)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(raw)))
            for k, v in (headers or {}).items():
                self.send_header(k, v)
            self.end_headers()
            self.wfile.write(raw)

        def _authorized(self) -> bool:
            if not state.api_key:
                return True
            got = self.headers.get("Authorization", "").removeprefix("Bearer ").strip() or self.headers.get("x-api-key", "")
            return hmac.compare_digest(got, state.api_key)

        def _body(self) -> dict:
            n = int(self.headers.get("Content-Length", "0") or 0)
            if n > 64 << 20:
                raise api.BadRequest("request body too large")
            raw = self.rfile.read(n) if n else b"{}"
            try:
                d = json.loads(raw or b"{}")
            except json.JSONDecodeError as e:
                raise api.BadRequest(f"invalid JSON: {e}") from e
            if not isinstance(d, dict):
                raise api.BadRequest("body must be a JSON object")
            return d

        def _sse_start(self) -> None:
            self.send_response(200)
            self.send_header("Content-Type", "text/event-stream")
            self.send_header("Cache-Control", "no-cache")
            self.send_header("Connection", "close")
            self.end_headers()

        def _sse(self, data, event: str | None = None) -> None:
            msg = (f"event: {event}\n" if event else "") + "data: " + (data if isinstance(data, str) else json.dumps(data)) + "\n\n"
            self.wfile.write(msg.encode())
            self.wfile.flush()

        # ---- GET ----------------------------------------------------------------------------------
        def do_GET(self):
            path = self.path.split("?", 1)[0]
            if path in ("/v1/realtime", "/v1/responses") and ws.wants_upgrade(self.headers):
                if not self._authorized():
                    return self._json(401, {"error": {"message": "invalid API key", "type": "authentication_error"}})
                sock = ws.upgrade(self)
                if sock is None:
                    return None
                if path == "/v1/realtime":
                    query = self.path.partition("?")[2]
                    model = next((kv[6:] for kv in query.split("&") if kv.startswith("model=")), None)
                    ws.serve_realtime(state, sock, model)
                else:
                    ws.serve_responses(state, sock)
                sock.close()
                return None
            if path == "/health":
                ok = state.sched.ready.is_set()
                return self._json(200 if ok else 503, {"status": "ok" if ok else "starting", "model": state.model_id})
            if path in ("/", "/v1/console"):
                from .console import PAGE
                raw = PAGE.encode()
                self.send_response(200)
                self.send_header("Content-Type", "text/html")
                self.send_header("Content-Length", str(len(raw)))
                self.end_headers()
                return self.wfile.write(raw)
            if not self._authorized():
                return self._json(401, {"error": {"message": "invalid API key", "type": "authentication_error"}})
            if path == "/v1/models":
                return self._json(200, {"object": "list", "data": [{"id": state.model_id, "object": "model", "created": int(state.started),
                                                                      "owned_by": "cuteafd_b200"}]})
            if path in ("/v1/console/state", "/v1/console/snapshot"):
                from .console import console_state
                return self._json(200, console_state(state))
            if path == "/v1/console/events":
                # the same document pushed as server-sent events (one per period) until the client goes away
                from .console import console_state
                q = dict(p.split("=", 1) for p in self.path.partition("?")[2].split("&") if "=" in p)
                period = min(10.0, max(0.05, float(q.get("period", 1.0))))
                count = min(3600, max(1, int(q.get("count", 3600))))
                self._sse_start()
                try:
                    for i in range(count):
                        self._sse(console_state(state), "snapshot")
                        if i + 1 < count:
                            time.sleep(period)
                except (BrokenPipeError, ConnectionResetError):
                    pass
                return None
            if path == "/console/memory":
                from ..utils.memory_ledger import LEDGER
                return self._json(200, LEDGER.report())
            if path == "/console/experts":
                return self._json(200, state.extras.get("expert_usage", lambda: {})())
            if path == "/v1/codex/models.json":
                # model catalog for clients that size their compaction from it: the served context window and reply limit
                be = state.sched.be
                window = int(getattr(be, "max_context_tokens", 0) or getattr(be, "max_pages", 0) * 64 or 16384)
                return self._json(200, {"models": [{"slug": state.model_id, "display_name": state.model_id, "context_window": window,
                                                    "max_output_tokens": min(window // 2, 32768), "supports_reasoning": False,
                                                    "supports_parallel_tool_calls": True, "wire_api": "responses"}]})
            if path == "/metrics":
                from .metrics import render
                raw = render(state).encode()
                self.send_response(200)
                self.send_header("Content-Type", "text/plain; version=0.0.4; charset=utf-8")
                self.send_header("Content-Length", str(len(raw)))
                self.end_headers()
                return self.wfile.write(raw)
            if path == "/v1/stats":
                s = state.sched.snapshot()
                be = state.sched.be
                if hasattr(be, "prefix"):
                    s["prefix"] = be.prefix.describe()
                if getattr(be, "tier", None) is not None:
                    s["host_tier"] = be.tier.describe()
                s["uptime_s"] = round(time.time() - state.started, 1)
                if getattr(state.sched, "profile", None) is not None:
                    s["profile"] = state.sched.profile.report()
                return self._json(200, s)
            if path == "/v1/thermal":
                from ..utils.thermal import monitor
                return self._json(200, monitor().report(60.0))
            if path == "/v1/fabric":
                from ..parallel.fabric import fabric_report
                return self._json(200, fabric_report())
            if path == "/memory":
                from ..utils.memory_ledger import LEDGER
                return self._json(200, LEDGER.report())
            if path == "/v1/media":
                return self._json(200, state.media.describe() if state.media else {"vision": False, "audio": False})
            if path == "/experts":
                return self._json(200, state.extras.get("expert_usage", lambda: {})())
            if path.startswith("/console/usage"):
                if not state.usage:
                    return self._json(200, {})
                q = dict(p.split("=", 1) for p in self.path.partition("?")[2].split("&") if "=" in p)
                tail = path[len("/console/usage"):].strip("/")
                if tail == "hourly":
                    return self._json(200, {"hourly": state.usage.hourly(int(q.get("hours", 24)))})
                if tail == "requests":
                    before = int(q["before"]) if "before" in q else None
                    return self._json(200, {"requests": state.usage.requests(int(q.get("limit", 50)), before)})
                if tail.startswith("request/"):
                    one = state.usage.request(int(tail.split("/", 1)[1])) if tail.split("/", 1)[1].isdigit() else None
                    return self._json(200, one) if one else self._json(404, {"error": {"message": "no such request"}})
                return self._json(200, state.usage.summary(float(q.get("hours", 24.0))))
            if path.startswith("/v1/responses/") and path.endswith("/input_items"):
                with state.lock:
                    conv = state.sessions.get(path.split("/")[3])
                if conv is None:
                    return self._json(404, {"error": {"message": "no such response"}})
                return self._json(200, api.input_items(conv[:-1]))
            if path.startswith("/v1/responses/"):
                rid = path.rsplit("/", 1)[1]
                with state.lock:
                    r = state.responses.get(rid)
                return self._json(200, r) if r else self._json(404, {"error": {"message": "no such response"}})
            return self._json(404, {"error": {"message": f"no route {path}"}})

        def do_DELETE(self):
            path = self.path.split("?", 1)[0]
            if path.startswith("/v1/responses/"):
                with state.lock:
                    ok = state.responses.pop(path.rsplit("/", 1)[1], None) is not None
                    state.sessions.pop(path.rsplit("/", 1)[1], None)
                return self._json(200 if ok else 404, {"deleted": ok})
            return self._json(404, {"error": {"message": "no route"}})

        # ---- POST ---------------------------------------------------------------------------------
        def do_POST(self):
            path = self.path.split("?", 1)[0]
            flavor = {"/v1/chat/completions": "openai", "/v1/messages": "anthropic", "/v1/responses": "responses",
                      "/v1/messages/count_tokens": "anthropic", "/v1/responses/input_tokens": "responses",
                      "/v1/responses/compact": "responses"}.get(path)
            if flavor is None and path.startswith("/v1/responses/") and path.endswith("/cancel"):
                flavor = "responses"
            if flavor is None and path != "/v1/fabric/phase":
                return self._json(404, {"error": {"message": f"no route {path}"}})
            if not self._authorized():
                st, body, hd = 401, {"error": {"message": "invalid API key", "type": "authentication_error"}}, {}
                return self._json(st, body, hd)
            if path == "/v1/fabric/phase":
                # a benchmark driver marks its phases; each mark closes the previous phase and returns what the
                # server saw during it (scheduler counters as deltas, the thermal window)
                try:
                    name = str(self._body().get("phase", ""))
                except api.BadRequest as e:
                    return self._json(400, {"error": {"message": str(e)}})
                from ..utils.thermal import monitor
                now, snap = time.monotonic(), state.sched.snapshot()
                with state.lock:
                    prev = state.extras.get("_phase")
                    state.extras["_phase"] = {"name": name, "t": now, "snap": snap}
                closed = None
                if prev:
                    keys = ("admitted", "finished", "failed", "rejected", "prefill_tokens", "cached_tokens", "decode_rounds",
                            "emitted_tokens", "verify_rows", "stalls")
                    closed = {"phase": prev["name"], "seconds": round(now - prev["t"], 3),
                              "delta": {k: snap.get(k, 0) - prev["snap"].get(k, 0) for k in keys},
                              "thermal": monitor().window(prev["t"], now)}
                return self._json(200, {"phase": name, "closed": closed})
            if path.startswith("/v1/responses/") and path.endswith("/cancel"):
                with state.lock:
                    r = state.responses.get(path.split("/")[3])
                # responses run in the foreground: by the time an id is known the response has completed
                return self._json(200, r) if r else self._json(404, {"error": {"message": "no such response"}})
            try:
                body = self._body()
                probe = api.parse_probe(self.headers)
                self._session = None
                if flavor == "responses":
                    with state.lock:
                        body, self._session = api.continue_session(body, state.sessions)
                self._compact = path == "/v1/responses/compact"
                if self._compact:
                    # the conversation plus one request for its summary; the reply is returned as an opaque item that a
                    # later request sends back in place of the turns it replaces
                    conv = body["input"] if isinstance(body.get("input"), list) else [{"role": "user", "content": body.get("input") or ""}]
                    body = dict(body, input=list(conv) + [{"role": "user", "content": api.COMPACT_REQUEST}], stream=False)
                    body.setdefault("max_output_tokens", 1024)
                req = api.build_request(body, state.tok, state.sched.be.vocab_size, probe, flavor, state.media,
                                        max_output_tokens=int(state.extras.get("max_output_tokens", 0) or 0))
            except api.BadRequest as e:
                st, eb, hd = api.error_body(FAIL_BAD_REQUEST, str(e), flavor)
                return self._json(st, eb, hd)
            if path.endswith("count_tokens") or path.endswith("input_tokens"):
                return self._json(200, {"input_tokens": len(req.prompt)})
            if not state.sched.ready.is_set():
                st, eb, hd = api.error_body(FAIL_UNAVAILABLE, "engine is starting", flavor)
                return self._json(st, eb, hd)
            t0 = time.time()
            state.sched.submit(req)
            model = body.get("model") or state.model_id
            self._acct = (model, flavor, t0, body)
            try:
                if body.get("stream"):
                    self._stream(req, model, flavor)
                else:
                    self._complete(req, model, flavor, t0)
            except (BrokenPipeError, ConnectionResetError):
                req.cancelled.set()                       # client went away: stop generating

        def _drain(self, req: Request):
            """Yield ("text", str) / ("done", finish, usage, rows) / ("error", kind, msg)."""
            dec = StreamDecoder(state.tok)
            eos = set(getattr(state.tok, "eos_ids", ()))
            said: list[str] = []
            first = None
            stopper = StopStream(getattr(req, "stop_texts", ()))
            while True:
                ev = req.events.get()
                if ev[0] == "tokens":
                    first = first or time.time()
                    text = stopper.push(dec.push([t for t in ev[1] if t not in eos]))
                    if text:
                        said.append(text)
                        yield ("text", text)
                    if stopper.hit is not None:
                        req.cancelled.set()                   # a stop string: nothing after it is generated or shown
                elif ev[0] == "done":
                    tail = stopper.push(dec.flush()) + stopper.flush()
                    if stopper.hit is not None:
                        ev = ("done", "stop", ev[2], ev[3] if len(ev) > 3 else [])
                    if tail:
                        said.append(tail)
                        yield ("text", tail)
                    acct = getattr(self, "_acct", None)
                    if state.usage and acct and ev[1] != "cancelled":       # streamed and plain replies both land here
                        model, flavor, t0, body = acct
                        state.usage.record(model, flavor, ev[2], time.time() - t0, ev[1], request=body, reply="".join(said),
                                           ttft=(first - t0) if first else None, client=self.client_address[0])
                    yield ev
                    return
                else:
                    yield ev
                    return

        def _complete(self, req: Request, model: str, flavor: str, t0: float) -> None:
            text, final = [], None
            for ev in self._drain(req):
                if ev[0] == "text":
                    text.append(ev[1])
                else:
                    final = ev
            if final[0] == "error":
                st, eb, hd = api.error_body(final[1], final[2], flavor)
                return self._json(st, eb, hd)
            _, finish, usage, rows = final
            out_text = "".join(text)
            if flavor == "anthropic":
                return self._json(200, api.anthropic_message(model, out_text, finish, usage))
            if flavor == "responses" and getattr(self, "_compact", False):
                if not out_text.strip():
                    return self._json(502, {"error": {"message": "compaction returned no summary", "type": "server_error"}})
                return self._json(200, api.compaction_object(out_text, usage))
            if flavor == "responses":
                obj = api.responses_object(model, out_text, finish, usage)
                with state.lock:
                    state.responses[obj["id"]] = obj
                    state.sessions[obj["id"]] = list(self._session or []) + [{"role": "assistant", "content": out_text}]
                return self._json(200, obj)
            lps = None
            if usage.get("top_rows") is not None:
                body = getattr(self, "_acct", (None, None, None, {}))[3] or {}
                if body.get("logprobs") or body.get("top_logprobs"):
                    lps = api.logprobs_block(state.tok, usage["top_rows"], int(body.get("top_logprobs") or 0))
            out = api.chat_completion(model, out_text, finish, usage, rows or None, lps)
            for key in ("score_rows", "state_hashes"):                             # probe diagnostics ride beside the reply
                if usage.get(key) is not None:
                    out.setdefault("probe", {})[key] = usage.pop(key)
            if usage.get("top_rows") is not None and lps is None:            # asked for through the probe header
                out.setdefault("probe", {})["top_rows"] = [{"token": t, "logprob": lp, "top_ids": ids, "top_logprobs": v}
                                                           for t, lp, ids, v in usage["top_rows"]]
            return self._json(200, out)

        def _stream(self, req: Request, model: str, flavor: str) -> None:
            self._sse_start()
            if flavor == "anthropic":
                mid, head = api.anthropic_events(model, len(req.prompt))
                for name, ev in head:
                    self._sse(ev, name)
                tcs, blocks = ToolCallStream(), 1

                def a_text(t: str) -> None:
                    if t:
                        self._sse({"type": "content_block_delta", "index": 0, "delta": {"type": "text_delta", "text": t}}, "content_block_delta")
                for ev in self._drain(req):
                    if ev[0] == "text":
                        vis, calls = tcs.push(ev[1])
                        a_text(vis)
                        for c in calls:                      # each call is its own tool_use block, its input one JSON delta
                            self._sse({"type": "content_block_start", "index": blocks, "content_block": {
                                "type": "tool_use", "id": "toolu_" + uuid.uuid4().hex[:20], "name": c["function"]["name"], "input": {}}},
                                "content_block_start")
                            self._sse({"type": "content_block_delta", "index": blocks,
                                       "delta": {"type": "input_json_delta", "partial_json": c["function"]["arguments"]}}, "content_block_delta")
                            self._sse({"type": "content_block_stop", "index": blocks}, "content_block_stop")
                            blocks += 1
                    elif ev[0] == "done":
                        a_text(tcs.flush())
                        self._sse({"type": "content_block_stop", "index": 0}, "content_block_stop")
                        stop = "tool_use" if tcs.calls else {"stop": "end_turn", "length": "max_tokens"}.get(ev[1], ev[1])
                        self._sse({"type": "message_delta", "delta": {"stop_reason": stop},
                                   "usage": {"output_tokens": ev[2].get("completion_tokens", 0)}}, "message_delta")
                        self._sse({"type": "message_stop"}, "message_stop")
                    else:
                        self._sse({"type": "error", "error": {"type": "api_error", "message": ev[2]}}, "error")
                return
            if flavor == "responses":
                rid = "resp_" + uuid.uuid4().hex[:24]
                self._sse({"type": "response.created", "response": {"id": rid, "status": "in_progress"}}, "response.created")
                text = []
                tcs = ToolCallStream()
                for ev in self._drain(req):
                    if ev[0] == "text":
                        text.append(ev[1])
                        vis, calls = tcs.push(ev[1])             # tool calls come as items of the completed response, not as text
                        if vis:
                            self._sse({"type": "response.output_text.delta", "delta": vis}, "response.output_text.delta")
                        for c in calls:
                            self._sse({"type": "response.function_call_arguments.done", "name": c["function"]["name"],
                                       "arguments": c["function"]["arguments"]}, "response.function_call_arguments.done")
                    elif ev[0] == "done":
                        rest = tcs.flush()
                        if rest:
                            self._sse({"type": "response.output_text.delta", "delta": rest}, "response.output_text.delta")
                        obj = api.responses_object(model, "".join(text), ev[1], ev[2], rid)
                        with state.lock:
                            state.responses[rid] = obj
                            state.sessions[rid] = list(getattr(self, "_session", None) or []) + [{"role": "assistant", "content": "".join(text)}]
                        self._sse({"type": "response.completed", "response": obj}, "response.completed")
                    else:
                        self._sse({"type": "error", "message": ev[2]}, "error")
                return
            cid = "chatcmpl-" + uuid.uuid4().hex[:24]
            self._sse(api.chat_chunk(cid, model, {"role": "assistant", "content": ""}))
            tcs = ToolCallStream()
            for ev in self._drain(req):
                if ev[0] == "text":
                    vis, calls = tcs.push(ev[1])
                    if vis:
                        self._sse(api.chat_chunk(cid, model, {"content": vis}))
                    for c in calls:
                        self._sse(api.chat_chunk(cid, model, {"tool_calls": [dict(c, index=tcs.calls - len(calls) + calls.index(c))]}))
                elif ev[0] == "done":
                    rest = tcs.flush()
                    if rest:
                        self._sse(api.chat_chunk(cid, model, {"content": rest}))
                    self._sse(api.chat_chunk(cid, model, {}, "tool_calls" if tcs.calls else ev[1], ev[2]))
                else:
                    self._sse({"error": {"message": ev[2], "code": ev[1]}})
            self._sse("[DONE]")

    return Handler


class Server:
    """Owns the HTTP listener and the scheduler thread."""

    def __init__(self, state: ServerState, host: str = "127.0.0.1", port: int = 0):
        self.state = state
        self.httpd = ThreadingHTTPServer((host, port), make_handler(state))
        self.httpd.daemon_threads = True
        self.port = self.httpd.server_address[1]
        self.t_http = threading.Thread(target=self.httpd.serve_forever, daemon=True)
        self.t_sched = threading.Thread(target=state.sched.run_forever, daemon=True)

    def start(self) -> "Server":
        self.t_sched.start()
        self.t_http.start()
        return self

    def stop(self) -> None:
        self.state.sched.stop()
        self.httpd.shutdown()
        self.httpd.server_close()


def build_state(args) -> ServerState:
    """Engine + scheduler + tokenizer from ``cuteafd serve`` arguments."""
    import torch

    from ..config import PRESETS, tiny_moe
    from ..runtime.speculation import NgramDrafter
    from .tokenizer import load_tokenizer
    from .usage import UsageLog
    snapshot = args.snapshot or None
    draft_len = max(1, min(int(getattr(args, "draft_length", 4) or 4), 16))      # tokens a drafter proposes per round
    if args.fake_engine or not torch.cuda.is_available():
        from ..ref.model import init_weights
        from ..runtime.backends import OracleBackend
        if snapshot:
            from ..loader.load import load_params
            cfg, params = load_params(snapshot)
        else:
            cfg = PRESETS.get(args.preset, tiny_moe)() if args.preset else tiny_moe()
            params = init_weights(cfg, seed=0)
        be = OracleBackend(cfg, params)
        if getattr(args, "expert_workers", ""):
            # routed experts on workers over TCP (``expertd --tcp-port``): each worker's plan hash covers its own range
            from ..parallel import wire
            workers = []
            for item in args.expert_workers.split(","):
                host, port, lo, hi = item.rsplit(":", 3)
                workers.append((host, int(port), int(lo), int(hi)))
            covered = sorted((lo, hi) for _, _, lo, hi in workers)
            if [lo for lo, _ in covered] != [0] + [hi for _, hi in covered[:-1]] or covered[-1][1] != cfg.num_experts:
                raise SystemExit(f"--expert-workers must partition the experts 0..{cfg.num_experts}; got {covered}")
            be.remote_experts = wire.RemoteExperts(
                workers, lambda lo, hi: wire.plan_hash({"model": cfg.name, "experts": cfg.num_experts, "range": [lo, hi]}))
            be.model.moe_fn = be.remote_experts
    else:
        if getattr(args, "expert_workers", ""):
            raise SystemExit("--expert-workers is wired to the host reference backend (--fake-engine); the CUDA engines "
                             "reach their expert ranks over NVLink (launch --expert-ranks N)")
        from ..runtime.backends import EngineBackend
        dev = torch.device("cuda:0")
        pages_per_seq = args.max_context_tokens // 64 + 2
        num_pages = pages_per_seq * args.concurrency + 64
        rows = args.concurrency * 8
        world = int(os.environ.get("WORLD_SIZE", "1"))
        if world > 1:
            # Disaggregated deployment (launched with one process per GPU): rank 0 runs attention, the dense backbone
            # and this HTTP server; the other ranks hold the routed experts and serve announced steps until rank 0
            # stops them.  The attention engine plugs into the same backend as the single-GPU engine.
            dep_engine = ""
            if getattr(args, "deployment", ""):
                with open(args.deployment) as f:
                    dep_engine = json.load(f).get("engine", "")
            if dep_engine == "tp":
                # Tensor-parallel attention group, experts on the same GPUs: rank 0 holds this scheduler and HTTP server,
                # the other ranks repeat its engine steps on their shard of the heads until it stops them.
                if getattr(args, "embedding_placement", "gpu") == "host":
                    raise SystemExit("--embedding-placement host is not available with a tensor-parallel attention group")
                args.host_cache_gib = 0.0           # a snapshot's pages differ per rank (each holds its own heads)
                cfg, eng = _build_tp_rank(args, snapshot, world, num_pages, rows)
            else:
                cfg, eng = _build_afd_rank(args, snapshot, world, num_pages, pages_per_seq, rows)
        elif snapshot:
            from ..loader.load import load_engine
            cfg, eng = load_engine(snapshot, dev, num_pages, max(2048, rows), rows, getattr(args, "kv_format", "auto"))
        else:
            cfg = PRESETS[args.preset or "qwen3-30b-a3b"]()
            if args.layers:
                cfg = cfg.replace(num_layers=args.layers)
            kvf = getattr(args, "kv_format", "auto")
            if cfg.is_mla and (kvf == "fp8_ds_mla" or (kvf == "auto" and cfg.indexer_heads)):
                cfg = cfg.replace(kv_format="fp8_ds_mla")
            if cfg.is_mla:
                from ..models.mla_moe import LatentCache as Cache, MlaMoeEngine as Engine, MlaMoeWeights as Weights
            else:
                from ..models.gqa_moe import GqaMoeEngine as Engine, GqaMoeWeights as Weights, KvCache as Cache
            eng = Engine(cfg, Weights.random_init(cfg, dev), Cache(cfg, num_pages, dev), max_tokens=max(2048, rows), max_seqs=rows)
        table = None
        if getattr(args, "embedding_placement", "gpu") == "host":
            if not snapshot:
                raise SystemExit("--embedding-placement host maps the table of a snapshot: give --snapshot")
            from ..loader.load import host_embedding_table
            table = host_embedding_table(snapshot)
            if not cfg.tie_embeddings:
                getattr(eng, "inner", eng).W.embed = None          # the device copy is not needed: free it
                torch.cuda.empty_cache()
        be = EngineBackend(eng, num_pages, pages_per_seq, prefill_chunk=2048, max_decode_rows=args.concurrency,
                           use_graphs=getattr(args, "decode_graphs", "on") != "off",
                           host_cache_bytes=int(float(getattr(args, "host_cache_gib", 0.0)) * (1 << 30)), host_embedding=table)
        if getattr(args, "prewarm", "") == "auto":              # no trace of an earlier run: the derived default list
            from ..planner.capacity import default_prewarm
            block = 0 if args.speculator == "off" else draft_len
            n = be.prewarm(default_prewarm(args.concurrency, block))
            print(f"prewarmed {n} decode graphs (default list)", flush=True)
        from ..utils.memory_ledger import LEDGER
        try:
            LEDGER.tag_tree("weights", "engine", eng.W)        # an arena's storage is already counted: adds nothing then
            LEDGER.tag_tree("kv", "engine", eng.kv)
            LEDGER.tag_tree("workspace", "engine", eng)
            LEDGER.tag_tree("workspace", "backend", be)
            if getattr(args, "memory_spool", ""):
                LEDGER.open_spool(args.memory_spool)
            for line in LEDGER.lines():
                print(line, flush=True)
        except Exception as e:                                 # noqa: BLE001 - accounting never stops a server from starting
            print(f"[memory] ledger unavailable: {e}", flush=True)
        pw = getattr(args, "prewarm", "")
        if pw and pw != "auto":
            if os.path.exists(pw):               # geometries a previous run saved (EngineBackend.save_prewarm)
                with open(pw) as f:
                    n = be.prewarm(json.load(f).get("geometries", []))
                print(f"prewarmed {n} decode graphs from {pw}", flush=True)
    be.prefix.max_entries = max(0, int(getattr(args, "prefix_cache_entries", 0) or 0))
    tok = load_tokenizer(snapshot, cfg.vocab_size)
    drafter = NgramDrafter(block=draft_len) if args.speculator in ("auto", "history", "ngram") else None
    if args.speculator in ("draft-model", "block-draft"):
        # a small checkpoint of the same vocabulary drafts the block: on the GPU next to the target when there is one
        # (its own engine and paged KV), else on the oracle decoder; "block-draft" produces the whole block in one pass
        # of the draft model (mask tokens after the last real one).  Verification by the target keeps the reply exact.
        from ..runtime.speculation import ModelDrafter
        if not getattr(args, "draft_snapshot", ""):
            raise SystemExit(f"--speculator {args.speculator} needs --draft-snapshot")
        block_mode = args.speculator == "block-draft"
        if args.fake_engine or not torch.cuda.is_available():
            from ..loader.load import load_params
            dcfg, dparams = load_params(args.draft_snapshot)
            make = lambda: ModelDrafter.from_oracle(dcfg, dparams, block=draft_len, parallel=block_mode)      # noqa: E731
        else:
            from ..loader.load import load_engine
            pages = (args.max_context_tokens // 64 + 2) * args.concurrency + 64
            dcfg, deng = load_engine(args.draft_snapshot, torch.device("cuda:0"), pages, 2048, 8)
            make = lambda: ModelDrafter.from_engine(deng, pages, args.max_context_tokens // 64 + 2, block=draft_len, parallel=block_mode)   # noqa: E731
        if dcfg.vocab_size != cfg.vocab_size:
            raise SystemExit(f"draft model vocabulary {dcfg.vocab_size} differs from the target's {cfg.vocab_size}")
        drafter = make()
    if args.speculator in ("auto", "mtp") and getattr(be, "has_mtp", False):
        from ..runtime.speculation import MtpDrafter
        drafter = MtpDrafter()              # native MTP depth of the checkpoint
    from ..runtime.repeat_guard import LoopAbortConfig
    loop = LoopAbortConfig(getattr(args, "loop_abort_run", 512), getattr(args, "loop_abort_copies", 8),
                           getattr(args, "loop_fast_span", 1024), getattr(args, "loop_fast_copies", 8))
    sched = Scheduler(be, max_active=args.concurrency, queue_depth=args.queue_depth, queue_wait_s=args.queue_wait,
                      loop_abort=loop if loop.enabled else None,
                      drafter=drafter, eos_ids=tuple(getattr(tok, "eos_ids", ())),
                      reserve_chunk_tokens=int(getattr(args, "kv_decode_reserve_chunk", 0) or 0),
                      early_end_tokens=int(getattr(args, "kv_early_termination_min_output_tokens", -1)))
    from ..utils.fault import FaultHooks
    hooks = FaultHooks()                      # refuses a configured fault without CUTEAFD_DEV_FAULT_HOOKS=1
    if hooks.plan:
        sched.faults = hooks
        for link in getattr(getattr(sched.be, "remote_experts", None), "links", []):
            link.faults = hooks
        hooks.arm()                           # the engine is built and prewarmed: visits count from here
        print(f"[serve] development fault hooks armed: {hooks.plan}", flush=True)
    prof = getattr(args, "profile", "") or os.environ.get("PROFILE", "")
    if prof:
        from ..utils.profile import Profile, parse_modes
        Profile(parse_modes(prof), getattr(args, "profile_dir", "") or ".", 64).attach(sched)
    trace_path = getattr(args, "speculation_trace", "") or os.environ.get("SPECULATION_TRACE", "")
    if trace_path:
        from ..utils.trace import JsonlTrace
        sched.trace = JsonlTrace(trace_path)
    stall_s = float(getattr(args, "stall_dump_seconds", 0) or 0)
    if stall_s > 0:
        from ..utils.diagnostics import StallWatchdog
        sched.watchdog = StallWatchdog(stall_s, getattr(args, "stack_dump_file", "") or None).start()
    usage = UsageLog(args.usage_db) if args.usage_db else None
    media = None
    if getattr(args, "media_encoder", ""):
        # the towers live in an encoder service (another process or host); this process keeps preprocessing and caching
        from ..media import MediaProcessor
        from ..media.remote import connect
        host, _, port = args.media_encoder.rpartition(":")
        vision, audio = connect(host or "127.0.0.1", int(port))
        if vision is not None or audio is not None:
            media = MediaProcessor(cfg.vocab_size, cfg.hidden, vision, audio)
    elif getattr(args, "media", "none") != "none":
        from ..media import AudioTower, AudioTowerConfig, MediaProcessor, VisionTower, VisionTowerConfig
        from ..media.loader import load_towers
        mdev = "cuda:0" if (torch.cuda.is_available() and not args.fake_engine) else "cpu"
        vision, audio = load_towers(snapshot, cfg.hidden, mdev) if snapshot else (None, None)
        if args.media == "random":           # geometry checks and benchmarks without a multimodal checkpoint
            small = dict(width=256, depth=2, heads=4, mlp=512, out_hidden=cfg.hidden)
            vision = vision or VisionTower(VisionTowerConfig(**small), VisionTower.random_weights(VisionTowerConfig(**small)), mdev)
            audio = audio or AudioTower(AudioTowerConfig(**small), AudioTower.random_weights(AudioTowerConfig(**small)), mdev)
        if vision is not None or audio is not None:
            media = MediaProcessor(cfg.vocab_size, cfg.hidden, vision, audio)
    return ServerState(sched, tok, getattr(args, "served_model_id", "") or cfg.name, args.api_key, usage, media=media,
                       extras={"max_output_tokens": int(getattr(args, "max_output_tokens", 0) or 0)})


_AFD_HANDLE = None


def _build_afd_rank(args, snapshot, world: int, num_pages: int, pages_per_seq: int, rows: int):
    """Join the deployment's process group and build this rank's half.  Expert ranks never return from here: they
    serve until the attention rank shuts the group down, then leave the process."""
    global _AFD_HANDLE
    import torch
    import torch.distributed as dist

    from ..config import PRESETS
    from ..parallel.afd import build_afd
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)
    dep = {}
    if getattr(args, "deployment", ""):
        with open(args.deployment) as f:
            dep = json.load(f)
        if dep.get("world_size", world) != world:
            raise SystemExit(f"deployment names {dep['world_size']} ranks, the process group has {world}")
    n_att = int(dep.get("attention_ranks", 1)) * int(dep.get("pipeline_stages", 1))
    if n_att != 1:
        # data-parallel attention replicas run in lockstep under one driver (the benchmark's SPMD generator); the HTTP
        # scheduler drives a single attention rank
        raise SystemExit("serve drives one attention rank per deployment; plan with --attention-ranks 1")
    if dep.get("kv_pool_tokens"):
        num_pages = max(num_pages, min(int(dep["kv_pool_tokens"]) // 64, num_pages * 4))
    if snapshot:
        # the attention rank reads everything but the routed experts; every expert rank reads its own expert range in
        # the stored format (E4M3 block-scaled, MXFP4, NVFP4 stay as stored)
        from ..loader.load import open_snapshot
        cfg = open_snapshot(snapshot).cfg
        kw = dict(snapshot=snapshot)
    else:
        cfg = PRESETS[args.preset or "qwen3-30b-a3b"]()
        if args.layers:
            cfg = cfg.replace(num_layers=args.layers)
        kw = {}
    h = build_afd(cfg, dev, rank, world, max_tokens=max(2048, rows), max_seqs=rows, num_pages=num_pages,
                  pages_per_seq=pages_per_seq, prefill_chunk=2048, n_attention=n_att, **kw)
    torch.cuda.synchronize()
    dist.barrier()
    if h.worker is not None:
        h.worker.serve()
        dist.barrier()
        dist.destroy_process_group()
        raise SystemExit(0)
    _AFD_HANDLE = h
    print(f"[serve] {h.parallelism}", flush=True)
    return cfg, h.generator.engine


_TP_ENGINE = None


def _build_tp_rank(args, snapshot, world: int, num_pages: int, rows: int):
    """Join the group and build this rank's shard of a tensor-parallel engine.  Rank 0 returns the mirrored engine for
    the backend; the other ranks follow it from here and leave the process when it stops them."""
    global _TP_ENGINE
    import torch
    import torch.distributed as dist

    from ..config import PRESETS
    from ..parallel.mirror import MirroredEngine, follow
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)
    if snapshot:
        from ..loader.load import load_params
        cfg, params = load_params(snapshot)
    else:
        cfg = PRESETS[args.preset or "qwen3-30b-a3b"]()
        if args.layers:
            cfg = cfg.replace(num_layers=args.layers)
        params = None
    cfg = cfg.replace(mtp_layers=0)                       # the MTP depth's own step is not mirrored
    if cfg.is_mla:
        from ..models.mla_moe import MlaMoeWeights as Weights
        from ..models.tp_mla import TpMlaMoeEngine as Engine
    else:
        from ..models.gqa_moe import GqaMoeWeights as Weights
        from ..models.tp_gqa import TpGqaMoeEngine as Engine
    W = Weights.from_params(cfg, params, dev) if params is not None else Weights.random_init(cfg, dev)   # same seed on every rank
    inner = Engine(cfg, W, num_pages, max_tokens=max(2048, rows), max_seqs=rows)
    torch.cuda.synchronize()
    dist.barrier()
    if rank != 0:
        steps = follow(inner)
        print(f"[serve] tensor-parallel rank {rank} followed {steps} steps", flush=True)
        dist.barrier()
        dist.destroy_process_group()
        raise SystemExit(0)
    _TP_ENGINE = MirroredEngine(inner)
    print(f"[serve] tensor-parallel attention over {world} GPUs, rank 0 drives", flush=True)
    return cfg, _TP_ENGINE


def run_server(args) -> int:
    state = build_state(args)
    from ..utils.diagnostics import install_stack_dump
    install_stack_dump(getattr(args, "stack_dump_file", "") or None)      # kill -USR1 <pid>: every thread's stack
    srv = Server(state, args.host, args.port).start()
    print(f"serving {state.model_id} on http://{args.host}:{srv.port}", flush=True)
    try:
        while True:
            time.sleep(3600)
    except KeyboardInterrupt:
        srv.stop()
        if _AFD_HANDLE is not None:                       # release the expert ranks, then leave the group together
            import torch.distributed as dist
            _AFD_HANDLE.shutdown()
            dist.barrier()
            dist.destroy_process_group()
        if _TP_ENGINE is not None:                        # release the following ranks the same way
            import torch.distributed as dist
            _TP_ENGINE.stop()
            dist.barrier()
            dist.destroy_process_group()
        if state.sched.trace is not None:
            state.sched.trace.close()
        be = state.sched.be
        if getattr(args, "prewarm", "") not in ("", "auto") and hasattr(be, "save_prewarm"):
            be.save_prewarm(args.prewarm)        # the next start captures this run's frequent geometries up front
    return 0
