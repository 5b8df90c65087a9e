"""Wire formats: OpenAI Chat Completions, Anthropic Messages and OpenAI Responses bodies to and
from the scheduler's ``Request`` / event stream.

Defaults match the reference: temperature 0 (greedy), top_p 1, min_p 0, no top_k, optional seed
(rust/crates/cuteafd-api/src/openai.rs:641-660).  Failure classes map to HTTP the same way: bad
request 400, unavailable 503, retry 429 with ``Retry-After: 1``, worker 500
(rust/crates/cuteafd-api/src/openai.rs:281-286; docs/client-apis.md:40-50).  ``usage.speculation``
carries {request_id, proposed, accepted, cycles} (docs/client-apis.md:31-38).  The probe header
``x-cuteafd-probe`` carries a JSON ProbeSpec: prompt_ids (synthetic token-id prompts),
no_speculation, record_rows, cold (skip the prefix cache), top_k (top ids and log-probabilities of every selected row),
score_from / want / score_positions / verify_rows (teacher-forced scoring of the prompt: one record per predicted
position, no generation) and record_state (hashes of the sequence's persistent state at the prompt and turn frontiers)
(rust/crates/cuteafd-api/src/openai/probe.rs:19-110).
"""
from __future__ import annotations

import json
import time
import uuid

from ..runtime import sampling
from ..runtime.scheduler import FAIL_BAD_REQUEST, FAIL_RETRY, FAIL_UNAVAILABLE, FAIL_WORKER, Request
from . import constraints
from .tokenizer import parse_tool_calls, render_chat

HTTP_OF = {FAIL_BAD_REQUEST: 400, FAIL_UNAVAILABLE: 503, FAIL_RETRY: 429, FAIL_WORKER: 500, "timeout": 504}
PROBE_HEADER = "x-cuteafd-probe"


class BadRequest(ValueError):
    pass


def _params(body: dict) -> sampling.SamplingParams:
    try:
        return sampling.SamplingParams(temperature=float(body.get("temperature", 0.0) or 0.0), top_p=float(body.get("top_p", 1.0) or 1.0),
                                       top_k=(int(body["top_k"]) if body.get("top_k") not in (None, 0, -1) else None),
                                       min_p=float(body.get("min_p", 0.0) or 0.0), seed=int(body.get("seed", 0) or 0))
    except (sampling.SamplingError, TypeError, ValueError) as e:
        raise BadRequest(str(e)) from e


def _stops(body: dict, tok) -> tuple[int, ...]:
    stop = body.get("stop") or body.get("stop_sequences") or []
    if isinstance(stop, str):
        stop = [stop]
    ids = []
    for s in stop:
        e = tok.encode(s)
        if len(e) == 1:
            ids.append(e[0])
    return tuple(ids) + tuple(getattr(tok, "eos_ids", ()))


def _stop_texts(body: dict, tok) -> tuple[str, ...]:
    """Every stop string, for the match on the decoded text: it ends the reply before the string whatever its
    tokenisation (a one-token stop also ends generation at the token level, which only saves the extra step)."""
    stop = body.get("stop") or body.get("stop_sequences") or []
    if isinstance(stop, str):
        stop = [stop]
    if not isinstance(stop, list) or len(stop) > 16 or not all(isinstance(s, str) for s in stop):
        raise BadRequest("stop must be a string or a list of at most 16 strings")
    return tuple(s for s in stop if s)


COMPACT_REQUEST = ("Summarize this conversation so that it can be continued from the summary alone. Keep the user's "
                   "requirements, the decisions taken, tool results and the work still pending. Answer with the summary only.")
COMPACT_PREFIX = "Summary of the conversation so far:\n"


def encode_opaque(kind: str, text: str) -> str:
    """Opaque item content a client stores and sends back (``encrypted_content``): tagged, base64; not secret."""
    import base64
    return "cafd1." + base64.urlsafe_b64encode(json.dumps({"kind": kind, "text": text}).encode()).decode()


def decode_opaque(blob: str, kind: str) -> str:
    import base64
    import binascii
    try:
        if not blob.startswith("cafd1."):
            raise ValueError
        d = json.loads(base64.urlsafe_b64decode(blob[6:].encode()))
        if d.get("kind") != kind:
            raise ValueError
        return str(d["text"])
    except (ValueError, KeyError, binascii.Error, UnicodeDecodeError) as e:
        raise BadRequest(f"unreadable {kind} item") from e


def compaction_object(summary: str, usage: dict) -> dict:
    return {"id": "resp_" + uuid.uuid4().hex[:24], "object": "response.compaction", "created_at": int(time.time()),
            "output": [{"id": "cmp_" + uuid.uuid4().hex[:20], "type": "compaction",
                        "encrypted_content": encode_opaque("compaction", summary)}],
            "usage": {"input_tokens": usage.get("prompt_tokens", 0), "output_tokens": usage.get("completion_tokens", 0),
                      "total_tokens": usage.get("prompt_tokens", 0) + usage.get("completion_tokens", 0)}}


def responses_items_to_messages(items: list) -> list[dict]:
    """Responses ``input`` items -> chat messages: ``function_call`` items are the assistant's calls (consecutive ones
    share a turn), ``function_call_output`` items turns of role ``tool``; reasoning items are dropped."""
    msgs: list[dict] = []
    for it in items:
        if not isinstance(it, dict):
            continue
        t = it.get("type", "message")
        if t == "function_call":
            call = _call(it.get("call_id") or it.get("id", ""), it.get("name", ""), it.get("arguments"))
            if msgs and msgs[-1].get("role") == "assistant" and msgs[-1].get("_calls_only"):
                msgs[-1]["tool_calls"].append(call)
            else:
                msgs.append({"role": "assistant", "content": "", "tool_calls": [call], "_calls_only": True})
        elif t == "compaction":                       # what /v1/responses/compact returned earlier: the summary it stands for
            msgs.append({"role": "user", "content": COMPACT_PREFIX + decode_opaque(str(it.get("encrypted_content", "")), "compaction")})
        elif t == "function_call_output":
            out = it.get("output")
            msgs.append({"role": "tool", "tool_call_id": it.get("call_id", ""), "content": out if isinstance(out, str) else json.dumps(out)})
        elif t == "message" or "role" in it:
            one = {"role": it.get("role", "user"), "content": it.get("content")}
            one.update({k: it[k] for k in ("tool_calls", "tool_call_id") if k in it})      # a stored conversation's own form
            msgs.append(one)
    for m in msgs:
        m.pop("_calls_only", None)
    return msgs


def normalize_tools(tools, flavor: str) -> list[dict] | None:
    """Tool declarations of any flavour -> OpenAI function tools (what the chat template shows the model).  Hosted tool
    types (web search and the like) are the gateway's business and are left out here."""
    out = []
    for t in tools or []:
        if not isinstance(t, dict):
            continue
        if isinstance(t.get("function"), dict):                                  # OpenAI chat
            out.append({"type": "function", "function": t["function"]})
        elif flavor == "anthropic" and "name" in t and "input_schema" in t:
            out.append({"type": "function", "function": {"name": t["name"], "description": t.get("description", ""),
                                                         "parameters": t["input_schema"]}})
        elif t.get("type") == "function" and "name" in t:                        # Responses: flat
            out.append({"type": "function", "function": {"name": t["name"], "description": t.get("description", ""),
                                                         "parameters": t.get("parameters") or {"type": "object", "properties": {}}}})
    return out or None


def _call(call_id: str, name: str, arguments) -> dict:
    return {"id": call_id, "type": "function",
            "function": {"name": name, "arguments": arguments if isinstance(arguments, str) else json.dumps(arguments or {})}}


def anthropic_messages(body: dict) -> list[dict]:
    """Anthropic Messages history -> chat messages: ``tool_use`` blocks become the assistant's tool calls and
    ``tool_result`` blocks turns of role ``tool``; other parts pass through for the template."""
    msgs = []
    if body.get("system"):
        sysm = body["system"]
        msgs.append({"role": "system", "content": sysm if isinstance(sysm, str) else "".join(p.get("text", "") for p in sysm)})
    for m in body.get("messages") or []:
        c = m.get("content")
        if not isinstance(c, list):
            msgs.append({"role": m.get("role", "user"), "content": c})
            continue
        keep, calls, results = [], [], []
        for p in c:
            if not isinstance(p, dict):
                continue
            if p.get("type") == "tool_use":
                calls.append(_call(p.get("id", ""), p.get("name", ""), p.get("input")))
            elif p.get("type") == "tool_result":
                rc = p.get("content")
                if isinstance(rc, list):
                    rc = "".join(x.get("text", "") for x in rc if isinstance(x, dict))
                results.append({"role": "tool", "tool_call_id": p.get("tool_use_id", ""), "content": rc if rc is not None else ""})
            else:
                keep.append(p)
        msgs.extend(results)                                                      # results answer the previous turn: they come first
        if keep or calls:
            one = {"role": m.get("role", "user"), "content": keep}
            if calls:
                one["tool_calls"] = calls
            msgs.append(one)
    return msgs


def build_request(body: dict, tok, vocab_size: int, probe: dict | None = None, flavor: str = "openai",
                  media=None, max_output_tokens: int = 0) -> Request:
    """``max_output_tokens`` > 0 (the deployment's MAX_OUTPUT_TOKENS): the most a request may ask for, and what a request
    that names no limit gets; 0 leaves the limit to the context and gives such a request 256 tokens."""
    # a probe too large for a header (a long synthetic prompt) may ride in the body instead
    probe = {**(body.get("cuteafd_probe") or {}), **(probe or {})}
    tools = normalize_tools(body.get("tools"), flavor)
    try:
        choice = constraints.tool_choice_of(body, flavor)
        tool_fmt = constraints.tool_call_format(tools, *choice)
    except ValueError as e:
        raise BadRequest(str(e)) from e
    if choice[0] == "none":
        tools = None                                       # the model is not shown tools it may not call
    if probe.get("prompt_ids"):
        prompt, spans = [int(t) for t in probe["prompt_ids"]], None
    else:
        if flavor == "anthropic":
            msgs = anthropic_messages(body)
        elif flavor == "responses":
            inp = body.get("input")
            msgs = [{"role": "user", "content": inp}] if isinstance(inp, str) else responses_items_to_messages(inp or [])
            if body.get("instructions"):
                msgs.insert(0, {"role": "system", "content": body["instructions"]})
        else:
            msgs = list(body.get("messages") or [])
        if not msgs:
            raise BadRequest("messages must not be empty")
        items: list = []
        text = render_chat(msgs, True, tools, media=items)
        if items:
            # image / audio parts: tower rows replace placeholder ids (``media`` is the deployment's MediaProcessor)
            from ..media.image import MediaError, bytes_from_url
            from .tokenizer import split_media
            if media is None:
                raise BadRequest("this deployment serves text only (no media tower is loaded)")
            try:
                segs = [s if isinstance(s, str) else (s[0], bytes_from_url(s[1])) for s in split_media(text, items)]
                prompt, spans = media.expand(segs, tok.encode)
            except MediaError as e:
                raise BadRequest(str(e)) from e
        else:
            prompt, spans = tok.encode(text), None
    max_tokens = body.get("max_tokens") or body.get("max_completion_tokens") or body.get("max_output_tokens") or (max_output_tokens or 256)
    if not isinstance(max_tokens, int) or isinstance(max_tokens, bool) or max_tokens < 1:
        raise BadRequest("max_tokens must be a positive integer")
    if max_output_tokens > 0:
        max_tokens = min(max_tokens, max_output_tokens)
    fmt = body.get("response_format")
    if fmt is None:                                        # the guided_* spellings some clients send at the top level
        if "guided_regex" in body:
            fmt = {"type": "regex", "pattern": body["guided_regex"]}
        elif "guided_choice" in body:
            fmt = {"type": "choice", "choices": body["guided_choice"]}
        elif "guided_json" in body:
            fmt = {"type": "json_schema", "schema": body["guided_json"]}
    if tool_fmt is not None and (fmt is None or tool_fmt["at_least_one"]):
        fmt = tool_fmt                                     # a forced call is the whole reply; strict tools under auto
    try:                                                   # yield to an explicit response_format
        cons = constraints.from_response_format(fmt, tok, vocab_size)
    except ValueError as e:
        raise BadRequest(str(e)) from e
    n_top = body.get("top_logprobs") or 0
    if not isinstance(n_top, int) or not 0 <= n_top <= 20:
        raise BadRequest("top_logprobs must be an integer between 0 and 20")
    keep = max(n_top, 1) if (body.get("logprobs") or n_top) else 0
    keep = max(keep, int(probe.get("top_k", 0) or 0))
    stop_texts = _stop_texts(body, tok)                    # validates the type of ``stop`` before anything encodes it
    score_from = probe.get("score_from")
    if score_from is not None:
        if isinstance(score_from, bool) or not isinstance(score_from, int) or not 0 <= score_from <= len(prompt):
            raise BadRequest("probe score_from must be an index into the prompt")
        if spans:
            raise BadRequest("probe score_from scores token prompts only")
    want = probe.get("want") or {}
    if not isinstance(want, dict):
        raise BadRequest("probe want must map positions to token ids")
    verify_rows = int(probe.get("verify_rows") or 0)
    if verify_rows < 0:
        raise BadRequest("probe verify_rows must be positive")
    pos = probe.get("score_positions")
    return Request(prompt=prompt, max_tokens=max_tokens, params=_params(body), stop_ids=_stops(body, tok),
                   speculation=not probe.get("no_speculation", False), record_rows=bool(probe.get("record_rows", False)),
                   constraint=cons, media=spans, top_logprobs=keep, cold=bool(probe.get("cold", False)),
                   stop_texts=stop_texts, score_from=score_from, score_want={int(k): [int(t) for t in v] for k, v in want.items()},
                   score_positions=None if pos is None else tuple(int(x) for x in pos), verify_rows=verify_rows,
                   record_state=bool(probe.get("record_state", False)))


def logprobs_block(tok, top_rows: list, n_top: int) -> dict:
    """OpenAI ``choices[].logprobs``: one entry per generated token with its log-probability and ``n_top`` alternatives."""
    def piece(t: int) -> dict:
        raw = tok.token_bytes(t) if t < tok.vocab_size else b""
        return {"token": raw.decode("utf-8", "replace"), "bytes": list(raw)}
    content = []
    for t, lp, ids, vals in top_rows:
        content.append(dict(piece(t), logprob=lp, top_logprobs=[dict(piece(i), logprob=v) for i, v in zip(ids[:n_top], vals[:n_top])]))
    return {"content": content}


def parse_probe(headers) -> dict:
    raw = headers.get(PROBE_HEADER)
    if not raw:
        return {}
    try:
        d = json.loads(raw)
    except json.JSONDecodeError as e:
        raise BadRequest(f"{PROBE_HEADER}: {e}") from e
    if not isinstance(d, dict):
        raise BadRequest(f"{PROBE_HEADER} must be a JSON object")
    return d


def usage_block(u: dict) -> dict:
    out = {"prompt_tokens": u.get("prompt_tokens", 0), "completion_tokens": u.get("completion_tokens", 0),
           "total_tokens": u.get("prompt_tokens", 0) + u.get("completion_tokens", 0),
           "prompt_tokens_details": {"cached_tokens": u.get("cached_tokens", 0)}}
    if "speculation" in u:
        out["speculation"] = u["speculation"]
    if u.get("finish_detail"):
        out["finish_detail"] = u["finish_detail"]            # "repetition": the loop detector ended the reply
    return out


# ---- OpenAI chat completions ---------------------------------------------------------------------------
def chat_completion(model: str, text: str, finish: str, usage: dict, probe_rows: list[str] | None = None,
                    logprobs: dict | None = None) -> dict:
    content, calls = parse_tool_calls(text)
    msg = {"role": "assistant", "content": content}
    if calls:
        msg["tool_calls"] = calls
        finish = "tool_calls"
    out = {"id": "chatcmpl-" + uuid.uuid4().hex[:24], "object": "chat.completion", "created": int(time.time()), "model": model,
           "choices": [{"index": 0, "message": msg, "finish_reason": finish}], "usage": usage_block(usage)}
    if probe_rows:
        out["probe"] = {"row_hashes": probe_rows}
    if logprobs is not None:
        out["choices"][0]["logprobs"] = logprobs
    return out


def chat_chunk(cid: str, model: str, delta: dict, finish: str | None = None, usage: dict | None = None) -> dict:
    out = {"id": cid, "object": "chat.completion.chunk", "created": int(time.time()), "model": model,
           "choices": [{"index": 0, "delta": delta, "finish_reason": finish}]}
    if usage is not None:
        out["usage"] = usage_block(usage)
    return out


# ---- Anthropic messages -----------------------------------------------------------------------------------
def anthropic_message(model: str, text: str, finish: str, usage: dict) -> dict:
    content, calls = parse_tool_calls(text)
    blocks = [{"type": "text", "text": content}] if content or not calls else []
    for c in calls:
        blocks.append({"type": "tool_use", "id": "toolu_" + uuid.uuid4().hex[:20], "name": c["function"]["name"],
                       "input": json.loads(c["function"]["arguments"] or "{}")})
    stop = {"stop": "end_turn", "length": "max_tokens"}.get(finish, finish)
    if calls:
        stop = "tool_use"
    return {"id": "msg_" + uuid.uuid4().hex[:24], "type": "message", "role": "assistant", "model": model, "content": blocks,
            "stop_reason": stop, "stop_sequence": None,
            "usage": {"input_tokens": usage.get("prompt_tokens", 0), "output_tokens": usage.get("completion_tokens", 0),
                      "cache_read_input_tokens": usage.get("cached_tokens", 0)}}


def anthropic_events(model: str, usage_in: int):
    mid = "msg_" + uuid.uuid4().hex[:24]
    start = {"type": "message_start", "message": {"id": mid, "type": "message", "role": "assistant", "model": model, "content": [],
                                                  "stop_reason": None, "usage": {"input_tokens": usage_in, "output_tokens": 0}}}
    return mid, [("message_start", start), ("content_block_start", {"type": "content_block_start", "index": 0,
                                                                     "content_block": {"type": "text", "text": ""}})]


# ---- OpenAI responses -------------------------------------------------------------------------------------
def responses_messages(body: dict) -> list[dict]:
    """The Responses request as a chat message list (instructions first)."""
    inp = body.get("input")
    msgs = [{"role": "user", "content": inp}] if isinstance(inp, str) else responses_items_to_messages(inp or [])
    if body.get("instructions"):
        msgs.insert(0, {"role": "system", "content": body["instructions"]})
    return msgs


def continue_session(body: dict, sessions: dict) -> tuple[dict, list[dict]]:
    """Resolve ``previous_response_id``: (request body whose input is the whole conversation, that conversation)."""
    msgs = responses_messages(body)
    prev = body.get("previous_response_id")
    if prev:
        hist = sessions.get(prev)
        if hist is None:
            raise BadRequest(f"previous_response_id {prev!r} is unknown (responses are kept in memory until deleted)")
        msgs = list(hist) + [m for m in msgs if m.get("role") != "system" or not any(h.get("role") == "system" for h in hist)]
    out = {k: v for k, v in body.items() if k not in ("previous_response_id", "instructions")}
    out["input"] = msgs
    return out, msgs


def input_items(msgs: list[dict]) -> dict:
    data = []
    for i, m in enumerate(msgs):
        c = m.get("content")
        text = c if isinstance(c, str) else "".join(p.get("text", "") for p in (c or []) if isinstance(p, dict))
        kind = "output_text" if m.get("role") == "assistant" else "input_text"
        data.append({"id": f"item_{i}", "type": "message", "role": m.get("role", "user"), "content": [{"type": kind, "text": text}]})
    return {"object": "list", "data": data, "has_more": False}



def responses_object(model: str, text: str, finish: str, usage: dict, rid: str | None = None) -> dict:
    rid = rid or "resp_" + uuid.uuid4().hex[:24]
    text, calls = parse_tool_calls(text)
    output = []
    if text or not calls:
        output.append({"type": "message", "id": "msg_" + uuid.uuid4().hex[:20], "role": "assistant", "status": "completed",
                       "content": [{"type": "output_text", "text": text, "annotations": []}]})
    for c in calls:                                                               # the model's tool calls as function_call items
        output.append({"type": "function_call", "id": "fc_" + uuid.uuid4().hex[:20], "call_id": "call_" + uuid.uuid4().hex[:20],
                       "name": c["function"]["name"], "arguments": c["function"]["arguments"], "status": "completed"})
    return {"id": rid, "object": "response", "created_at": int(time.time()), "model": model,
            "status": "completed" if finish in ("stop", "length") else "incomplete",
            "output": output,
            "output_text": text,
            "usage": {"input_tokens": usage.get("prompt_tokens", 0), "output_tokens": usage.get("completion_tokens", 0),
                      "total_tokens": usage.get("prompt_tokens", 0) + usage.get("completion_tokens", 0)}}


def error_body(kind: str, message: str, flavor: str = "openai") -> tuple[int, dict, dict]:
    status = HTTP_OF.get(kind, 500)
    headers = {"Retry-After": "1"} if kind == FAIL_RETRY else {}
    if flavor == "anthropic":
        t = {400: "invalid_request_error", 429: "rate_limit_error", 503: "overloaded_error"}.get(status, "api_error")
        return status, {"type": "error", "error": {"type": t, "message": message}}, headers
    t = {400: "invalid_request_error", 429: "rate_limit_exceeded", 503: "service_unavailable"}.get(status, "server_error")
    return status, {"error": {"message": message, "type": t, "code": kind}}, headers
