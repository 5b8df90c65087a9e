"""Benchmark and quality panels run against a live server over its HTTP API, so they exercise exactly what a client
gets (tokenizer, templates, scheduler, prefix cache, speculation, engine) whatever backend serves.

    python -m cuteafd_b200.cli bench --url http://127.0.0.1:8000 --panels smoke,cache_exact,lossless,speed
    python -m cuteafd_b200.cli bench --url ... --panels sweep --levels 1,4,8,16 --max-tokens 128
    python -m cuteafd_b200.cli bench --url ... --panels sustained --seconds 60 --concurrency 8

Panels
  smoke        /health, /v1/models, one short completion, one streamed completion
  cache_exact  the same prompt twice: the second is served from the prefix cache and must reproduce every selected
               logit row bit for bit (row hashes through the probe header) and the same text
  lossless     greedy decoding with and without speculative drafts gives the same tokens
  template     chat rendering is stable: the prompt token count of the same conversation does not change between
               calls, and grows when a turn is appended (``/v1/responses/input_tokens``)
  tools        a tool declaration reaches the template and a constrained reply (``response_format`` choice) comes back
               as one of the choices
  speed        C1 decode tok/s and TTFT on a short prompt, and prefill tok/s + TTFT on a long one (streamed, timed at
               the client)
  sweep        aggregate decode tok/s at each concurrency of ``levels`` with a distinct prompt per stream
  sustained    ``concurrency`` streams kept busy for ``seconds``: requests, tokens/s, TTFT p50 / p99, failures
  agentic      ``sessions`` conversations over one shared system prefix, ``turns`` turns each with the reply fed back:
               share of prompt tokens served from the prefix cache, emitted tok/s, failures
  context_load cold prompts of growing length (``lengths``, cut at the served context window): TTFT and prefill tok/s
               at each, every one answered
  fidelity     teacher-forced scoring of sealed reference windows (``windows`` = file written by ``fidelity seal``)
               through the probe: KL and top-1 agreement of the served model against the sealed distributions, held
               against ``kl_bar`` / ``top1_bar``

Every panel returns ``{"panel", "ok", ...numbers}``; the runner attaches the server's thermal window for the time the
panel ran (``/v1/thermal``) the way every phase of the reference's card carries its throttle summary.

Counterpart: rust/crates/cuteafd-bench/src/baseline.rs:1-25 (card), the quick-quality checks (cache_exact, lossless
speculation, template round-trip) and the panels / sustained / sweep / smoke modes of the reference's bench crate.
"""
from __future__ import annotations

import http.client
import json
import random
import statistics
import threading
import time
import urllib.parse

PROBE = "x-cuteafd-probe"
WORDS = ("tensor memory barrier tile warp cluster stream graph expert router token cache page latent index prefix "
         "draft verify commit lane queue batch kernel copy fence flag epoch slot").split()


class Client:
    def __init__(self, url: str, api_key: str = "", timeout: float = 600.0):
        u = urllib.parse.urlparse(url)
        self.host, self.port, self.key, self.timeout = u.hostname, u.port or 80, api_key, timeout

    def _conn(self) -> http.client.HTTPConnection:
        return http.client.HTTPConnection(self.host, self.port, timeout=self.timeout)

    def _headers(self, extra: dict | None = None) -> dict:
        h = {"Content-Type": "application/json"}
        if self.key:
            h["Authorization"] = "Bearer " + self.key
        h.update(extra or {})
        return h

    def get(self, path: str):
        c = self._conn()
        c.request("GET", path, headers=self._headers())
        r = c.getresponse()
        raw = r.read()
        c.close()
        try:
            return r.status, json.loads(raw)
        except json.JSONDecodeError:
            return r.status, raw

    def post(self, path: str, body: dict, headers: dict | None = None):
        c = self._conn()
        c.request("POST", path, json.dumps(body), self._headers(headers))
        r = c.getresponse()
        raw = r.read()
        c.close()
        return r.status, json.loads(raw or b"{}")

    def stream(self, body: dict) -> dict:
        """Streamed chat completion timed at the client: {"status", "text", "ttft_s", "seconds", "usage", "chunks"}."""
        c = self._conn()
        t0 = time.perf_counter()
        c.request("POST", "/v1/chat/completions", json.dumps(dict(body, stream=True)), self._headers())
        r = c.getresponse()
        if r.status != 200:
            raw = r.read()
            c.close()
            return {"status": r.status, "text": "", "ttft_s": None, "seconds": time.perf_counter() - t0, "usage": {}, "chunks": 0,
                    "error": raw[:200].decode("utf-8", "replace")}
        text, first, usage, chunks = [], None, {}, 0
        for line in r:
            if not line.startswith(b"data: "):
                continue
            data = line[6:].strip()
            if data == b"[DONE]":
                break
            ev = json.loads(data)
            if "error" in ev:
                c.close()
                return {"status": 500, "text": "".join(text), "ttft_s": first, "seconds": time.perf_counter() - t0, "usage": {},
                        "chunks": chunks, "error": str(ev["error"])[:200]}
            delta = ev["choices"][0]["delta"].get("content")
            if delta:
                first = first if first is not None else time.perf_counter() - t0
                text.append(delta)
                chunks += 1
            usage = ev.get("usage") or usage
        c.close()
        return {"status": 200, "text": "".join(text), "ttft_s": first, "seconds": time.perf_counter() - t0, "usage": usage, "chunks": chunks}


def prompt_of(n_words: int, seed: int) -> str:
    rnd = random.Random(seed)
    return " ".join(rnd.choice(WORDS) for _ in range(n_words))


def _chat(text: str, max_tokens: int, **kw) -> dict:
    return dict({"messages": [{"role": "user", "content": text}], "max_tokens": max_tokens, "temperature": 0}, **kw)


# ---- panels ------------------------------------------------------------------------------------------
def smoke(c: Client, o: dict) -> dict:
    st_h, health = c.get("/health")
    st_m, models = c.get("/v1/models")
    st_c, out = c.post("/v1/chat/completions", _chat("say hello", 8))
    s = c.stream(_chat("count to five", 8))
    ok = st_h == 200 and st_m == 200 and st_c == 200 and s["status"] == 200 and bool(models.get("data"))
    return {"ok": ok, "health": health.get("status") if isinstance(health, dict) else None,
            "model": models["data"][0]["id"] if ok else None, "completion_tokens": out.get("usage", {}).get("completion_tokens"),
            "streamed_chunks": s["chunks"]}


def cache_exact(c: Client, o: dict) -> dict:
    """Exact prefix-cache restore: the same request three times.  The second and third are served from the cache and must
    agree bit for bit (the hash of every selected logit row); all three must give the same text.  Whether the cold first
    run also has the warm runs' row bits is reported, not required: it computes the prompt as one large chunk where a
    warm run computes only the tail, and an engine whose GEMMs are not batch-invariant rounds those differently."""
    body = _chat(prompt_of(o.get("prompt_words", 160), 11), o.get("max_tokens", 16))
    probe = {PROBE: json.dumps({"record_rows": True, "no_speculation": True})}
    runs = [c.post("/v1/chat/completions", body, probe) for _ in range(3)]
    if any(st != 200 for st, _ in runs):
        return {"ok": False, "status": [st for st, _ in runs]}
    (_, a), (_, b), (_, d) = runs
    rows = [r.get("probe", {}).get("row_hashes") for r in (a, b, d)]
    cached = b["usage"]["prompt_tokens_details"]["cached_tokens"]
    warm_rows = rows[1] == rows[2] and bool(rows[1])
    same_text = len({r["choices"][0]["message"]["content"] for r in (a, b, d)}) == 1
    return {"ok": warm_rows and same_text and cached > 0, "cached_tokens": cached, "prompt_tokens": b["usage"]["prompt_tokens"],
            "rows_identical": warm_rows, "cold_rows_identical": rows[0] == rows[1], "text_identical": same_text}


def lossless(c: Client, o: dict) -> dict:
    unit = prompt_of(12, 5)
    body = _chat((unit + " ") * 10, o.get("max_tokens", 32))            # repetitive: drafts get proposed
    st1, plain = c.post("/v1/chat/completions", body, {PROBE: json.dumps({"no_speculation": True})})
    st2, spec = c.post("/v1/chat/completions", body)
    if st1 != 200 or st2 != 200:
        return {"ok": False, "status": [st1, st2]}
    sp = spec["usage"].get("speculation", {})
    same = plain["choices"][0]["message"]["content"] == spec["choices"][0]["message"]["content"]
    return {"ok": same, "text_identical": same, "proposed": sp.get("proposed"), "accepted": sp.get("accepted"), "cycles": sp.get("cycles"),
            "completion_tokens": spec["usage"]["completion_tokens"]}


def template(c: Client, o: dict) -> dict:
    conv = [{"role": "user", "content": "first question"}, {"role": "assistant", "content": "first answer"},
            {"role": "user", "content": "second question"}]
    n1 = c.post("/v1/responses/input_tokens", {"input": conv})[1].get("input_tokens")
    n2 = c.post("/v1/responses/input_tokens", {"input": conv})[1].get("input_tokens")
    n3 = c.post("/v1/responses/input_tokens", {"input": conv + [{"role": "assistant", "content": "x"}, {"role": "user", "content": "y"}]})[1].get("input_tokens")
    ok = isinstance(n1, int) and n1 == n2 and isinstance(n3, int) and n3 > n1
    return {"ok": ok, "tokens": n1, "tokens_after_append": n3}


def tools(c: Client, o: dict) -> dict:
    tool = {"type": "function", "function": {"name": "get_time", "description": "current time", "parameters": {"type": "object", "properties": {}}}}
    base = c.post("/v1/responses/input_tokens", {"input": "what time is it"})[1].get("input_tokens", 0)
    with_tool = c.post("/v1/responses/input_tokens", {"input": "what time is it", "tools": [tool]})[1].get("input_tokens", 0)
    st, out = c.post("/v1/chat/completions", _chat("pick one", 8, response_format={"type": "choice", "choices": ["get_time", "none"]}))
    text = out["choices"][0]["message"]["content"] if st == 200 else None
    return {"ok": st == 200 and text in ("get_time", "none") and with_tool >= base, "choice": text,
            "template_tokens_with_tool": with_tool, "template_tokens": base}


def speed(c: Client, o: dict) -> dict:
    n = o.get("max_tokens", 64)
    c.stream(_chat(prompt_of(16, 1), 8))                               # warm-up: graphs, caches
    short = c.stream(_chat(prompt_of(16, 2), n))
    long_words = o.get("prefill_words", 2048)
    long = c.stream(_chat(prompt_of(long_words, 3), 4))
    if short["status"] != 200 or long["status"] != 200:
        return {"ok": False, "errors": [short.get("error"), long.get("error")]}
    toks = short["usage"].get("completion_tokens", 0)
    decode_s = short["seconds"] - (short["ttft_s"] or 0.0)
    ptoks = long["usage"].get("prompt_tokens", 0)
    return {"ok": toks > 0 and ptoks > 0, "c1_decode_tok_s": round((toks - 1) / decode_s, 2) if decode_s > 0 and toks > 1 else None,
            "c1_ttft_s": short["ttft_s"], "prefill_tokens": ptoks, "prefill_ttft_s": long["ttft_s"],
            "prefill_tok_s": round(ptoks / long["ttft_s"], 1) if long["ttft_s"] else None}


def _fan(c: Client, bodies: list[dict]) -> tuple[list[dict], float]:
    out: list[dict | None] = [None] * len(bodies)

    def one(i: int) -> None:
        out[i] = c.stream(bodies[i])
    ts = [threading.Thread(target=one, args=(i,)) for i in range(len(bodies))]
    t0 = time.perf_counter()
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    return out, time.perf_counter() - t0


def sweep(c: Client, o: dict) -> dict:
    n = o.get("max_tokens", 64)
    levels = {}
    for k in o.get("levels", [1, 4, 8]):
        res, wall = _fan(c, [_chat(prompt_of(24, 100 * k + i), n) for i in range(k)])      # a distinct prompt per stream
        toks = sum(r["usage"].get("completion_tokens", 0) for r in res if r["status"] == 200)
        ttft = [r["ttft_s"] for r in res if r["ttft_s"] is not None]
        levels[str(k)] = {"tok_s": round(toks / wall, 2), "failed": sum(r["status"] != 200 for r in res),
                          "ttft_p50_s": round(statistics.median(ttft), 4) if ttft else None}
    return {"ok": all(v["failed"] == 0 and v["tok_s"] > 0 for v in levels.values()), "levels": levels}


def sustained(c: Client, o: dict) -> dict:
    seconds, conc, n = o.get("seconds", 10.0), o.get("concurrency", 4), o.get("max_tokens", 32)
    stop = time.perf_counter() + seconds
    lock = threading.Lock()
    rec = {"requests": 0, "tokens": 0, "failed": 0, "retry": 0, "ttft": []}

    def worker(w: int) -> None:
        i = 0
        while time.perf_counter() < stop:
            r = c.stream(_chat(prompt_of(24, 7919 * w + i), n))
            i += 1
            with lock:
                rec["requests"] += 1
                if r["status"] == 200:
                    rec["tokens"] += r["usage"].get("completion_tokens", 0)
                    if r["ttft_s"] is not None:
                        rec["ttft"].append(r["ttft_s"])
                elif r["status"] == 429:
                    rec["retry"] += 1                                   # capacity refusal: the client's cue to back off
                    time.sleep(0.05)
                else:
                    rec["failed"] += 1
    t0 = time.perf_counter()
    ts = [threading.Thread(target=worker, args=(w,)) for w in range(conc)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    wall = time.perf_counter() - t0
    tt = sorted(rec["ttft"])
    return {"ok": rec["failed"] == 0 and rec["tokens"] > 0, "requests": rec["requests"], "failed": rec["failed"], "retried_429": rec["retry"],
            "tok_s": round(rec["tokens"] / wall, 2), "ttft_p50_s": round(tt[len(tt) // 2], 4) if tt else None,
            "ttft_p99_s": round(tt[min(len(tt) - 1, int(len(tt) * 0.99))], 4) if tt else None, "seconds": round(wall, 2)}


def agentic(c: Client, o: dict) -> dict:
    """The shape of an agent workload: a long shared preamble, several sessions, every turn re-sends the conversation so
    far (rust/crates/cuteafd-bench/src/panels/agentic.rs in the reference).  After a session's first turn almost every
    prompt token should come from the prefix cache."""
    sessions, turns, n = int(o.get("sessions", 4)), int(o.get("turns", 4)), int(o.get("max_tokens", 16))
    system = "You are a careful assistant. " + prompt_of(int(o.get("prefix_words", 400)), 5)
    lock = threading.Lock()
    rec = {"prompt": 0, "cached": 0, "later_prompt": 0, "later_cached": 0, "emitted": 0, "failed": 0}

    def session(s: int) -> None:
        msgs = [{"role": "system", "content": system}]
        for t in range(turns):
            msgs.append({"role": "user", "content": f"step {t} of task {s}: " + prompt_of(24, 100 * s + t)})
            st, out = c.post("/v1/chat/completions", {"messages": msgs, "max_tokens": n, "temperature": 0})
            with lock:
                if st != 200:
                    rec["failed"] += 1
                    return
                u = out["usage"]
                cached = u.get("prompt_tokens_details", {}).get("cached_tokens", 0)
                rec["prompt"] += u["prompt_tokens"]
                rec["cached"] += cached
                rec["emitted"] += u["completion_tokens"]
                if t:
                    rec["later_prompt"] += u["prompt_tokens"]
                    rec["later_cached"] += cached
            msgs.append({"role": "assistant", "content": out["choices"][0]["message"]["content"] or "."})
    t0 = time.perf_counter()
    ts = [threading.Thread(target=session, args=(s,)) for s in range(sessions)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    wall = time.perf_counter() - t0
    share = rec["cached"] / max(rec["prompt"], 1)
    later = rec["later_cached"] / max(rec["later_prompt"], 1)
    return {"ok": rec["failed"] == 0 and rec["emitted"] > 0 and later >= float(o.get("cache_bar", 0.5)), "sessions": sessions, "turns": turns,
            "prompt_tokens": rec["prompt"], "cache_share": round(share, 4), "cache_share_after_first_turn": round(later, 4),
            "emitted_tokens": rec["emitted"], "tok_s": round(rec["emitted"] / wall, 2), "failed": rec["failed"], "seconds": round(wall, 2)}


def _ids_chat(ids: list[int], max_tokens: int, **probe) -> dict:
    """A request whose prompt is given as token ids (the probe rides in the body: long prompts do not fit a header)."""
    return {"messages": [{"role": "user", "content": "."}], "max_tokens": max_tokens, "temperature": 0,
            "cuteafd_probe": dict({"prompt_ids": ids, "no_speculation": True}, **probe)}


def context_load(c: Client, o: dict) -> dict:
    st, cat = c.get("/v1/codex/models.json")
    window = int(cat["models"][0].get("context_window", 0)) if st == 200 and isinstance(cat, dict) and cat.get("models") else 0
    vocab = int(o.get("vocab", 256))
    rnd = random.Random(11)
    rows, ok = {}, True
    for n in o.get("lengths", [1024, 4096, 16384, 65536]):
        if window and n > window - 16:
            continue
        # one generated token, not streamed: the reply arrives when the first token exists, whatever text it decodes to
        t0 = time.perf_counter()
        st_r, out = c.post("/v1/chat/completions", _ids_chat([rnd.randrange(1, vocab) for _ in range(n)], 1, cold=True))
        dt = time.perf_counter() - t0
        good = st_r == 200 and out.get("usage", {}).get("prompt_tokens") == n
        ok = ok and good
        rows[str(n)] = {"ok": good, "ttft_s": round(dt, 4), "prefill_tok_s": round(n / dt, 1) if good and dt > 0 else None,
                        "error": None if good else str(out.get("error", st_r))[:200]}
    return {"ok": ok and bool(rows), "context_window": window, "lengths": rows}


def fidelity(c: Client, o: dict) -> dict:
    """KL(sealed || served) and top-1 agreement over the sealed windows, computed from the served model's log-probabilities
    of every sealed id (``want``) at every position (rust/crates/cuteafd-bench/src/fidelity.rs in the reference; the file
    format is ``bench/fidelity.py``'s)."""
    import math

    from .fidelity import load_sealed
    if not o.get("windows"):
        return {"ok": False, "error": "fidelity needs the sealed windows file (--windows)"}
    sealed, info = load_sealed(o["windows"])
    toks, ids, lps, rest = sealed["tokens"], sealed["top_ids"], sealed["top_logprobs"], sealed["rest_logprob"]
    W, L = toks.shape
    kls, agree = [], []
    for w in range(min(W, int(o.get("fidelity_windows", 8)))):
        want = {str(p): [int(t) for t in ids[w, p - 1].tolist() if t >= 0] for p in range(1, L)}
        st, out = c.post("/v1/chat/completions", _ids_chat([int(t) for t in toks[w].tolist()], 1, cold=True, score_from=1, want=want, top_k=1))
        rows = {r["position"]: r for r in (out.get("probe") or {}).get("score_rows", [])} if st == 200 else {}
        if len(rows) < L - 1:
            return {"ok": False, "error": f"window {w}: status {st}, {len(rows)} of {L - 1} scored rows"}
        for p in range(1, L):
            q = rows[p]["want"]
            kl, q_mass = 0.0, 0.0
            for t, lp in zip(ids[w, p - 1].tolist(), lps[w, p - 1].tolist()):
                if t < 0:
                    continue
                lq = q[str(t)] if str(t) in q else q[t]
                q_mass += math.exp(lq)
                kl += math.exp(lp) * (lp - lq)
            lr = float(rest[w, p - 1])
            kl += math.exp(lr) * (lr - math.log(max(1.0 - q_mass, 1e-12)))
            kls.append(max(kl, 0.0))
            agree.append(1.0 if rows[p]["top_ids"][0] == int(ids[w, p - 1, 0]) else 0.0)
    kls.sort()
    kl_mean, top1 = sum(kls) / len(kls), sum(agree) / len(agree)
    return {"ok": kl_mean <= float(o.get("kl_bar", 0.05)) and top1 >= float(o.get("top1_bar", 0.93)), "windows": min(W, int(o.get("fidelity_windows", 8))),
            "positions": len(kls), "kl_mean": round(kl_mean, 6), "kl_p99": round(kls[min(len(kls) - 1, int(len(kls) * 0.99))], 6),
            "top1": round(top1, 4), "reference": info.get("model")}


PANELS = {"smoke": smoke, "cache_exact": cache_exact, "lossless": lossless, "template": template, "tools": tools, "speed": speed,
          "sweep": sweep, "sustained": sustained, "agentic": agentic, "context_load": context_load, "fidelity": fidelity}
QUICK = ("smoke", "cache_exact", "lossless", "template", "tools")


def run(url: str, panels: list[str], api_key: str = "", options: dict | None = None, log=print) -> dict:
    c = Client(url, api_key)
    out = {"url": url, "panels": []}
    for name in panels:
        if name not in PANELS:
            raise ValueError(f"unknown panel {name!r} (choose from {', '.join(PANELS)})")
        t0 = time.time()
        try:
            res = PANELS[name](c, options or {})
        except (OSError, KeyError, ValueError, http.client.HTTPException) as e:
            res = {"ok": False, "error": f"{type(e).__name__}: {e}"}
        res = dict({"panel": name, "seconds": round(time.time() - t0, 2)}, **res)
        try:
            st, th = c.get("/v1/thermal")
        except (OSError, http.client.HTTPException):
            st, th = 0, None                                   # the server is gone: the panel's own result says so
        if st == 200 and isinstance(th, dict) and th.get("available"):
            res["thermal"] = {g: {"verdict": w.get("verdict"), "sm_mhz": (w.get("sm_mhz") or {}).get("median")}
                              for g, w in (th.get("window") or {}).items()}
        out["panels"].append(res)
        log(json.dumps(res))
    out["ok"] = all(p["ok"] for p in out["panels"])
    return out
