"""Hosted web search for the gateway: providers, a per-session page cache, and the tool loop.

Clients that expect a server-side search tool (Anthropic ``web_search_*``, Responses ``web_search``) declare it in
``tools``; the gateway shows the upstream model a plain function tool ``web_search(query)``, runs the search itself
when the model calls it, appends the hits as a tool message and asks the model again (``run_tool_loop``, at most
``MAX_ROUNDS`` searches per request).  ``POST /v1/alpha/search`` exposes the same providers directly with the
``search`` / ``open`` / ``find`` / ``time`` commands client-executed search extensions use; anything else answers with
an explicit "unsupported" tool output instead of failing the request.

Providers (the base URL is configuration, so a test or an air-gapped site points them at a local service):

* ``Exa``      ``POST {base}/search`` with ``x-api-key``; body ``{query, numResults, includeDomains, excludeDomains,
               contents: {text: {maxCharacters}}}``; hits carry extracted page text, so ``open`` needs no second fetch.
* ``Searxng``  ``GET {base}/search?q=...&format=json``; hits carry snippets; domain filters are applied here.

``SearchSession`` keeps what a session has seen: hits get short references (``ref_1`` ...) that ``open`` and ``find``
take; a page is only ever served from this cache (an uncached URL is never fetched on the client's behalf); entries
expire after an hour without use and the cache is bounded.

Counterpart: rust/crates/cuteafd-api/src/gateway/search.rs (SearchQuery / SearchHit / SearchProvider, hosted tool),
search/providers.rs (Exa, SearXNG), docs/client-apis.md:105-118 (``/v1/alpha/search`` semantics).
"""
from __future__ import annotations

import json
import threading
import time
import urllib.error
import urllib.parse
import urllib.request
from dataclasses import asdict, dataclass, field

TOOL_NAME = "web_search"
MAX_ROUNDS = 3
HOSTED_TYPES = ("web_search", "web_search_preview", "web_search_20250305")


class SearchError(RuntimeError):
    pass


@dataclass
class SearchQuery:
    query: str
    allowed_domains: list[str] = field(default_factory=list)
    blocked_domains: list[str] = field(default_factory=list)
    max_results: int = 5


@dataclass
class SearchHit:
    url: str
    title: str
    content: str
    published: str | None = None


def _host(url: str) -> str:
    return (urllib.parse.urlparse(url).hostname or "").lower()


def domain_ok(url: str, q: SearchQuery) -> bool:
    h = _host(url)

    def under(d: str) -> bool:
        d = d.lower().lstrip(".")
        return h == d or h.endswith("." + d)
    if q.allowed_domains and not any(under(d) for d in q.allowed_domains):
        return False
    return not any(under(d) for d in q.blocked_domains)


def _http_json(req: urllib.request.Request, timeout: float) -> dict:
    try:
        with urllib.request.urlopen(req, timeout=timeout) as r:
            return json.loads(r.read())
    except urllib.error.HTTPError as e:
        raise SearchError(f"search provider answered {e.code}") from e
    except (urllib.error.URLError, TimeoutError, json.JSONDecodeError) as e:
        raise SearchError(f"search provider unavailable: {e}") from e


class Exa:
    name = "exa"

    def __init__(self, api_key: str, base: str = "https://api.exa.ai", max_chars: int = 4000, timeout: float = 20.0):
        self.key, self.base, self.max_chars, self.timeout = api_key, base.rstrip("/"), max_chars, timeout

    def search(self, q: SearchQuery, recency_days: int | None = None) -> list[SearchHit]:
        body = {"query": q.query, "numResults": q.max_results, "contents": {"text": {"maxCharacters": self.max_chars}}}
        if q.allowed_domains:
            body["includeDomains"] = q.allowed_domains
        if q.blocked_domains:
            body["excludeDomains"] = q.blocked_domains
        if recency_days:
            body["startPublishedDate"] = time.strftime("%Y-%m-%dT%H:%M:%S.000Z", time.gmtime(time.time() - recency_days * 86400))
        req = urllib.request.Request(self.base + "/search", json.dumps(body).encode(),
                                     {"Content-Type": "application/json", "x-api-key": self.key})
        res = _http_json(req, self.timeout).get("results", [])
        hits = [SearchHit(r.get("url", ""), r.get("title") or r.get("url", ""), (r.get("text") or r.get("summary") or "")[: self.max_chars],
                          r.get("publishedDate")) for r in res if r.get("url")]
        return [h for h in hits if domain_ok(h.url, q)][: q.max_results]


class Searxng:
    name = "searxng"

    def __init__(self, base: str, timeout: float = 20.0):
        self.base, self.timeout = base.rstrip("/"), timeout

    def search(self, q: SearchQuery, recency_days: int | None = None) -> list[SearchHit]:
        args = {"q": q.query, "format": "json"}
        if recency_days:
            args["time_range"] = "day" if recency_days <= 1 else "week" if recency_days <= 7 else "month" if recency_days <= 31 else "year"
        req = urllib.request.Request(self.base + "/search?" + urllib.parse.urlencode(args), headers={"Accept": "application/json"})
        res = _http_json(req, self.timeout).get("results", [])
        hits = [SearchHit(r.get("url", ""), r.get("title") or r.get("url", ""), r.get("content") or "", r.get("publishedDate"))
                for r in res if r.get("url")]
        return [h for h in hits if domain_ok(h.url, q)][: q.max_results]


def provider_from_env(env: dict) -> "Exa | Searxng | None":
    """``EXA_API_KEY`` (+ optional ``EXA_BASE_URL``) or ``SEARXNG_URL``; None when neither is set."""
    if env.get("EXA_API_KEY"):
        return Exa(env["EXA_API_KEY"], env.get("EXA_BASE_URL", "https://api.exa.ai"))
    if env.get("SEARXNG_URL"):
        return Searxng(env["SEARXNG_URL"])
    return None


# ---- session cache -----------------------------------------------------------------------------------
class SearchSession:
    """Pages and references one client session has seen."""
    TTL = 3600.0
    MAX_PAGES = 256

    def __init__(self, clock=time.monotonic):
        self.clock = clock
        self.lock = threading.Lock()
        self.pages: dict[str, tuple[float, SearchHit]] = {}      # url -> (last use, hit)
        self.refs: dict[str, str] = {}                            # ref -> url
        self._n = 0

    def _expire(self) -> None:
        now = self.clock()
        for url in [u for u, (t, _) in self.pages.items() if now - t > self.TTL]:
            del self.pages[url]
        while len(self.pages) > self.MAX_PAGES:
            del self.pages[min(self.pages, key=lambda u: self.pages[u][0])]
        self.refs = {r: u for r, u in self.refs.items() if u in self.pages}

    def remember(self, hits: list[SearchHit]) -> list[dict]:
        out = []
        with self.lock:
            now = self.clock()
            for h in hits:
                self.pages[h.url] = (now, h)
                ref = next((r for r, u in self.refs.items() if u == h.url), None)
                if ref is None:
                    self._n += 1
                    ref = f"ref_{self._n}"
                    self.refs[ref] = h.url
                out.append(dict(asdict(h), ref=ref))
            self._expire()
        return out

    def open(self, ref_or_url: str) -> SearchHit | None:
        with self.lock:
            self._expire()
            url = self.refs.get(ref_or_url, ref_or_url)
            got = self.pages.get(url)
            if got is None:
                return None
            self.pages[url] = (self.clock(), got[1])
            return got[1]

    def find(self, ref_or_url: str, pattern: str, width: int = 160, limit: int = 8) -> list[str] | None:
        page = self.open(ref_or_url)
        if page is None:
            return None
        text, low, pat = page.content, page.content.lower(), pattern.lower()
        out, at = [], 0
        while pat and len(out) < limit:
            i = low.find(pat, at)
            if i < 0:
                break
            out.append(text[max(0, i - width // 2): i + len(pat) + width // 2])
            at = i + len(pat)
        return out


def alpha_search(provider, session: SearchSession, body: dict) -> dict:
    """One ``/v1/alpha/search`` command.  Always answers with a tool output; errors are outputs too."""
    cmd = body.get("command") or ("search" if "query" in body else "")
    try:
        if cmd == "search":
            if provider is None:
                return {"ok": False, "output": "no search provider is configured"}
            q = SearchQuery(str(body.get("query", "")), list(body.get("allowed_domains", [])), list(body.get("blocked_domains", [])),
                            max(1, min(int(body.get("max_results", 5)), 20)))
            if not q.query.strip():
                return {"ok": False, "output": "empty query"}
            return {"ok": True, "provider": provider.name, "results": session.remember(provider.search(q, body.get("recency")))}
        if cmd == "open":
            page = session.open(str(body.get("ref") or body.get("url") or ""))
            if page is None:
                return {"ok": False, "output": "that page is not in this session's cache (references expire after an hour): search again"}
            return {"ok": True, "page": asdict(page)}
        if cmd == "find":
            got = session.find(str(body.get("ref") or body.get("url") or ""), str(body.get("pattern", "")))
            if got is None:
                return {"ok": False, "output": "that page is not in this session's cache: open a search result first"}
            return {"ok": True, "matches": got}
        if cmd == "time":
            return {"ok": True, "utc": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime())}
    except SearchError as e:
        return {"ok": False, "output": str(e)}
    return {"ok": False, "output": f"unsupported command {cmd!r} (supported: search, open, find, time)"}


# ---- hosted tool ------------------------------------------------------------------------------------------
def wants_hosted_search(body: dict) -> dict | None:
    """The client's hosted search tool declaration, if any."""
    for t in body.get("tools") or []:
        if isinstance(t, dict) and (t.get("type") in HOSTED_TYPES or str(t.get("type", "")).startswith("web_search")):
            return t
    return None


def function_tool() -> dict:
    return {"type": "function", "function": {
        "name": TOOL_NAME, "description": "Search the web. Returns titles, URLs and page text.",
        "parameters": {"type": "object", "properties": {"query": {"type": "string"}}, "required": ["query"]}}}


def format_hits(hits: list[dict]) -> str:
    if not hits:
        return "no results"
    return "\n\n".join(f"[{h['ref']}] {h['title']}\n{h['url']}" + (f" ({h['published']})" if h.get("published") else "") +
                       f"\n{h['content']}" for h in hits)


def run_tool_loop(chat, fwd: dict, decl: dict, provider, session: SearchSession) -> tuple[dict, list[dict]]:
    """``chat(body) -> reply`` calls the upstream.  Returns (final reply, searches run: [{query, results}])."""
    fwd = dict(fwd, tools=list(fwd.get("tools") or []) + [function_tool()], messages=list(fwd["messages"]))
    ran: list[dict] = []
    budget = int(decl.get("max_uses") or MAX_ROUNDS)
    for _ in range(min(budget, MAX_ROUNDS) + 1):
        reply = chat(fwd)
        msg = reply["choices"][0]["message"]
        calls = [c for c in msg.get("tool_calls") or [] if c.get("function", {}).get("name") == TOOL_NAME]
        if not calls or len(ran) >= min(budget, MAX_ROUNDS):
            return reply, ran
        fwd["messages"].append({"role": "assistant", "content": msg.get("content") or "", "tool_calls": msg["tool_calls"]})
        for c in calls:
            try:
                args = json.loads(c["function"].get("arguments") or "{}")
            except json.JSONDecodeError:
                args = {}
            q = SearchQuery(str(args.get("query", "")), list(decl.get("allowed_domains") or []), list(decl.get("blocked_domains") or []))
            try:
                hits = session.remember(provider.search(q)) if q.query.strip() else []
                text = format_hits(hits)
            except SearchError as e:
                hits, text = [], f"search failed: {e}"
            ran.append({"query": q.query, "results": hits})
            fwd["messages"].append({"role": "tool", "tool_call_id": c.get("id", ""), "content": text})
    return reply, ran
