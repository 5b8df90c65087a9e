"""Live console: one JSON document that describes what the server is doing now, and the page that renders it.

``console_state(state)`` gathers, without stopping the serve loop (the scheduler's lists are copied, counters read):

* ``lanes``      one row per request in flight: phase (prefill / decode / stalled), decode lane, prompt progress,
                 generated tokens, KV length, draft acceptance and tokens per verify cycle, age, time to first token
* ``pipeline``   queue depth, admitted / finished / failed / rejected, prefill and decode shares of recent step time,
                 packed prefill steps, KV stalls, loop aborts
* ``drafts``     lifetime proposed / accepted / acceptance, explore skips, budget cuts, verify-row histogram
* ``graphs``     decode graph bank: captured geometries, replays, eager steps
* ``prefix``     prefix cache hits, shared tokens, pages held
* ``memory``     ledger by kind and per device (tracked / used / untracked)
* ``thermal``    latest sample and last-minute verdict per GPU
* ``experts``    routed-expert token counts per layer when the deployment publishes them

Routes: ``/`` and ``/v1/console`` (page), ``/v1/console/state`` (this JSON), ``/console/memory``, ``/console/experts``.

Counterpart: rust/crates/cuteafd-daemon/src/shared/console.rs (+ console/*), rust/crates/cuteafd-api/src/openai/
console.rs, memory.rs, expert_usage.rs; docs/dashboard.md.
"""
from __future__ import annotations

import time


def console_state(state) -> dict:
    sched = state.sched
    snap = sched.snapshot()
    be = sched.be
    life = snap.get("draft_policy", {})
    prop = life.get("proposed", 0)
    out = {
        "model": state.model_id,
        "uptime_s": round(time.time() - state.started, 1),
        "ready": sched.ready.is_set(),
        "lanes": sched.lanes(),
        "pipeline": {k: snap.get(k) for k in ("queued", "prefilling", "active", "admitted", "finished", "failed", "rejected",
                                              "prefill_tokens", "cached_tokens", "decode_rounds", "emitted_tokens",
                                              "packed_steps", "stalls", "quarantined", "loop_aborts", "time_share",
                                              "lane_rounds", "kv")},
        "drafts": dict(life, acceptance=round(life.get("accepted", 0) / prop, 3) if prop else None,
                       tokens_per_round=round(snap["emitted_tokens"] / snap["decode_rounds"], 2) if snap.get("decode_rounds") else None,
                       verify_row_hist=snap.get("verify_row_hist", {})),
    }
    if hasattr(be, "graph_stats"):
        out["graphs"] = be.graph_stats()
    if hasattr(be, "prefix"):
        out["prefix"] = be.prefix.describe()
    from ..utils.memory_ledger import LEDGER
    rep = LEDGER.report()
    out["memory"] = {"by_kind": rep["by_kind"], "devices": rep["devices"], "failures": len(rep["failures"])}
    try:
        from ..utils.thermal import monitor
        th = monitor().report(60.0)
        out["thermal"] = {"available": th["available"],
                          "gpus": {str(g): {"sm_mhz": w.get("sm_mhz", {}).get("median"), "power_w": w.get("power_w", {}).get("max"),
                                            "temp_c": w.get("temp_c", {}).get("max"), "verdict": w.get("verdict")}
                                   for g, w in th.get("window", {}).items()}}
    except Exception:                                              # noqa: BLE001 - telemetry never breaks the console
        out["thermal"] = {"available": False, "gpus": {}}
    fn = state.extras.get("expert_usage")
    if fn:
        out["experts"] = fn()
    if state.usage:
        out["usage"] = state.usage.summary(1.0)
    return out


PAGE = """<!doctype html><meta charset=utf-8><title>cuteafd_b200 console</title>
<style>
body{font:13px/1.4 ui-monospace,monospace;margin:1.5em;background:#0c0f12;color:#d6dde4}
h1{font-size:16px;margin:0 0 .6em}h2{font-size:13px;margin:1.4em 0 .3em;color:#8fb6ff}
table{border-collapse:collapse}td,th{padding:2px 10px;text-align:right;border-bottom:1px solid #1e252c}
th{color:#7d8a97;font-weight:normal}td:first-child,th:first-child{text-align:left}
.bar{display:inline-block;height:8px;background:#3d7eff;vertical-align:middle}
.ok{color:#7ee787}.warn{color:#f0b429}.bad{color:#ff6b6b}.dim{color:#66727f}
#grid{display:grid;grid-template-columns:repeat(auto-fit,minmax(330px,1fr));gap:0 2em}
</style>
<h1 id=title>cuteafd_b200</h1>
<h2>requests in flight</h2><table id=lanes></table>
<div id=grid>
<div><h2>pipeline</h2><table id=pipe></table></div>
<div><h2>drafts</h2><table id=drafts></table></div>
<div><h2>memory</h2><table id=mem></table></div>
<div><h2>GPUs</h2><table id=gpus></table></div>
<div><h2>prefix cache / graphs</h2><table id=cache></table></div>
<div><h2>last hour</h2><table id=usage></table></div>
</div>
<script>
const gib=b=>b==null?'':(b/2**30).toFixed(2)+' GiB';
const esc=s=>String(s??'').replace(/[&<>]/g,c=>({'&':'&amp;','<':'&lt;','>':'&gt;'}[c]));
function kv(id,obj){document.getElementById(id).innerHTML=Object.entries(obj).filter(([k,v])=>v!==undefined)
 .map(([k,v])=>`<tr><td>${esc(k)}</td><td>${esc(typeof v==='object'&&v!==null?JSON.stringify(v):v)}</td></tr>`).join('')}
const key=new URLSearchParams(location.search).get('key');   // a server started with an API key: open /?key=...
async function tick(){
 let s;try{s=await (await fetch('/v1/console/state',{headers:key?{Authorization:'Bearer '+key}:{}})).json()}catch(e){return}
 if(s.error){document.getElementById('title').textContent='API key required: open /?key=<key>';return}
 document.getElementById('title').textContent=`${s.model} · up ${s.uptime_s}s · ${s.ready?'ready':'starting'}`;
 const cols=['rid','phase','lane','prompt','generated','kv_len','acceptance','tok/cycle','ttft_s','age_s'];
 document.getElementById('lanes').innerHTML='<tr>'+cols.map(c=>`<th>${c}</th>`).join('')+'</tr>'+
  (s.lanes.length?s.lanes.map(l=>`<tr><td>${l.rid}</td><td class=${l.phase=='stalled'?'warn':'ok'}>${l.phase}</td><td>${l.lane}</td>
  <td>${l.prompt_done}/${l.prompt_tokens} <span class=dim>(${l.cached_tokens} cached)</span></td>
  <td>${l.generated}/${l.max_tokens} <span class=bar style="width:${Math.round(60*l.generated/l.max_tokens)}px"></span></td>
  <td>${l.kv_len}</td><td>${l.acceptance??''}</td><td>${l.tokens_per_cycle??''}</td><td>${l.ttft_s??''}</td><td>${l.age_s}</td></tr>`).join('')
  :'<tr><td class=dim colspan=10>idle</td></tr>');
 kv('pipe',s.pipeline);kv('drafts',s.drafts);
 const m={};for(const[k,v]of Object.entries(s.memory.by_kind))m[k]=gib(v);
 for(const[d,r]of Object.entries(s.memory.devices))m[d]=`tracked ${gib(r.tracked)} · used ${gib(r.used)} · untracked ${gib(r.untracked)}`;
 if(s.memory.failures)m['allocation failures']=s.memory.failures;kv('mem',m);
 const g={};for(const[i,w]of Object.entries(s.thermal.gpus))g['gpu'+i]=`${w.sm_mhz??'?'} MHz · ${w.power_w??'?'} W · ${w.temp_c??'?'} °C · ${w.verdict}`;
 kv('gpus',Object.keys(g).length?g:{telemetry:'unavailable'});
 kv('cache',Object.assign({},s.prefix||{},s.graphs||{}));kv('usage',s.usage||{accounting:'off'});
}
tick();setInterval(tick,1000);
</script>
"""
