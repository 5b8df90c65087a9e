"""Development fault hooks: a configured site fails once on the host, the step's requests end with the worker class,
and the scheduler keeps serving.  No GPU work is ever made to fail."""
import pytest
import torch

from cuteafd_b200.config import tiny_moe
from cuteafd_b200.ref.model import init_weights
from cuteafd_b200.runtime.backends import OracleBackend
from cuteafd_b200.runtime.scheduler import FAIL_WORKER, Request, Scheduler, collect
from cuteafd_b200.utils.fault import ENABLE, PREFIX, FaultHooks, InjectedFault


@pytest.fixture(scope="module")
def oracle():
    cfg = tiny_moe()
    return cfg, init_weights(cfg, seed=0)


def _run(sched, reqs, steps=4000):
    for r in reqs:
        sched.submit(r)
    for _ in range(steps):
        if not sched.step() and sched.waiting.empty() and not sched.pending and not sched.prefilling and not sched.decoding:
            break
    return [collect(r, timeout=1.0) for r in reqs]


def test_hooks_are_refused_without_the_development_switch():
    with pytest.raises(ValueError, match="development"):
        FaultHooks(env={PREFIX + "BEFORE_DECODE": "1"})
    with pytest.raises(ValueError, match="unknown fault site"):
        FaultHooks(env={ENABLE: "1", PREFIX + "NOWHERE": "1"})
    with pytest.raises(ValueError, match="from 1"):
        FaultHooks(env={ENABLE: "1", PREFIX + "BEFORE_DECODE": "0"})
    assert FaultHooks(env={}).plan == {}


def test_a_site_fires_once_on_its_nth_visit_after_arming():
    h = FaultHooks(env={ENABLE: "1", PREFIX + "BEFORE_DECODE": "3"})
    h.hit("BEFORE_DECODE")                                          # before readiness: not counted
    h.arm()
    h.hit("BEFORE_DECODE"); h.hit("BEFORE_DECODE"); h.hit("BEFORE_PREFILL")
    with pytest.raises(InjectedFault) as e:
        h.hit("BEFORE_DECODE")
    assert e.value.site == "BEFORE_DECODE" and not e.value.device
    for _ in range(5):
        h.hit("BEFORE_DECODE")                                      # once only
    assert h.fired == ["BEFORE_DECODE"]


@pytest.mark.parametrize("site,quarantined", [("BEFORE_PREFILL", 0), ("BEFORE_DECODE", 0), ("AFTER_SUBMISSION", 1)])
def test_scheduler_survives_an_injected_fault(oracle, site, quarantined):
    cfg, params = oracle
    be = OracleBackend(cfg, params)
    s = Scheduler(be)
    s.faults = FaultHooks(env={ENABLE: "1", PREFIX + site: "1"})
    s.faults.arm()
    out = _run(s, [Request([1, 2, 3, 4], max_tokens=6)])[0]
    assert out["error"] and out["error"][0] == FAIL_WORKER and "injected fault" in out["error"][1]
    assert s.stats.failed == 1 and s.reserve.leased == 0
    assert s.stats.quarantined == quarantined                       # host-side failure: pages go back to the pool
    ok = _run(s, [Request([1, 2, 3, 4], max_tokens=6)])[0]
    clean = _run(Scheduler(OracleBackend(cfg, params)), [Request([1, 2, 3, 4], max_tokens=6)])[0]
    assert ok["error"] is None and ok["tokens"] == clean["tokens"]  # the next request is served, unchanged
