"""Development fault hooks: failures injected on the host at named sites, to exercise the failure paths without ever
faulting a GPU.

``CUTEAFD_DIAG_FAULT_<SITE>=N`` makes site ``<SITE>`` raise ``InjectedFault`` once, on its N-th visit after the hooks
were armed (the server arms them when it is ready, so start-up traffic such as prewarm does not count).  The variables
are honoured only with ``CUTEAFD_DEV_FAULT_HOOKS=1``; without it a set variable is an error at start-up, so a production
configuration cannot carry one by accident.  Every site sits on the host before the step's work is submitted: the
failure is an exception of the scheduler's own thread, which takes the step's requests through the same worker-failure
path a device error would (release, or quarantine when the step may have reached the GPU).

Sites: ``BEFORE_PREFILL``, ``BEFORE_DECODE`` (host-side: nothing of the step was launched, pages are released),
``AFTER_SUBMISSION`` (raised as a device-class failure after the backend call returned: pages are quarantined),
``WIRE_SEND`` (the TCP expert link, before a request leaves).

Counterpart: rust/crates/cuteafd-daemon/src/shared/fault.rs:1-97 (``CUTEAFD_DIAG_FAULT_<SITE>=N`` behind the
``dev-fault-hooks`` feature, fire once on the N-th visit after readiness, release builds refuse).
"""
from __future__ import annotations

import os

SITES = ("BEFORE_PREFILL", "BEFORE_DECODE", "AFTER_SUBMISSION", "WIRE_SEND")
ENABLE, PREFIX = "CUTEAFD_DEV_FAULT_HOOKS", "CUTEAFD_DIAG_FAULT_"


class InjectedFault(RuntimeError):
    """Raised by a fault site.  ``device`` tells the scheduler which failure class to book it under."""

    def __init__(self, site: str, device: bool):
        super().__init__(f"injected fault at {site}")
        self.site, self.device = site, device


class FaultHooks:
    def __init__(self, env=None):
        env = os.environ if env is None else env
        asked = {k[len(PREFIX):]: v for k, v in env.items() if k.startswith(PREFIX)}
        if asked and env.get(ENABLE, "0") != "1":
            raise ValueError(f"{PREFIX}{next(iter(asked))} is set but {ENABLE}=1 is not: fault hooks are a development feature")
        self.plan: dict[str, int] = {}
        for site, v in asked.items():
            if site not in SITES:
                raise ValueError(f"unknown fault site {site} (choose from {', '.join(SITES)})")
            n = int(v)
            if n < 1:
                raise ValueError(f"{PREFIX}{site} counts visits from 1")
            self.plan[site] = n
        self.visits = {s: 0 for s in self.plan}
        self.fired: list[str] = []
        self.armed = False

    def arm(self) -> None:
        """Visits count from here (readiness)."""
        self.armed = True
        self.visits = {s: 0 for s in self.plan}

    def hit(self, site: str) -> None:
        if not self.armed or site not in self.plan or site in self.fired:
            return
        self.visits[site] += 1
        if self.visits[site] == self.plan[site]:
            self.fired.append(site)
            raise InjectedFault(site, device=site == "AFTER_SUBMISSION")


NONE = FaultHooks(env={})          # what a scheduler holds when nothing is configured: every ``hit`` is a no-op
