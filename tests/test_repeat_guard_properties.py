"""Loop-abort detector: the C++ form and the Python form fire at the same token with the same rule and period on any
stream, a stream without an exact loop never fires, and an injected loop fires where the rules' arithmetic says."""
import random

import pytest
from hypothesis import given, settings
from hypothesis import strategies as st

from cuteafd_b200.runtime.repeat_guard import LoopAbortConfig, RepeatGuard


def _native(cfg):
    try:
        from cuteafd_b200.runtime.native import NativeRepeatGuard, enabled
        return NativeRepeatGuard(cfg) if enabled() else None
    except (OSError, AttributeError, ImportError):
        return None


def _stream(seed: int, prefix: int, period: int, copies: int, noise_every: int) -> list[int]:
    rnd = random.Random(seed)
    out = [rnd.randrange(50, 5000) for _ in range(prefix)]
    block = [rnd.randrange(50, 5000) for _ in range(period)]
    for c in range(copies):
        out += block
        if noise_every and (c + 1) % noise_every == 0:
            out.append(rnd.randrange(5000, 6000))             # a break in the loop: the count starts again
    return out


@settings(max_examples=60)
@given(seed=st.integers(0, 999), prefix=st.integers(0, 300), period=st.sampled_from([1, 2, 7, 64, 255, 256, 257, 300, 700]),
       copies=st.integers(1, 14), noise_every=st.sampled_from([0, 0, 3, 5]),
       cfg=st.sampled_from([LoopAbortConfig(), LoopAbortConfig(64, 3, 128, 3), LoopAbortConfig(0, 8, 200, 4), LoopAbortConfig(100, 4, 0, 8)]))
def test_both_forms_agree_on_every_stream(seed, prefix, period, copies, noise_every, cfg):
    toks = _stream(seed, prefix, period, copies, noise_every)
    py, nat = RepeatGuard(cfg), _native(cfg)
    fired_py = next((i + 1 for i, t in enumerate(toks) if py.push(t)), None)
    if nat is not None:
        fired_nat = next((i + 1 for i, t in enumerate(toks) if nat.push(t)), None)
        assert fired_nat == fired_py, (fired_nat, fired_py, py.hit)
    if fired_py is not None:
        assert py.hit["rule"] in ("fast", "repeat") and py.hit["at"] == fired_py
        if py.hit["rule"] == "fast":
            assert py.hit["period"] <= 256 and period % py.hit["period"] == 0 or py.hit["period"] % period == 0
    if copies == 1 and prefix + period < 64:
        assert fired_py is None


def test_random_text_never_fires_and_a_single_token_fires_at_the_span():
    rnd = random.Random(3)
    g = RepeatGuard(LoopAbortConfig())
    assert not any(g.push(rnd.randrange(100000)) for _ in range(20000))
    g = RepeatGuard(LoopAbortConfig())
    at = next(i + 1 for i in range(5000) if g.push(7))
    assert at == 1025 and g.hit["rule"] == "fast" and g.hit["period"] == 1
