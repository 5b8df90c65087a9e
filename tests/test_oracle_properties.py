"""Properties of the fp32 oracle decoder that every engine test leans on: feeding a prompt in chunks gives the logits
and the cached rows of feeding it at once, whatever the chunk boundaries (python/reference/tests/
test_prefill_chunking_ref.py:32-43 and test_prefill_kv_boundaries_ref.py:28-39 in the reference), for every attention
form the engines implement; and truncating the cache and replaying gives the same continuation."""
import pytest
import torch
from hypothesis import given, settings
from hypothesis import strategies as st

from cuteafd_b200.config import ModelConfig, tiny_moe
from cuteafd_b200.ref.model import KvState, RefDecoder, init_weights


def _gqa(**kw) -> ModelConfig:
    return ModelConfig(name="gqa-tiny", family="qwen3_moe", vocab_size=256, num_layers=2, hidden=64, attention="gqa", num_heads=4,
                       num_kv_heads=2, head_dim=32, qk_norm=True, rope_theta=1.0e4, rope_interleaved=False, dense_ffn=128,
                       first_dense_layers=1, num_experts=4, expert_ffn=32, top_k=2, scoring="softmax", num_shared_experts=0,
                       norm_topk_prob=True).replace(**kw)


CONFIGS = {
    "mla": lambda: tiny_moe().replace(num_layers=2, vocab_size=256),
    "gqa": _gqa,
    "sliding-window": lambda: _gqa(sliding_window=9, window_layers=(1, 0)),
    "partial-rotary+bias": lambda: _gqa(family="glm4_moe", qk_norm=False, rotary_dim=16, attention_bias=True, scoring="sigmoid",
                                        router_bias=True),
}
_CACHE: dict = {}


def _model(name: str):
    if name not in _CACHE:
        cfg = CONFIGS[name]()
        _CACHE[name] = (cfg, RefDecoder(cfg, init_weights(cfg, seed=3)))
    return _CACHE[name]


@pytest.mark.parametrize("name", list(CONFIGS))
@settings(max_examples=12, deadline=None)
@given(cuts=st.lists(st.integers(1, 39), max_size=6, unique=True), seed=st.integers(0, 5))
def test_chunked_prefill_equals_whole_prefill(name, cuts, seed):
    cfg, ref = _model(name)
    toks = torch.randint(0, cfg.vocab_size, (40,), generator=torch.Generator().manual_seed(seed))
    whole_kv = KvState(cfg)
    with torch.no_grad():
        whole = ref.forward(toks, whole_kv)
        kv, outs, lo = KvState(cfg), [], 0
        for hi in sorted(cuts) + [40]:
            outs.append(ref.forward(toks[lo:hi], kv))
            lo = hi
    got = torch.cat(outs)
    assert torch.allclose(got, whole, atol=2e-4, rtol=1e-4), (got - whole).abs().max().item()
    for layer in range(cfg.num_layers):                       # the cached rows do not know where the chunks ended
        a, b = torch.cat(kv.rows[layer]), torch.cat(whole_kv.rows[layer])
        assert a.shape == b.shape and torch.allclose(a.float(), b.float(), atol=2e-4, rtol=1e-4)


@pytest.mark.parametrize("name", list(CONFIGS))
def test_truncate_and_replay_gives_the_same_continuation(name):
    """Rejected speculative rows: dropping the cache back to the accepted length and feeding the kept token again
    reproduces the step that would have run without the drafts."""
    cfg, ref = _model(name)
    toks = torch.randint(0, cfg.vocab_size, (30,), generator=torch.Generator().manual_seed(9))
    with torch.no_grad():
        kv = KvState(cfg)
        ref.forward(toks[:20], kv)
        plain = ref.forward(toks[20:21], kv)                   # one ordinary decode step
        kv2 = KvState(cfg)
        ref.forward(toks[:20], kv2)
        ref.forward(torch.cat([toks[20:21], toks[5:9]]), kv2)  # the same token followed by four drafts that get rejected
        kv2.truncate(20)
        again = ref.forward(toks[20:21], kv2)
    assert torch.allclose(plain, again, atol=2e-4, rtol=1e-4)
    assert kv.length() == kv2.length() == 21
