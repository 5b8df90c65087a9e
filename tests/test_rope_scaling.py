"""Long-context rope scaling: frequency tables against the transformers implementation, config round trip, and the
oracle's use of them."""
import math

import pytest
import torch

from cuteafd_b200 import tiny_moe
from cuteafd_b200.config import deepseek_v3
from cuteafd_b200.loader import snapshot
from cuteafd_b200.ref import ops
from cuteafd_b200.ref.model import KvState, RefDecoder, init_weights


def _hf_table(kind: str, dim: int, theta: float, params: dict):
    rope = pytest.importorskip("transformers.modeling_rope_utils")
    from transformers import LlamaConfig
    rp = dict(params, rope_type=kind, rope_theta=theta)
    try:
        cfg = LlamaConfig(hidden_size=dim * 4, num_attention_heads=4, head_dim=dim, max_position_embeddings=131072, rope_parameters=rp)
    except TypeError:
        pytest.skip("this transformers version takes rope settings differently")
    inv, att = rope.ROPE_INIT_FUNCTIONS[kind](cfg, "cpu")
    return inv.float(), float(att)


def test_yarn_table_matches_transformers():
    cfg = tiny_moe().replace(rope_theta=10000.0, rope_scaling="yarn", rope_factor=40.0, rope_original_max=4096,
                             rope_beta_fast=32.0, rope_beta_slow=1.0, rope_mscale=1.0, rope_mscale_all_dim=1.0)
    mine = ops.rope_inv_freq(cfg, 64)
    theirs, att = _hf_table("yarn", 64, 10000.0, {"factor": 40.0, "original_max_position_embeddings": 4096, "beta_fast": 32.0,
                                                  "beta_slow": 1.0, "mscale": 1.0, "mscale_all_dim": 1.0})
    assert torch.allclose(mine, theirs, rtol=1e-6, atol=0)
    mag, scale_mul = ops.rope_magnitudes(cfg)
    assert mag == pytest.approx(att) == pytest.approx(1.0)                     # equal mscales: nothing on cos / sin
    assert scale_mul == pytest.approx((0.1 * math.log(40.0) + 1.0) ** 2)       # DeepSeek: on the softmax scale instead
    plain = cfg.replace(rope_mscale_all_dim=0.0)
    theirs, att = _hf_table("yarn", 64, 10000.0, {"factor": 40.0, "original_max_position_embeddings": 4096})
    assert ops.rope_magnitudes(plain) == (pytest.approx(att), 1.0) and att == pytest.approx(0.1 * math.log(40.0) + 1.0)


def test_llama3_and_linear_tables_match_transformers():
    cfg = tiny_moe().replace(rope_theta=500000.0, rope_scaling="llama3", rope_factor=8.0, rope_original_max=8192,
                             rope_low_freq_factor=1.0, rope_high_freq_factor=4.0)
    theirs, att = _hf_table("llama3", 128, 500000.0, {"factor": 8.0, "original_max_position_embeddings": 8192,
                                                      "low_freq_factor": 1.0, "high_freq_factor": 4.0})
    mine = ops.rope_inv_freq(cfg, 128)
    assert torch.allclose(mine, theirs, rtol=1e-6, atol=0) and att == 1.0 and ops.rope_magnitudes(cfg) == (1.0, 1.0)
    base = ops.rope_inv_freq(cfg.replace(rope_scaling="none"), 128)
    assert torch.equal(mine[:8], base[:8]) and torch.allclose(mine[-1], base[-1] / 8.0)      # fast dims kept, slow dims interpolated
    lin = ops.rope_inv_freq(cfg.replace(rope_scaling="linear", rope_factor=4.0), 128)
    assert torch.allclose(lin, base / 4.0)


def test_config_round_trip_and_refusals():
    cfg = deepseek_v3()
    assert cfg.rope_scaling == "yarn" and cfg.rope_factor == 40.0
    back = snapshot.from_hf_config(snapshot.to_hf_config(cfg))
    for f in ("rope_scaling", "rope_factor", "rope_original_max", "rope_beta_fast", "rope_beta_slow", "rope_mscale", "rope_mscale_all_dim"):
        assert getattr(back, f) == getattr(cfg, f), f
    llama = {"model_type": "llama", "vocab_size": 128256, "num_hidden_layers": 2, "hidden_size": 4096, "num_attention_heads": 32,
             "num_key_value_heads": 8, "intermediate_size": 14336, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
             "max_position_embeddings": 131072,
             "rope_scaling": {"factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 8192,
                              "rope_type": "llama3"}}
    c = snapshot.from_hf_config(llama)
    assert (c.family, c.attention, c.head_dim, c.num_kv_heads, c.num_experts) == ("llama", "gqa", 128, 8, 0)
    assert c.rope_scaling == "llama3" and c.rope_original_max == 8192 and not c.is_moe_layer(1) and not c.rope_interleaved
    from cuteafd_b200.loader import families
    assert families.detect(llama).id == "llama"
    with pytest.raises(ValueError, match="rope scaling"):
        snapshot.from_hf_config(dict(llama, rope_scaling={"rope_type": "longrope", "factor": 4.0}))
    with pytest.raises(ValueError, match="bias"):
        snapshot.from_hf_config(dict(llama, attention_bias=True))
    assert snapshot.from_hf_config(dict(llama, model_type="mistral", sliding_window=4096)).window_of(1) == 4096
    with pytest.raises(ValueError, match="layer_types"):
        snapshot.from_hf_config(dict(llama, layer_types=["chunked_attention", "full_attention"]))
    v5 = dict(llama)                                                  # newer configs keep theta inside rope_parameters
    del v5["rope_scaling"], v5["rope_theta"]
    v5["rope_parameters"] = {"rope_type": "default", "rope_theta": 500000.0}
    c5 = snapshot.from_hf_config(v5)
    assert c5.rope_theta == 500000.0 and c5.rope_scaling == "none"


def test_oracle_uses_the_scaled_table_and_llama_runs():
    cfg = tiny_moe()
    params = init_weights(cfg, seed=0)
    toks = torch.arange(40) % cfg.vocab_size
    plain = RefDecoder(cfg, params).forward(toks, KvState(cfg))
    ycfg = cfg.replace(rope_scaling="yarn", rope_factor=40.0, rope_original_max=16, rope_mscale=1.0, rope_mscale_all_dim=1.0)
    dec = RefDecoder(ycfg, params)
    assert dec.scale_mul > 1.3 and not torch.equal(dec.inv_freq, RefDecoder(cfg, params).inv_freq)
    scaled = dec.forward(toks, KvState(ycfg))
    assert torch.isfinite(scaled).all() and not torch.allclose(scaled, plain)
    # factor 1 is the identity whatever the kind says
    same = RefDecoder(cfg.replace(rope_scaling="yarn", rope_factor=1.0), params).forward(toks, KvState(cfg))
    assert torch.equal(same, plain)
    # a dense llama-shaped model goes through the same decoder (every layer dense, rotate-half rope)
    lcfg = cfg.replace(family="llama", attention="gqa", num_heads=2, num_kv_heads=1, head_dim=64, hidden=128, dense_ffn=256,
                       num_experts=0, first_dense_layers=cfg.num_layers, num_shared_experts=0, top_k=0, rope_interleaved=False,
                       rope_scaling="llama3", rope_factor=8.0, rope_original_max=32)
    out = RefDecoder(lcfg, init_weights(lcfg, seed=1)).forward(toks, KvState(lcfg))
    assert out.shape == (40, lcfg.vocab_size) and torch.isfinite(out).all()
