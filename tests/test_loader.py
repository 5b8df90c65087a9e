"""Checkpoint layer on CPU: codecs, safetensors catalog, format detection, family registry,
random-init snapshots in every shipped format, and decode-to-oracle round trips."""
import json
import os

import pytest
import torch

from cuteafd_b200 import ModelConfig, tiny_moe
from cuteafd_b200.loader import families, formats, load, snapshot
from cuteafd_b200.loader.safetensors_io import Catalog, write_file
from cuteafd_b200.quant import codecs


def small() -> ModelConfig:
    return tiny_moe().replace(expert_ffn=128, hidden=256, dense_ffn=256)


def test_fp8_block_and_row_codecs():
    w = torch.randn(300, 512) * 0.02
    q, s = codecs.fp8_quant_block128(w)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (3, 4)
    assert (codecs.fp8_dequant_block128(q, s) - w).abs().max() < 0.07 * w.abs().max()
    x = torch.randn(5, 256)
    qx, sx = codecs.fp8_quant_rows(x)
    assert sx.shape == (5, 2)
    assert (codecs.fp8_dequant_rows(qx, sx) - x).abs().max() < 0.07 * x.abs().max()
    z, sz = codecs.fp8_quant_rows(torch.zeros(2, 128))
    assert torch.all(sz == 1.0) and torch.all(z.float() == 0)


def test_fp4_codecs_and_nibble_order():
    codes = torch.tensor([[1, 2, 3, 4]], dtype=torch.uint8)
    packed = codecs.pack_nibbles(codes)
    assert packed.tolist() == [[0x21, 0x43]]                 # even element in the low nibble
    assert torch.equal(codecs.unpack_nibbles(packed), codes)
    w = torch.randn(64, 256) * 0.02
    p, e = codecs.mxfp4_quant(w)
    assert p.shape == (64, 128) and e.shape == (64, 8) and e.dtype == torch.uint8
    assert (codecs.mxfp4_dequant(p, e) - w).abs().max() < 0.3 * w.abs().max()
    p, bs, g = codecs.nvfp4_quant(w)
    assert bs.dtype == torch.float8_e4m3fn and bs.shape == (64, 16) and g.shape == (1,)
    assert (codecs.nvfp4_dequant(p, bs, g) - w).abs().max() < 0.3 * w.abs().max()
    exact = torch.tensor([[0.5, -1.5, 6.0, -0.0] * 8]) * 2.0      # representable values survive exactly
    p, e = codecs.mxfp4_quant(exact)
    assert torch.equal(codecs.mxfp4_dequant(p, e), exact)


def test_exl3_decode_properties():
    g = torch.Generator().manual_seed(0)
    for bits in (2, 4):
        t, suh, svh = codecs.exl3_random(128, 256, bits, g)
        inner = codecs.exl3_decode_inner(t)
        assert inner.shape == (128, 256) and torch.isfinite(inner).all()
        w = codecs.exl3_dequant(t, suh, svh)
        assert w.shape == (128, 256)
        # the rotations are orthonormal: energy is preserved up to the sign-scale vectors
        assert torch.allclose(w.pow(2).sum(), (inner.double() * svh.double().abs()[None]).pow(2).sum(), rtol=1e-6)
    h = codecs.hadamard128(torch.eye(128))
    assert torch.allclose(h @ h.T, torch.eye(128, dtype=torch.float64), atol=1e-9)


def test_safetensors_catalog_roundtrip(tmp_path):
    tensors = {"a.weight": torch.randn(8, 16).to(torch.bfloat16), "b": torch.arange(10, dtype=torch.int32),
               "c.weight": torch.randn(4, 128).to(torch.float8_e4m3fn), "d": torch.randint(-9, 9, (3, 2, 32), dtype=torch.int16)}
    write_file(str(tmp_path / "model.safetensors"), tensors, {"format": "pt"})
    cat = Catalog(str(tmp_path))
    assert cat.names() == sorted(tensors)
    for k, v in tensors.items():
        got = cat.read(k)
        assert got.dtype == v.dtype and torch.equal(got.view(torch.uint8), v.view(torch.uint8))
    assert torch.equal(cat.read_rows("a.weight", 2, 3), tensors["a.weight"][2:5])
    assert len(cat.sha256("b")) == 64
    assert cat.total_bytes() == sum(t.numel() * t.element_size() for t in tensors.values())


@pytest.mark.parametrize("fmt", ["bf16", "fp8_block128", "nvfp4", "mxfp4", "exl3_k4"])
def test_random_snapshot_formats(tmp_path, fmt):
    cfg = small()
    d = snapshot.write_random_snapshot(cfg, str(tmp_path / fmt), fmt=fmt, seed=3)
    assert os.path.exists(os.path.join(d, "model.safetensors.index.json"))
    snap = load.open_snapshot(d)
    assert snap.family is not None and snap.model is not None
    assert snap.cfg.hidden == cfg.hidden and snap.cfg.num_experts == cfg.num_experts
    assert snap.hints() == []
    op = snap.operands["model.layers.1.mlp.experts.3.down_proj"]
    assert op.format.startswith(fmt.split("_k")[0])
    assert op.shape == (cfg.hidden, cfg.expert_ffn)
    assert snap.model.classify(op.weight) == ("routed_expert", 1, 3)
    assert snap.model.classify("model.layers.0.mlp.down_proj.weight")[0] == "dense_ffn"
    assert snap.model.classify("model.layers.1.mlp.gate.weight")[0] == "router"
    w = formats.dequantize(op, snap.catalog)
    assert w.shape == (cfg.hidden, cfg.expert_ffn) and torch.isfinite(w).all()
    if not fmt.startswith("exl3"):
        from cuteafd_b200.ref.model import init_weights
        ref = init_weights(cfg.replace(weight_format=fmt), seed=3)["model.layers.1.mlp.experts.3.down_proj.weight"]
        tol = {"bf16": 0.01, "fp8_block128": 0.08}.get(fmt, 0.3)
        assert (w - ref).abs().max() < tol * ref.abs().max()


def test_loaded_params_run_the_oracle(tmp_path):
    from cuteafd_b200.ref.model import KvState, RefDecoder
    cfg = small()
    d = snapshot.write_random_snapshot(cfg, str(tmp_path / "s"), fmt="fp8_block128", seed=0, scope="linear")
    cfg2, params = load.load_params(d)
    assert cfg2.weight_format == "fp8_block128"
    logits = RefDecoder(cfg2, params).forward(torch.arange(12) % cfg.vocab_size, KvState(cfg2))
    assert logits.shape == (12, cfg.vocab_size) and torch.isfinite(logits).all()


def test_unsupported_is_a_result_not_a_crash(tmp_path):
    cfg = small()
    d = snapshot.write_random_snapshot(cfg, str(tmp_path / "s"), fmt="bf16")
    hf = json.load(open(os.path.join(d, "config.json")))
    hf["model_type"] = "some_future_arch"
    assert families.detect(hf) is None
    snap = load.open_snapshot(d)
    op = snap.operands["model.layers.1.mlp.gate"]
    bad = formats.QuantOperand(op.name, "e4m3", op.shape, op.weight)
    hint = snap.model.accepts(bad, "router")
    assert isinstance(hint, families.Hint) and "router" in hint.what


def test_hf_config_roundtrip():
    from cuteafd_b200 import deepseek_v3, deepseek_v32, qwen3_30b_a3b
    for cfg in (qwen3_30b_a3b(), deepseek_v3(), deepseek_v32(), tiny_moe()):
        back = snapshot.from_hf_config(snapshot.to_hf_config(cfg))
        for f in ("hidden", "num_layers", "num_heads", "num_experts", "top_k", "expert_ffn", "attention", "scoring",
                  "num_groups", "topk_groups", "first_dense_layers", "mtp_layers", "indexer_heads", "weight_format"):
            assert getattr(back, f) == getattr(cfg, f), (cfg.name, f)


def test_mixtral_style_names_are_canonicalised(tmp_path):
    """A checkpoint that names its MoE block ``block_sparse_moe`` and its projections w1 / w3 / w2 loads like any other:
    the catalogue shows canonical names, the operands classify as routed experts, the oracle gives the same logits."""
    from cuteafd_b200.loader.safetensors_io import write_sharded
    from cuteafd_b200.ref.model import KvState, RefDecoder, init_weights
    cfg = tiny_moe().replace(family="qwen3_moe", attention="gqa", num_heads=2, num_kv_heads=2, head_dim=64, hidden=128,
                             expert_ffn=128, dense_ffn=128, num_experts=4, top_k=2, vocab_size=256, num_shared_experts=0,
                             scoring="softmax", first_dense_layers=0, qk_norm=False)
    params = init_weights(cfg, seed=5)
    proj = {"gate_proj": "w1", "up_proj": "w3", "down_proj": "w2"}
    renamed = {}
    for k, v in params.items():
        k2 = k.replace(".mlp.gate.", ".block_sparse_moe.gate.")
        if ".mlp.experts." in k2:
            k2 = k2.replace(".mlp.experts.", ".block_sparse_moe.experts.")
            for a, b in proj.items():
                k2 = k2.replace("." + a + ".", "." + b + ".")
        renamed[k2] = v.to(torch.bfloat16)
    assert any(".block_sparse_moe.experts.0.w1.weight" in k for k in renamed)
    d = str(tmp_path / "mixtral")
    os.makedirs(d)
    hf = snapshot.to_hf_config(cfg)
    hf.update(model_type="mixtral", num_local_experts=cfg.num_experts)
    hf.pop("num_experts", None); hf.pop("qk_norm", None)
    json.dump(hf, open(os.path.join(d, "config.json"), "w"))
    write_sharded(d, renamed, 1 << 20)
    snap = load.open_snapshot(d)
    assert snap.family is not None and snap.family.id == "qwen3_moe" and snap.cfg.num_experts == 4 and not snap.cfg.qk_norm
    op = snap.operands["model.layers.1.mlp.experts.2.up_proj"]
    assert snap.model.classify(op.weight) == ("routed_expert", 1, 2) and snap.hints() == []
    cfg2, loaded = load.load_params(d)
    toks = torch.arange(9) % cfg.vocab_size
    want = RefDecoder(cfg, {k: v.to(torch.bfloat16).float() for k, v in params.items()}).forward(toks, KvState(cfg))
    got = RefDecoder(cfg2, loaded).forward(toks, KvState(cfg2))
    assert torch.allclose(got, want, atol=1e-4)


def test_new_presets_are_consistent():
    from cuteafd_b200 import PRESETS, kimi_k2, mixtral_8x7b
    m, k = mixtral_8x7b(), kimi_k2()
    assert PRESETS["mixtral-8x7b"]().num_experts == 8 and m.head_dim * m.num_heads == m.hidden
    assert k.is_mla and k.num_experts == 384 and 128 % k.num_heads == 0
    for cfg in (m, k):
        back = snapshot.from_hf_config(snapshot.to_hf_config(cfg))
        assert back.num_experts == cfg.num_experts and back.num_heads == cfg.num_heads and back.attention == cfg.attention


def test_sliced_checkpoint_copy(tmp_path):
    """An expert rank's slice holds its experts only, the attention slice everything else; bytes are the source's."""
    import json as _json
    from cuteafd_b200 import tiny_moe
    from cuteafd_b200.cli import main
    from cuteafd_b200.loader.slice import slice_snapshot
    cfg = tiny_moe()
    src = snapshot.write_random_snapshot(cfg, str(tmp_path / "src"), fmt="fp8_block128", seed=2)
    full = Catalog(src)
    ex = slice_snapshot(src, str(tmp_path / "experts"), roles={"routed_expert"}, expert_range=(2, 5), shard_bytes=1 << 16)
    cat = Catalog(str(tmp_path / "experts"))
    names = cat.names()
    assert names and all(".mlp.experts." in n and 2 <= int(n.split(".mlp.experts.")[1].split(".")[0]) < 5 for n in names)
    assert any(n.endswith("weight_scale_inv") for n in names)                       # scales travel with their weights
    assert all(cat.sha256(n) == full.sha256(n) for n in names) and ex["tensors"] == len(names) and ex["bytes"] < ex["source_bytes"]
    assert len({e.file for e in cat.entries.values()}) > 1                          # sharded by the byte limit
    idx = _json.load(open(tmp_path / "experts" / "model.safetensors.index.json"))
    assert set(idx["weight_map"]) == set(names) and (tmp_path / "experts" / "config.json").exists()
    assert main(["plan", src, "--fetch", str(tmp_path / "attn"), "--exclude-role", "routed_expert"]) == 0
    attn = Catalog(str(tmp_path / "attn"))
    assert not any(".mlp.experts." in n for n in attn.names()) and "model.embed_tokens.weight" in attn
    assert set(attn.names()) | {n for n in full.names() if ".mlp.experts." in n} == set(full.names())
    assert _json.load(open(tmp_path / "attn" / "slice.json"))["exclude"] == ["routed_expert"]
    with pytest.raises(ValueError, match="matches no tensor"):
        slice_snapshot(src, str(tmp_path / "none"), roles={"routed_expert"}, expert_range=(100, 101))


def test_load_params_only_and_exclude_partition_the_checkpoint(tmp_path):
    from cuteafd_b200 import tiny_moe
    cfg = tiny_moe()
    src = snapshot.write_random_snapshot(cfg, str(tmp_path / "s"), fmt="fp8_block128", seed=6)
    _, everything = load.load_params(src)
    _, experts = load.load_params(src, only=".mlp.experts.")
    _, rest = load.load_params(src, exclude=".mlp.experts.")
    assert experts and all(".mlp.experts." in n for n in experts) and not any(".mlp.experts." in n for n in rest)
    assert set(experts) | set(rest) == set(everything) and not set(experts) & set(rest)
    assert not any(n.endswith("weight_scale_inv") for n in rest)            # an excluded operand's scales go with it


def test_config_mapping_refuses_what_it_cannot_serve():
    base = {"model_type": "qwen3_moe", "vocab_size": 1000, "num_hidden_layers": 4, "hidden_size": 256, "num_attention_heads": 2,
            "num_key_value_heads": 1, "head_dim": 128, "intermediate_size": 512, "moe_intermediate_size": 128, "num_experts": 8,
            "num_experts_per_tok": 2}
    assert snapshot.from_hf_config(dict(base, mlp_only_layers=[0, 1])).first_dense_layers == 2
    for bad, msg in ((dict(shared_expert_intermediate_size=512), "shared expert"), (dict(decoder_sparse_step=2), "interleaved"),
                     (dict(mlp_only_layers=[1, 3]), "first layers"), (dict(attention_bias=True), "biases"),
                     (dict(model_type="gpt_oss"), "unsupported model_type")):
        with pytest.raises(ValueError, match=msg):
            snapshot.from_hf_config(dict(base, **bad))


def test_load_params_keep_reads_one_expert_range(tmp_path):
    from cuteafd_b200 import tiny_moe
    from cuteafd_b200.ref.split import expert_range
    cfg = tiny_moe()
    src = snapshot.write_random_snapshot(cfg, str(tmp_path / "s"), fmt="fp8_block128", seed=8)
    lo, hi = expert_range(cfg.num_experts, 3, 1)
    _, got = load.load_params(src, keep=lambda pre: ".mlp.experts." in pre and lo <= int(pre.split(".mlp.experts.")[1].split(".")[0]) < hi)
    ids = {int(n.split(".mlp.experts.")[1].split(".")[0]) for n in got if ".mlp.experts." in n}
    assert ids == set(range(lo, hi)) and all(".mlp.experts." in n for n in got)
    _, everything = load.load_params(src)
    assert all(torch.equal(got[n], everything[n]) for n in got)


def test_glm4_moe_and_qwen2_configs_map_onto_the_gqa_engine(tmp_path):
    """glm4_moe (biased q / k / v, partial rotary, sigmoid routing with a correction bias, shared expert, MTP) and dense
    qwen2 (biased q / k / v) map onto the GQA geometry; a random snapshot round-trips; the oracle's partial rotary leaves
    the unrotated dims alone and matches a full rotation of the rotated slice."""
    import torch
    from cuteafd_b200.config import PRESETS
    from cuteafd_b200.loader import families, snapshot
    from cuteafd_b200.loader.load import open_snapshot
    from cuteafd_b200.ref import ops
    hf = {"model_type": "glm4_moe", "vocab_size": 151552, "hidden_size": 4096, "num_hidden_layers": 46, "num_attention_heads": 96,
          "num_key_value_heads": 8, "head_dim": 128, "partial_rotary_factor": 0.5, "attention_bias": True, "use_qk_norm": False,
          "rope_theta": 1000000, "rms_norm_eps": 1e-5, "intermediate_size": 10944, "moe_intermediate_size": 1408,
          "n_routed_experts": 128, "n_shared_experts": 1, "num_experts_per_tok": 8, "first_k_dense_replace": 1, "n_group": 1,
          "topk_group": 1, "routed_scaling_factor": 1.0, "norm_topk_prob": True, "num_nextn_predict_layers": 1}
    cfg = snapshot.from_hf_config(hf)
    want = PRESETS["glm-4.5-air"]()
    assert cfg.replace(name=want.name) == want
    assert families.detect(hf).id == "glm4_moe" and cfg.rope_dim == 64
    q2 = snapshot.from_hf_config({"model_type": "qwen2", "vocab_size": 1000, "hidden_size": 512, "num_hidden_layers": 2,
                                  "num_attention_heads": 4, "num_key_value_heads": 2, "intermediate_size": 1024})
    assert q2.family == "qwen2" and q2.attention_bias and q2.num_experts == 0 and families.detect({"model_type": "qwen2"}).id == "qwen2"
    import pytest
    with pytest.raises(ValueError):
        snapshot.from_hf_config(dict(hf, partial_rotary_factor=0.25))
    small = want.replace(vocab_size=512, num_layers=2, hidden=256, num_heads=4, num_kv_heads=2, dense_ffn=512, num_experts=8,
                         expert_ffn=128, top_k=2, mtp_layers=0)
    path = snapshot.write_random_snapshot(small, str(tmp_path / "glm"), fmt="bf16", seed=1)
    snap = open_snapshot(path)
    assert snap.cfg == small and snap.family.id == "glm4_moe" and snap.hints() == []
    assert any(n.endswith("self_attn.q_proj.bias") for n in snap.catalog.entries)
    # partial rotary in the oracle
    x = torch.randn(5, 3, 128).to(torch.bfloat16)
    pos = torch.arange(10, 15)
    inv = ops.rope_inv_freq(small, 64)
    for inter in (False, True):
        y = ops.apply_rope(x, pos, small.rope_theta, inter, inv)
        assert torch.equal(y[..., 64:], x[..., 64:])
        assert torch.equal(y[..., :64], ops.apply_rope(x[..., :64].contiguous(), pos, small.rope_theta, inter, inv))


def test_sliding_window_fields_map_per_layer():
    """A bare ``sliding_window`` windows every layer (Mistral); the Qwen form windows the layers from ``max_window_layers``
    on and only with ``use_sliding_window``; ``layer_types`` names them one by one and survives a config round trip."""
    from cuteafd_b200.loader.snapshot import from_hf_config, to_hf_config
    base = {"vocab_size": 1000, "hidden_size": 512, "num_hidden_layers": 4, "num_attention_heads": 4, "num_key_value_heads": 2,
            "head_dim": 128, "intermediate_size": 1024, "sliding_window": 256}
    c = from_hf_config(dict(base, model_type="mistral"))
    assert [c.window_of(i) for i in range(4)] == [256] * 4 and c.window_layers == ()
    c = from_hf_config(dict(base, model_type="qwen3"))
    assert c.sliding_window == 0
    c = from_hf_config(dict(base, model_type="qwen3", use_sliding_window=True, max_window_layers=3))
    assert [c.window_of(i) for i in range(4)] == [0, 0, 0, 256]
    c = from_hf_config(dict(base, model_type="llama", layer_types=["sliding_attention", "full_attention"] * 2))
    assert [c.window_of(i) for i in range(4)] == [256, 0, 256, 0]
    assert from_hf_config(to_hf_config(c)).window_layers == (1, 0, 1, 0)
    with pytest.raises(ValueError):
        from_hf_config(dict(base, model_type="llama", layer_types=["chunked_attention"] * 4))


def test_host_layout_lists_and_copies_each_hosts_share(tmp_path, capsys):
    """A host that runs an attention rank and an expert rank holds the union once; a dry run copies nothing; a second
    fetch of the same selection is skipped; the experts of two hosts partition the routed experts."""
    import json as _json
    from cuteafd_b200 import tiny_moe
    from cuteafd_b200.cli import main
    from cuteafd_b200.loader.safetensors_io import Catalog
    from cuteafd_b200.loader import slice as SL
    cfg = tiny_moe()
    src = snapshot.write_random_snapshot(cfg, str(tmp_path / "src"), fmt="bf16", seed=4)
    half = cfg.num_experts // 2
    lay = tmp_path / "layout.json"
    lay.write_text(_json.dumps({"front": ["attention", f"experts:0:{half}"], "back": [f"experts:{half}:{cfg.num_experts}"]}))
    assert main(["plan", src, "--file-layout", str(lay), "--files"]) == 0
    listed = _json.loads(capsys.readouterr().out)
    full = Catalog(src)
    assert set(listed) == {"front", "back"} and listed["front"]["bytes"] + listed["back"]["bytes"] == full.total_bytes()
    assert main(["plan", src, "--file-layout", str(lay), "--fetch", str(tmp_path / "dry"), "--dry-run"]) == 0
    assert _json.loads(capsys.readouterr().out) == listed and not (tmp_path / "dry").exists()
    assert main(["plan", src, "--file-layout", str(lay), "--fetch", str(tmp_path / "out")]) == 0
    capsys.readouterr()
    front, back = Catalog(str(tmp_path / "out" / "front")), Catalog(str(tmp_path / "out" / "back"))
    assert set(front.names()) | set(back.names()) == set(full.names()) and not set(front.names()) & set(back.names())
    assert all(".mlp.experts." in n for n in back.names()) and "model.embed_tokens.weight" in front
    for n in list(back.names())[:3] + list(front.names())[:3]:
        assert torch.equal((back if n in back else front).read(n).view(torch.uint8), full.read(n).view(torch.uint8))
    assert main(["plan", src, "--file-layout", str(lay), "--host", "back", "--fetch", str(tmp_path / "out" / "back")]) == 0
    assert _json.loads(capsys.readouterr().out)["back"]["skipped"] is True             # same selection already there
    assert main(["plan", src, "--file-layout", str(lay), "--host", "back", "--fetch", str(tmp_path / "out" / "back"), "--force"]) == 0
    assert "skipped" not in _json.loads(capsys.readouterr().out)["back"]
    assert main(["plan", src, "--file-layout", str(lay), "--host", "nowhere", "--files"]) == 2
    for bad in ({}, {"h": []}, {"h": "attention"}):
        lay.write_text(_json.dumps(bad))
        with pytest.raises(ValueError, match="host layout"):
            SL.read_layout(str(lay))
    with pytest.raises(ValueError, match="first:end"):
        SL.parse_share("experts:3")
    with pytest.raises(ValueError, match="empty expert range"):
        SL.parse_share("experts:5:5")
