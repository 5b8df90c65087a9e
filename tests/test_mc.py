"""Multi-core repositories: discovery, verified view selection, the catalog restricted to a view's index, the
publication check, and the fail-closed rules."""
import hashlib
import json
import os
import shutil

import pytest
import torch

from cuteafd_b200 import tiny_moe
from cuteafd_b200.loader import load, mc, snapshot
from cuteafd_b200.loader.safetensors_io import Catalog, write_file


def make_repo(tmp_path, seed=3):
    """An MC repository from a random bf16 snapshot: the ``original`` view is the snapshot's own index; the ``k8-compact``
    view replaces every attention o-projection by a stand-in tensor of another shape stored under the same name in its
    own shard (what matters here is which bytes each view's index names, not the trellis coding)."""
    cfg = tiny_moe()
    d = snapshot.write_random_snapshot(cfg, str(tmp_path / "repo"), fmt="bf16", seed=seed)
    with open(os.path.join(d, "model.safetensors.index.json")) as f:
        index = json.load(f)
    core = sorted(n for n in index["weight_map"] if n.endswith("self_attn.o_proj.weight"))
    assert core
    full = Catalog(d)
    compact = {n: (full.read(n).float() * 0.5).to(torch.bfloat16)[:, : full.read(n).shape[1] // 2].contiguous() for n in core}
    write_file(os.path.join(d, "core-k8.safetensors"), compact, {"format": "pt"})
    k8 = {"metadata": index.get("metadata", {}), "weight_map": dict(index["weight_map"], **{n: "core-k8.safetensors" for n in core})}
    with open(os.path.join(d, "model.k8.safetensors.index.json"), "w") as f:
        json.dump(k8, f)
    shutil.copy(os.path.join(d, "config.json"), os.path.join(d, "config.k8.json"))
    for fn in ("quantize_config.json", "quantize_config.k8.json"):
        with open(os.path.join(d, fn), "w") as f:
            json.dump({"bits": 16 if fn == "quantize_config.json" else 8}, f)
    variants = {"original": {"index": "model.safetensors.index.json", "config": "config.json", "quantize": "quantize_config.json", "core_tensors": core},
                "k8-compact": {"index": "model.k8.safetensors.index.json", "config": "config.k8.json", "quantize": "quantize_config.k8.json",
                               "core_tensors": core}}
    mc.publish(d, variants, source={"repo": "org/source", "revision": "abc"})
    return d, core, full


def test_views_select_their_own_bytes(tmp_path, monkeypatch):
    d, core, full = make_repo(tmp_path)
    info = mc.validate(d)
    assert set(info["views"]) == {"original", "k8-compact"} and info["views"]["k8-compact"]["core_bits"] == 8
    m = mc.discover(d)
    orig, k8 = mc.select(m, "original"), mc.select(m, "k8-compact")
    assert orig.view.fingerprint != k8.view.fingerprint and orig.identity != k8.identity and not orig.convert_fp8
    fp8 = mc.select(m, "fp8-compact")
    assert fp8.convert_fp8 and fp8.view.name == "original" and fp8.identity != orig.identity
    assert fp8.settings()["core-fp8-recipe"] == mc.FP8_RECIPE and orig.settings()["core-fp8-recipe"] is None
    # the loader: default view is the original; the compact view reads the stand-in core from its own shard and the
    # shared tensors from the same files; the other view's bytes are not part of the catalog
    a = load.open_snapshot(d)
    b = load.open_snapshot(d, core_view="k8-compact")
    n = core[0]
    assert a.view.name == "original" and b.view.name == "k8-compact"
    assert torch.equal(a.catalog.read(n), full.read(n)) and b.catalog.read(n).shape[1] * 2 == full.read(n).shape[1]
    assert os.path.basename(b.catalog.entries[n].file) == "core-k8.safetensors"
    shared = [x for x in a.catalog.names() if x not in core]
    assert set(a.catalog.names()) == set(b.catalog.names()) and all(a.catalog.entries[x].file == b.catalog.entries[x].file for x in shared)
    monkeypatch.setenv("CUTEAFD_CORE_VIEW", "k8-compact")                       # what serve --core-view sets
    assert load.open_snapshot(d).view.name == "k8-compact"
    monkeypatch.delenv("CUTEAFD_CORE_VIEW")
    # a plain checkpoint has only its own core
    plain = snapshot.write_random_snapshot(tiny_moe(), str(tmp_path / "plain"), fmt="bf16", seed=1)
    assert load.open_snapshot(plain).view is None
    with pytest.raises(mc.McError, match="needs an MC checkpoint"):
        load.open_snapshot(plain, core_view="fp8-compact")
    with pytest.raises(mc.McError, match="has no k6-compact view"):
        load.open_snapshot(d, core_view="k6-compact")
    with pytest.raises(mc.McError, match="unknown core view"):
        load.open_snapshot(d, core_view="k4")


def test_plan_reports_the_view(tmp_path, capsys):
    from cuteafd_b200.cli import main
    d, core, _ = make_repo(tmp_path)
    assert main(["plan", d, "--core-view", "fp8-compact"]) == 0
    out = capsys.readouterr().out
    assert "core view  fp8-compact" in out and mc.FP8_RECIPE in out
    os.environ.pop("CUTEAFD_CORE_VIEW", None)
    assert main(["plan", d, "--json"]) == 0
    assert json.loads(capsys.readouterr().out)["core_view"]["core-view"] == "original"


def edit(d, fn):
    path = os.path.join(d, mc.DISCOVERY)
    with open(path) as f:
        doc = json.load(f)
    fn(doc)
    with open(path, "w") as f:
        json.dump(doc, f)


def test_fail_closed(tmp_path):
    d, core, _ = make_repo(tmp_path)
    keep = open(os.path.join(d, mc.DISCOVERY)).read()

    def restore():
        with open(os.path.join(d, mc.DISCOVERY), "w") as f:
            f.write(keep)
    cases = [
        (lambda doc: doc.update(schema="cuteafd-mc-v2"), "unknown MC schema"),
        (lambda doc: doc.update(required_features=["sparse-core"]), "requires features"),
        (lambda doc: doc.update(original_core_dtype="F8_E4M3"), "not MC"),
        (lambda doc: doc["variants"].append(dict(doc["variants"][0])), "listed twice"),
        (lambda doc: doc["variants"][1].update(name="k4-compact"), "unknown variant"),
        (lambda doc: doc["variants"][1].update(core_bits=6), "core_bits must be 8"),
        (lambda doc: doc["variants"][1].update(index="../model.k8.safetensors.index.json"), "unsafe"),
        (lambda doc: doc["variants"][0].update(core_tensors=list(reversed(doc["variants"][0]["core_tensors"])) * 1 + ["a"]), "unique and sorted"),
        (lambda doc: doc["variants"][0].update(core_tensors=[]), "non-empty"),
        (lambda doc: doc.update(variants=doc["variants"][:1]), "at least one compact view"),
        (lambda doc: doc.update(shared_inventory_sha256="xyz"), "not a SHA-256"),
    ]
    for change, msg in cases:
        edit(d, change)
        with pytest.raises(mc.McError, match=msg):
            mc.discover(d)
        restore()
    # checks that need the view's files
    edit(d, lambda doc: doc["variants"][1].update(fingerprint="0" * 64))
    with pytest.raises(mc.McError, match="fingerprint mismatch"):
        mc.select(mc.discover(d), "k8-compact")
    assert mc.select(mc.discover(d), "original") is not None                   # the other view is untouched
    restore()
    edit(d, lambda doc: doc.update(shared_inventory_sha256=hashlib.sha256(b"other").hexdigest()))
    with pytest.raises(mc.McError, match="shared inventory"):
        mc.select(mc.discover(d), "original")
    restore()
    with open(os.path.join(d, "config.k8.json"), "a") as f:                    # one byte of metadata changes the view
        f.write("\n")
    with pytest.raises(mc.McError, match="does not match its recorded hash"):
        mc.select(mc.discover(d), "k8-compact")
    assert mc.select(mc.discover(d), "fp8-compact").view.name == "original"
    with pytest.raises(mc.McError):
        mc.validate(d)
    # unknown fields are ignored by readers
    shutil.copy(os.path.join(d, "config.json"), os.path.join(d, "config.k8.json"))
    edit(d, lambda doc: (doc.update(advisory={"note": 1}), doc["variants"][0].update(comment="x")))
    assert mc.validate(d)["schema"] == mc.SCHEMA
    # an index that names a tensor its shard does not hold
    with open(os.path.join(d, "model.k8.safetensors.index.json")) as f:
        idx = json.load(f)
    moved = next(n for n in idx["weight_map"] if n not in core)
    idx["weight_map"][moved] = "core-k8.safetensors"
    with pytest.raises(ValueError, match="does not hold it"):
        Catalog(d, weight_map=idx["weight_map"])
    # publishing refuses views whose shared tensors differ
    with open(os.path.join(d, "model.k8.safetensors.index.json"), "w") as f:
        json.dump(idx, f)
    with pytest.raises(mc.McError, match="does not share"):
        mc.publish(d, {"original": {"index": "model.safetensors.index.json", "config": "config.json", "quantize": "quantize_config.json", "core_tensors": core},
                       "k8-compact": {"index": "model.k8.safetensors.index.json", "config": "config.k8.json",
                                      "quantize": "quantize_config.k8.json", "core_tensors": core}})
