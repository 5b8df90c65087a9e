"""Sliced checkpoint copy: write only the tensors some ranks need into a new snapshot directory, byte for byte.

    slice_snapshot(src, dst, roles={"routed_expert"}, expert_range=(64, 128))     # an expert rank's share
    slice_snapshot(src, dst, exclude={"routed_expert"})                           # the attention ranks' share

A 600 GB checkpoint does not have to be copied to every host of a deployment: an expert host needs its expert range,
the attention hosts everything but the routed experts.  Tensors are copied as stored (no decode: scales, packed words
and global scales travel with their weight because they share its name prefix and therefore its role), into shards of
bounded size with a fresh ``model.safetensors.index.json``; config, tokenizer and the other side files are copied
whole.  ``slice.json`` records what was kept, so a loader can tell a slice from a damaged download.

Counterpart: ``cuteafd plan --files / --fetch`` (rust/crates/cuteafd-daemon/src/commands/plan.rs, docs/
sliced-checkpoints.md:1-47: role-only slices of a checkpoint).
"""
from __future__ import annotations

import json
import os
import shutil

from . import families, snapshot
from .safetensors_io import Catalog, write_file


def _plain(selectors: list[dict] | None):
    """Selectors as JSON (sets and tuples become sorted lists)."""
    if selectors is None:
        return None
    return [{k: sorted(v) if isinstance(v, set) else list(v) for k, v in sel.items()} for sel in selectors]


def select(cat: Catalog, model, roles: set[str] | None = None, exclude: set[str] | None = None,
           expert_range: tuple[int, int] | None = None, layers: tuple[int, int] | None = None) -> list[str]:
    """Tensor names (as stored) that belong to the slice."""
    keep = []
    for name in cat.names():
        role, layer, expert = model.classify(families.canonical_name(name))
        if roles is not None and role not in roles:
            continue
        if exclude and role in exclude:
            continue
        if expert_range is not None and role == "routed_expert" and not (expert_range[0] <= expert < expert_range[1]):
            continue
        if layers is not None and layer is not None and not (layers[0] <= layer < layers[1]):
            continue
        keep.append(name)
    return keep


def parse_share(text: str) -> dict:
    """One entry of a host layout -> selector keywords of ``select``.

    ``attention``: everything but the routed experts (what an attention rank or a tensor-parallel rank reads);
    ``experts:lo:hi``: the routed experts [lo, hi) and nothing else (an expert rank's share); ``all``: the whole
    checkpoint; any other word: the tensors of that role (``head``, ``embedding``, ``vision``, ...)."""
    if text == "all":
        return {}
    if text == "attention":
        return {"exclude": {"routed_expert"}}
    if text.startswith("experts:"):
        try:
            _, lo, hi = text.split(":")
            lo, hi = int(lo), int(hi)
        except ValueError as e:
            raise ValueError(f"share {text!r}: write experts:first:end") from e
        if not 0 <= lo < hi:
            raise ValueError(f"share {text!r}: empty expert range")
        return {"roles": {"routed_expert"}, "expert_range": (lo, hi)}
    return {"roles": {text}}


def read_layout(path: str) -> dict[str, list[dict]]:
    """A host layout file: JSON ``{"host": ["attention", "experts:0:64", ...], ...}`` -> selectors per host."""
    with open(path) as f:
        doc = json.load(f)
    if not isinstance(doc, dict) or not doc or not all(isinstance(v, list) and v and all(isinstance(x, str) for x in v) for v in doc.values()):
        raise ValueError("a host layout maps each host name to a non-empty list of shares")
    return {host: [parse_share(x) for x in shares] for host, shares in doc.items()}


def select_any(cat: Catalog, model, selectors: list[dict]) -> list[str]:
    """Union of several selections, in catalog order (a host that runs several ranks holds each tensor once)."""
    keep: set[str] = set()
    for sel in selectors:
        keep.update(select(cat, model, **sel))
    return [n for n in cat.names() if n in keep]


def inventory(src: str, selectors: list[dict]) -> dict:
    """What a slice would hold, without writing it: tensors, bytes and the source files they sit in."""
    src = snapshot.resolve(src)
    cfg, hf = snapshot.read_config(src)
    fam = families.detect(hf)
    if fam is None:
        raise ValueError("no family recognises this checkpoint")
    cat = Catalog(src)
    try:
        names = select_any(cat, fam.open(cfg, hf), selectors)
        return {"tensors": len(names), "bytes": sum(cat.entries[n].nbytes for n in names), "source_bytes": cat.total_bytes(),
                "files": sorted({os.path.basename(cat.entries[n].file) for n in names})}
    finally:
        cat.close()


def slice_snapshot(src: str, dst: str, roles: set[str] | None = None, exclude: set[str] | None = None,
                   expert_range: tuple[int, int] | None = None, layers: tuple[int, int] | None = None,
                   shard_bytes: int = 4 << 30, selectors: list[dict] | None = None, force: bool = False) -> dict:
    """``selectors`` (a host's shares, see ``read_layout``) replace the single selection of the other arguments.  A
    destination that already holds this very selection of this source is left alone unless ``force``."""
    src = snapshot.resolve(src)
    cfg, hf = snapshot.read_config(src)
    fam = families.detect(hf)
    if fam is None:
        raise ValueError("no family recognises this checkpoint")
    model = fam.open(cfg, hf)
    cat = Catalog(src)
    names = select_any(cat, model, selectors) if selectors is not None else select(cat, model, roles, exclude, expert_range, layers)
    if not names:
        raise ValueError("the selection matches no tensor")
    want = {"source": src, "roles": sorted(roles) if roles else None, "exclude": sorted(exclude) if exclude else None,
            "expert_range": list(expert_range) if expert_range else None, "layers": list(layers) if layers else None,
            "shares": _plain(selectors), "tensors": len(names), "bytes": sum(cat.entries[n].nbytes for n in names),
            "source_bytes": cat.total_bytes()}
    have = os.path.join(dst, "slice.json")
    if not force and os.path.isfile(have):
        with open(have) as f:
            old = json.load(f)
        if all(old.get(k) == v for k, v in want.items()) and os.path.isfile(os.path.join(dst, "model.safetensors.index.json")):
            cat.close()
            return dict(old, skipped=True)
    os.makedirs(dst, exist_ok=True)
    # file order of the source keeps the reads sequential
    names.sort(key=lambda n: (cat.entries[n].file, cat.entries[n].begin))
    weight_map: dict[str, str] = {}
    cur: dict = {}
    size = total = shard = 0

    def flush() -> None:
        nonlocal cur, size, shard
        if not cur:
            return
        fn = f"slice-{shard:05d}.safetensors"
        write_file(os.path.join(dst, fn), cur, {"format": "pt"})
        for n in cur:
            weight_map[n] = fn
        cur, size, shard = {}, 0, shard + 1
    for n in names:
        e = cat.entries[n]
        if cur and size + e.nbytes > shard_bytes:
            flush()
        cur[n] = cat.read(n)
        size += e.nbytes
        total += e.nbytes
    flush()
    with open(os.path.join(dst, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f, indent=1, sort_keys=True)
    for side in os.listdir(src):
        p = os.path.join(src, side)
        if os.path.isfile(p) and not side.endswith(".safetensors") and side != "model.safetensors.index.json":
            shutil.copy(p, os.path.join(dst, side))
    info = want
    assert total == want["bytes"]
    with open(os.path.join(dst, "slice.json"), "w") as f:
        json.dump(info, f, indent=1)
    cat.close()
    return info
