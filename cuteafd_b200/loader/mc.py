"""Multi-core ("MC") checkpoints: one repository that holds the routed experts and the other shared tensors once and
several complete, mutually exclusive variants of the dense core, each behind its own index / config / quantisation
metadata.  A view is what its index names; bytes of other views that sit in shared shards are not part of it.

    m = discover(snapshot_dir)                 # None for a plain checkpoint
    v = select(m, "k8-compact")                # verified: metadata hashes, shared inventory, fingerprint
    v.index, v.config, v.core_tensors

Views: ``original`` (the source's own core, 16 bits), ``k8-compact`` / ``k6-compact`` (the core as 8- or 6-bit
trellis tensors), and ``fp8-compact``, which is not stored: it is the ``original`` view with its ``core_tensors``
encoded to E4M3 with 128 x 128 block scales when they are loaded (``FP8_RECIPE``).  A plain checkpoint has only its own
core and refuses every selector but ``original``.

``publish`` writes the discovery file for a directory whose variants' files are in place (what a quantisation run does
last); ``validate`` re-derives everything a reader checks, for all variants, plus the cross-view rules.

Counterpart: docs/mc-checkpoints.md:1-140 (views table, ``cuteafd-mc.json`` schema ``cuteafd-mc-v1``, shared inventory
digest over ``name NUL shard NL`` of the non-core entries, view fingerprint over the three metadata files, fail-closed
rules), rust/crates/cuteafd-daemon/src/cli.rs:349-380 (``--core-view``, the settings a card records).
"""
from __future__ import annotations

import hashlib
import json
import os
from dataclasses import dataclass, field

DISCOVERY = "cuteafd-mc.json"
SCHEMA = "cuteafd-mc-v1"
MAX_JSON_BYTES = 64 << 20
CORE_BITS = {"original": 16, "k8-compact": 8, "k6-compact": 6}
VIEWS = ("original", "k8-compact", "k6-compact", "fp8-compact")
FP8_RECIPE = "e4m3-block128-rne-amax448"            # row-major E4M3, fp32 scale per 128 x 128 block, scale = amax / 448
KNOWN_FEATURES: tuple[str, ...] = ()


class McError(ValueError):
    pass


@dataclass
class View:
    name: str
    index: str
    config: str
    quantize: str
    core_bits: int
    core_tensors: list[str]
    metadata_sha256: dict[str, str]
    fingerprint: str


@dataclass
class Manifest:
    directory: str
    source: dict
    original_core_dtype: str
    shared_inventory_sha256: str
    variants: dict[str, View] = field(default_factory=dict)
    raw_sha256: str = ""


@dataclass
class Selected:
    """A verified view.  ``convert_fp8``: the loader encodes ``core_tensors`` to E4M3 block-128 (the fp8-compact view)."""
    name: str
    view: View
    convert_fp8: bool
    identity: str                                   # discovery file + selector (+ recipe): what a card records

    def settings(self) -> dict:
        return {"core-view": self.name, "core-view-fingerprint": self.view.fingerprint,
                "core-fp8-recipe": FP8_RECIPE if self.convert_fp8 else None}


def _read_json(path: str) -> tuple[dict, bytes]:
    size = os.path.getsize(path)
    if size > MAX_JSON_BYTES:
        raise McError(f"{os.path.basename(path)} is {size} bytes, more than a metadata file may be")
    with open(path, "rb") as f:
        raw = f.read()
    try:
        doc = json.loads(raw)
    except json.JSONDecodeError as e:
        raise McError(f"{os.path.basename(path)}: {e}") from e
    if not isinstance(doc, dict):
        raise McError(f"{os.path.basename(path)} is not a JSON object")
    return doc, raw


def _safe(name) -> bool:
    return isinstance(name, str) and bool(name) and not any(c in name for c in "/\\\0\n") and name not in (".", "..")


def _hex(v) -> bool:
    return isinstance(v, str) and len(v) == 64 and all(c in "0123456789abcdef" for c in v)


def discover(directory: str) -> Manifest | None:
    """The manifest of an MC repository, structurally checked; None when ``cuteafd-mc.json`` is absent (a plain
    checkpoint).  Nothing but the discovery file is read."""
    path = os.path.join(directory, DISCOVERY)
    if not os.path.isfile(path):
        return None
    doc, raw = _read_json(path)
    if doc.get("schema") != SCHEMA:
        raise McError(f"unknown MC schema {doc.get('schema')!r}")
    need = doc.get("required_features", [])
    if not isinstance(need, list) or not all(isinstance(x, str) for x in need):
        raise McError("required_features must be a list of strings")
    missing = [x for x in need if x not in KNOWN_FEATURES]
    if missing:
        raise McError(f"the checkpoint requires features this loader does not have: {', '.join(missing)}")
    dtype = doc.get("original_core_dtype")
    if dtype not in ("BF16", "F32"):
        raise McError(f"original_core_dtype {dtype!r}: an MC source core is BF16 or F32 (an FP8-origin model is not MC)")
    if not _hex(doc.get("shared_inventory_sha256")):
        raise McError("shared_inventory_sha256 is not a SHA-256 digest")
    m = Manifest(directory, dict(doc.get("source") or {}), dtype, doc["shared_inventory_sha256"], raw_sha256=hashlib.sha256(raw).hexdigest())
    variants = doc.get("variants")
    if not isinstance(variants, list) or not variants:
        raise McError("the manifest lists no variants")
    for v in variants:
        if not isinstance(v, dict):
            raise McError("a variant is not an object")
        name = v.get("name")
        if name not in CORE_BITS:
            raise McError(f"unknown variant {name!r}")
        if name in m.variants:
            raise McError(f"variant {name} is listed twice")
        files = [v.get("index"), v.get("config"), v.get("quantize")]
        if not all(_safe(f) for f in files):
            raise McError(f"variant {name}: unsafe or missing file name")
        if v.get("core_bits") != CORE_BITS[name]:
            raise McError(f"variant {name}: core_bits must be {CORE_BITS[name]}")
        core = v.get("core_tensors")
        if not isinstance(core, list) or not core or not all(isinstance(t, str) and "\0" not in t and "\n" not in t for t in core):
            raise McError(f"variant {name}: core_tensors must be a non-empty list of tensor names")
        if core != sorted(set(core)):
            raise McError(f"variant {name}: core_tensors must be unique and sorted")
        sums = v.get("metadata_sha256")
        if not isinstance(sums, dict) or set(sums) != set(files) or not all(_hex(h) for h in sums.values()):
            raise McError(f"variant {name}: metadata_sha256 must name exactly its index, config and quantisation files")
        if not _hex(v.get("fingerprint")):
            raise McError(f"variant {name}: fingerprint is not a SHA-256 digest")
        m.variants[name] = View(name, files[0], files[1], files[2], CORE_BITS[name], core, dict(sums), v["fingerprint"])
    if "original" not in m.variants or len(m.variants) < 2:
        raise McError("an MC repository holds the original view and at least one compact view")
    return m


def shared_inventory_digest(weight_map: dict, core_tensors) -> str:
    """SHA-256 over the non-core entries sorted by tensor name: name, NUL, shard basename, newline."""
    core = set(core_tensors)
    h = hashlib.sha256()
    for name in sorted(weight_map):
        if name in core:
            continue
        shard = weight_map[name]
        if not _safe(shard) or "\0" in name or "\n" in name:
            raise McError(f"unsafe name in the index: {name!r} -> {shard!r}")
        h.update(name.encode() + b"\0" + shard.encode() + b"\n")
    return h.hexdigest()


def view_fingerprint(name: str, shared_digest: str, metadata_sha256: dict[str, str]) -> str:
    h = hashlib.sha256(f"cuteafd-mc-view-v1\0{name}\0{shared_digest}\0".encode())
    for fn in sorted(metadata_sha256):
        h.update(f"{fn}\0{metadata_sha256[fn]}\n".encode())
    return h.hexdigest()


def verify_view(m: Manifest, v: View) -> dict:
    """Everything a reader checks before it opens a shard of this view; returns the view's ``weight_map``."""
    for fn, want in v.metadata_sha256.items():
        path = os.path.join(m.directory, fn)
        if not os.path.isfile(path):
            raise McError(f"view {v.name}: {fn} is missing")
        if os.path.getsize(path) > MAX_JSON_BYTES:
            raise McError(f"view {v.name}: {fn} is larger than a metadata file may be")
        with open(path, "rb") as f:
            got = hashlib.sha256(f.read()).hexdigest()
        if got != want:
            raise McError(f"view {v.name}: {fn} does not match its recorded hash")
    index, _ = _read_json(os.path.join(m.directory, v.index))
    wm = index.get("weight_map")
    if not isinstance(wm, dict) or not wm:
        raise McError(f"view {v.name}: {v.index} has no weight_map")
    absent = [t for t in v.core_tensors if t not in wm]
    if absent:
        raise McError(f"view {v.name}: core tensor {absent[0]} is not in {v.index}")
    if shared_inventory_digest(wm, v.core_tensors) != m.shared_inventory_sha256:
        raise McError(f"view {v.name}: its shared tensors differ from the repository's shared inventory")
    if view_fingerprint(v.name, m.shared_inventory_sha256, v.metadata_sha256) != v.fingerprint:
        raise McError(f"view {v.name}: fingerprint mismatch")
    return wm


def select(m: Manifest | None, view: str = "original") -> Selected | None:
    """The verified view a deployment serves.  A plain checkpoint (``m`` None) has only its own core: ``original``
    selects nothing (None), anything else is refused."""
    if view not in VIEWS:
        raise McError(f"unknown core view {view!r} (choose from {', '.join(VIEWS)})")
    if m is None:
        if view != "original":
            raise McError(f"core view {view} needs an MC checkpoint ({DISCOVERY}); this one is plain")
        return None
    stored = "original" if view == "fp8-compact" else view
    if stored not in m.variants:
        raise McError(f"this repository has no {stored} view (it has {', '.join(sorted(m.variants))})")
    v = m.variants[stored]
    verify_view(m, v)
    h = hashlib.sha256(f"{m.raw_sha256}\0{view}\0".encode())
    if view == "fp8-compact":
        h.update(FP8_RECIPE.encode())
    return Selected(view, v, view == "fp8-compact", h.hexdigest())


def validate(directory: str) -> dict:
    """Publication check: every variant verifies, all views share one inventory (implied by the digest), the original
    index names no trellis core tensor and no view's core leaks into another's index."""
    m = discover(directory)
    if m is None:
        raise McError(f"{directory} has no {DISCOVERY}")
    maps = {name: verify_view(m, v) for name, v in m.variants.items()}
    trellis = (".trellis", ".suh", ".svh", ".mcg", ".mul1")
    for t in maps["original"]:
        if t.endswith(trellis) and any(t.startswith(c.rsplit(".", 1)[0] + ".") for c in m.variants["original"].core_tensors):
            raise McError(f"the original view names a trellis core tensor: {t}")
    for a, va in m.variants.items():
        for b, wb in maps.items():
            if a == b:
                continue
            own_b = set(m.variants[b].core_tensors)
            leaked = [t for t in va.core_tensors if t in wb and t not in own_b]
            if leaked:
                raise McError(f"core tensor {leaked[0]} of view {a} is indexed by view {b}")
    return {"schema": SCHEMA, "views": {n: {"core_bits": v.core_bits, "core_tensors": len(v.core_tensors), "fingerprint": v.fingerprint,
                                          "tensors": len(maps[n])} for n, v in m.variants.items()},
            "shared_inventory_sha256": m.shared_inventory_sha256}


def publish(directory: str, variants: dict[str, dict], source: dict | None = None, original_core_dtype: str = "BF16") -> dict:
    """Write ``cuteafd-mc.json`` for a directory whose views are in place.  ``variants``: name -> {"index", "config",
    "quantize", "core_tensors"}.  Hashes, the shared inventory digest and the fingerprints are computed here; views whose
    shared tensors differ are refused."""
    if "original" not in variants or len(variants) < 2 or any(n not in CORE_BITS for n in variants):
        raise McError("publish needs the original view and at least one of k8-compact / k6-compact")
    shared = None
    out = []
    for name in sorted(variants, key=list(CORE_BITS).index):
        spec = variants[name]
        files = [spec["index"], spec["config"], spec["quantize"]]
        if not all(_safe(f) for f in files):
            raise McError(f"variant {name}: unsafe file name")
        sums = {}
        for fn in files:
            with open(os.path.join(directory, fn), "rb") as f:
                sums[fn] = hashlib.sha256(f.read()).hexdigest()
        index, _ = _read_json(os.path.join(directory, spec["index"]))
        core = sorted(set(spec["core_tensors"]))
        digest = shared_inventory_digest(index.get("weight_map") or {}, core)
        if shared is None:
            shared = digest
        elif digest != shared:
            raise McError(f"view {name} does not share the original view's non-core tensors")
        out.append({"name": name, "index": files[0], "config": files[1], "quantize": files[2], "core_bits": CORE_BITS[name],
                    "core_tensors": core, "metadata_sha256": sums, "fingerprint": view_fingerprint(name, digest, sums)})
    doc = {"schema": SCHEMA, "required_features": [], "source": source or {}, "original_core_dtype": original_core_dtype,
           "shared_inventory_sha256": shared, "variants": out}
    tmp = os.path.join(directory, DISCOVERY + ".tmp")
    with open(tmp, "w") as f:
        json.dump(doc, f, indent=1, sort_keys=True)
    os.replace(tmp, os.path.join(directory, DISCOVERY))
    return doc
