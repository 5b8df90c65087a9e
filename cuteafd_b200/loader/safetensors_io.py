"""Minimal safetensors reader / writer: header catalog, zero-copy tensor and row-window reads.

The on-disk format is an 8-byte little-endian header length, a JSON header
(name -> dtype, shape, data_offsets), then raw little-endian tensor bytes.  The catalog reads only
headers, so planning a 600 GB checkpoint touches a few megabytes; tensor reads map the file and
slice.  Counterpart: rust/crates/cuteafd-loader/src/catalog.rs, tensors.rs:1-60 (header catalog,
tensor / row-window reads with sha256).
"""
from __future__ import annotations

import hashlib
import json
import mmap
import os
import struct
from dataclasses import dataclass

import warnings

import torch


def _view(buf, nbytes: int, offset: int) -> torch.Tensor:
    """Bytes of a read-only file mapping as a uint8 tensor (no copy).  Every caller converts or copies what it reads and
    nothing writes through the view, so torch's warning about a non-writable buffer says nothing new here."""
    with warnings.catch_warnings():
        warnings.filterwarnings("ignore", message="The given buffer is not writable")
        return torch.frombuffer(buf, dtype=torch.uint8, count=nbytes, offset=offset)

DTYPES = {
    "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "F8_E4M3": (torch.float8_e4m3fn, 1), "F8_E5M2": (torch.float8_e5m2, 1),
    "U8": (torch.uint8, 1), "I8": (torch.int8, 1), "I16": (torch.int16, 2), "I32": (torch.int32, 4),
    "I64": (torch.int64, 8), "F64": (torch.float64, 8), "BOOL": (torch.bool, 1),
}
NAMES = {v[0]: k for k, v in DTYPES.items()}


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str
    shape: tuple[int, ...]
    file: str
    begin: int          # byte offset inside the file (absolute)
    end: int

    @property
    def nbytes(self) -> int:
        return self.end - self.begin

    @property
    def numel(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n


def read_header(path: str) -> tuple[dict, int]:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        if n > 512 << 20:
            raise ValueError(f"{path}: implausible header length {n}")
        header = json.loads(f.read(n))
    return header, 8 + n


class Catalog:
    """Every tensor of a snapshot directory by name (headers only)."""

    def __init__(self, directory: str, rename=None, weight_map: dict[str, str] | None = None):
        """``rename(name) -> name`` maps a checkpoint's tensor names onto the canonical ones the loaders use (families
        whose files say ``block_sparse_moe.experts.3.w1`` for ``mlp.experts.3.gate_proj``); nothing is rewritten.
        ``weight_map`` (tensor name -> shard, an index file's) restricts the catalog to one view of a repository that
        holds several: only the named tensors belong, only the shards they sit in are opened, and a named tensor that
        its shard does not hold is an error."""
        self.directory = directory
        self.entries: dict[str, TensorEntry] = {}
        self.metadata: dict[str, dict] = {}
        files = sorted(f for f in os.listdir(directory) if f.endswith(".safetensors"))
        if weight_map is not None:
            files = sorted(set(weight_map.values()))
        if not files:
            raise FileNotFoundError(f"no .safetensors files under {directory}")
        for fn in files:
            path = os.path.join(directory, fn)
            header, base = read_header(path)
            self.metadata[fn] = header.pop("__metadata__", {})
            for name, info in header.items():
                if weight_map is not None and weight_map.get(name) != fn:
                    continue                                  # another view's bytes in a shared shard
                b, e = info["data_offsets"]
                if info["dtype"] not in DTYPES:
                    raise ValueError(f"{fn}:{name}: unsupported dtype {info['dtype']}")
                name = rename(name) if rename else name
                self.entries[name] = TensorEntry(name, info["dtype"], tuple(info["shape"]), path, base + b, base + e)
        self._maps: dict[str, mmap.mmap] = {}
        if weight_map is not None:
            lost = [n for n in weight_map if (rename(n) if rename else n) not in self.entries]
            if lost:
                raise ValueError(f"the index names {lost[0]} in {weight_map[lost[0]]}, which does not hold it")

    def __contains__(self, name: str) -> bool:
        return name in self.entries

    def names(self) -> list[str]:
        return sorted(self.entries)

    def total_bytes(self) -> int:
        return sum(e.nbytes for e in self.entries.values())

    def _map(self, path: str) -> mmap.mmap:
        if path not in self._maps:
            with open(path, "rb") as f:
                self._maps[path] = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        return self._maps[path]

    def read(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        dt, size = DTYPES[e.dtype]
        buf = self._map(e.file)
        t = _view(buf, e.nbytes, e.begin)
        return t.view(dt).view(e.shape) if e.numel else torch.empty(e.shape, dtype=dt)

    def read_rows(self, name: str, first: int, count: int) -> torch.Tensor:
        """Rows [first, first+count) of a tensor's leading dimension, without touching the rest."""
        e = self.entries[name]
        dt, size = DTYPES[e.dtype]
        row = e.numel // e.shape[0] * size
        buf = self._map(e.file)
        t = _view(buf, row * count, e.begin + first * row)
        return t.view(dt).view((count, *e.shape[1:]))

    def sha256(self, name: str) -> str:
        e = self.entries[name]
        return hashlib.sha256(self._map(e.file)[e.begin:e.end]).hexdigest()

    def close(self) -> None:
        for m in self._maps.values():
            m.close()
        self._maps.clear()


def write_file(path: str, tensors: dict[str, torch.Tensor], metadata: dict[str, str] | None = None) -> None:
    header: dict = {}
    if metadata:
        header["__metadata__"] = metadata
    offset = 0
    blobs = []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in NAMES:
            raise ValueError(f"{name}: dtype {t.dtype} has no safetensors name")
        raw = t.view(torch.uint8).reshape(-1).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)
    os.replace(tmp, path)


def write_sharded(directory: str, tensors: dict[str, torch.Tensor], shard_bytes: int = 4 << 30) -> dict:
    """Write shards + model.safetensors.index.json in the Hugging Face snapshot layout."""
    os.makedirs(directory, exist_ok=True)
    shards: list[dict[str, torch.Tensor]] = [{}]
    size = 0
    for name in sorted(tensors):
        nb = tensors[name].numel() * tensors[name].element_size()
        if size and size + nb > shard_bytes:
            shards.append({})
            size = 0
        shards[-1][name] = tensors[name]
        size += nb
    weight_map = {}
    total = 0
    for i, sh in enumerate(shards):
        fn = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        write_file(os.path.join(directory, fn), sh, {"format": "pt"})
        for name, t in sh.items():
            weight_map[name] = fn
            total += t.numel() * t.element_size()
    index = {"metadata": {"total_size": total}, "weight_map": weight_map}
    with open(os.path.join(directory, "model.safetensors.index.json"), "w") as f:
        json.dump(index, f, indent=1, sort_keys=True)
    return index
