"""Layer-major oracle run: every window through layer 0, then every window through layer 1, and so on, with one
layer's weights resident at a time and the activations on disk between layers.

This is how reference activations of a checkpoint far larger than the host's memory are made: the peak is one layer's
parameters plus one window's activations, whatever the depth.  The run is resumable: each layer's output is written to
a temporary file and renamed, then ``latest.json`` is replaced the same way, so a run that dies between layers starts
again after the last layer it finished and produces the same bytes.  A directory made for other tokens or another
snapshot is refused, not continued.

Files: ``tokens.bin`` int32 [W, L]; ``layerNN.bin`` fp32 [W, L, hidden] (the residual stream after layer NN);
``logits.bin`` fp32 [W, L, vocab]; ``manifest.json`` (shapes, model name, digest); ``latest.json`` (layers done).

Counterpart: python/reference/layer_major.py:1-22 (one layer resident at a time, atomic ``latest.json`` resume) and the
tokens.bin / layerNN.bin / logits.bin dumps its golden runner compares against.
"""
from __future__ import annotations

import hashlib
import json
import os

import numpy as np
import torch

from .model import KvState, RefDecoder


def _atomic_write(path: str, data: bytes) -> None:
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(data)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)


def _save(path: str, t: torch.Tensor) -> None:
    _atomic_write(path, t.detach().cpu().contiguous().numpy().tobytes())


def _load(path: str, dtype, shape) -> torch.Tensor:
    return torch.from_numpy(np.fromfile(path, dtype=dtype).reshape(shape).copy())


def layer_params(snapshot: str, prefix: str) -> dict[str, torch.Tensor]:
    """The decoded parameters whose names contain ``prefix`` (one layer, the embedding, the final norm and head)."""
    from ..loader.load import load_params
    return load_params(snapshot, only=prefix)[1]


def run(snapshot: str, tokens: torch.Tensor, out_dir: str, after_layer=None, log=None) -> dict:
    """``tokens`` int64 [W, L]: W independent windows, each from position 0.  ``after_layer(i)`` is called once layer i is on
    disk (tests interrupt the run there).  Returns the manifest."""
    from ..loader.load import open_snapshot
    cfg = open_snapshot(snapshot).cfg
    W, L = tokens.shape
    os.makedirs(out_dir, exist_ok=True)
    digest = hashlib.sha256(tokens.to(torch.int32).numpy().tobytes() + json.dumps([cfg.name, cfg.num_layers, cfg.hidden, W, L]).encode()
                            ).hexdigest()[:16]
    manifest = {"model": cfg.name, "windows": W, "seq": L, "hidden": cfg.hidden, "vocab": cfg.vocab_size, "layers": cfg.num_layers,
                "digest": digest}
    latest_path = os.path.join(out_dir, "latest.json")
    done = -1                                         # index of the last finished layer; -1 = embedding not written yet
    if os.path.exists(latest_path):
        with open(latest_path) as f:
            latest = json.load(f)
        if latest.get("digest") != digest:
            raise ValueError(f"{out_dir} holds a run over other tokens or another checkpoint ({latest.get('digest')} != {digest})")
        done = int(latest["layer"])
    say = log or (lambda *_: None)

    def mark(layer: int) -> None:
        _atomic_write(latest_path, json.dumps({"layer": layer, "digest": digest}).encode())

    def act_path(layer: int) -> str:
        return os.path.join(out_dir, f"layer{layer:02d}.bin" if layer >= 0 else "embedding.bin")

    with torch.no_grad():
        if done < 0 and not os.path.exists(act_path(-1)):
            _save(os.path.join(out_dir, "tokens.bin"), tokens.to(torch.int32))
            table = layer_params(snapshot, "model.embed_tokens")["model.embed_tokens.weight"]
            _save(act_path(-1), table[tokens].float())
            del table
            _atomic_write(os.path.join(out_dir, "manifest.json"), json.dumps(manifest, indent=1).encode())
        positions = torch.arange(L)
        for i in range(max(done + 1, 0), cfg.num_layers):
            say(f"layer {i}")
            dec = RefDecoder(cfg, layer_params(snapshot, f"model.layers.{i}."))
            h_in = _load(act_path(i - 1), np.float32, (W, L, cfg.hidden))
            out = torch.empty_like(h_in)
            for w in range(W):
                out[w] = dec.layer(i, h_in[w], positions, KvState(cfg)).float()
            _save(act_path(i), out)
            mark(i)
            del dec
            if after_layer is not None:
                after_layer(i)
        if not os.path.exists(os.path.join(out_dir, "logits.bin")) or done < cfg.num_layers:
            say("head")
            p = layer_params(snapshot, "model.norm")
            p.update(layer_params(snapshot, "model.embed_tokens" if cfg.tie_embeddings else "lm_head"))
            dec = RefDecoder(cfg, p)
            h = _load(act_path(cfg.num_layers - 1), np.float32, (W, L, cfg.hidden))
            _save(os.path.join(out_dir, "logits.bin"), torch.stack([dec.head(h[w]) for w in range(W)]).float())
            mark(cfg.num_layers)
    return manifest


def read(out_dir: str) -> dict:
    """The finished run as tensors: {"tokens", "layers": [per-layer residuals], "logits", "manifest"}."""
    with open(os.path.join(out_dir, "manifest.json")) as f:
        m = json.load(f)
    with open(os.path.join(out_dir, "latest.json")) as f:
        if json.load(f)["layer"] != m["layers"]:
            raise ValueError(f"{out_dir}: the run has not finished")
    W, L, H, V = m["windows"], m["seq"], m["hidden"], m["vocab"]
    return {"manifest": m, "tokens": _load(os.path.join(out_dir, "tokens.bin"), np.int32, (W, L)).long(),
            "layers": [_load(os.path.join(out_dir, f"layer{i:02d}.bin"), np.float32, (W, L, H)) for i in range(m["layers"])],
            "logits": _load(os.path.join(out_dir, "logits.bin"), np.float32, (W, L, V))}
