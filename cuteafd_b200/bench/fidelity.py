"""Fidelity against sealed windows: how far a model's next-token distributions are from a reference's, measured on
fixed token windows whose reference distributions were computed once and stored.

    cuteafd fidelity seal  <reference snapshot> windows.safetensors --windows 16 --seq 128 [--tokens text.txt]
    cuteafd fidelity check <test snapshot>      windows.safetensors          # KL, top-1 agreement per window and overall

A sealed file holds, per window, the token ids and, per position, the reference's top-``K`` token ids with their
log-probabilities and the log of the probability mass outside the top K.  Checking needs no reference model: the test
model's distribution is folded onto the same K + 1 outcomes (the K ids and "anything else") and

    KL(ref || test) = sum_k p_k (log p_k - log q_k) + p_rest (log p_rest - log q_rest)

is a lower bound of the full-vocabulary KL that is tight once K covers the mass (K = 64 covers > 0.999 on trained
models).  ``top1`` is the share of positions where the test model's arg-max equals the reference's.  The digest of the
tokens and the reference tensors is stored with them and verified on load, so a window file cannot be edited into
agreement.

This is the quantisation pipeline's acceptance check (a re-encoded snapshot against its bf16 source) and, with the
engine as the test model, the engine-vs-oracle check over more than one row.

Counterpart: the reference's fidelity panel and sealed fidelity windows (python/reference/ sealed windows; bench quick
quality: KL / top-1 against them).
"""
from __future__ import annotations

import hashlib
import json

import torch

from ..loader.safetensors_io import write_file

TOP_K = 64


def _digest(tensors: dict[str, torch.Tensor]) -> str:
    h = hashlib.sha256()
    for name in sorted(tensors):
        h.update(name.encode())
        h.update(tensors[name].contiguous().view(torch.uint8).numpy().tobytes())
    return h.hexdigest()


@torch.no_grad()
def logits_fn_for(cfg, params):
    """Window -> logits [L, vocab] through the oracle decoder (a fresh KV state per window)."""
    from ..ref.model import KvState, RefDecoder
    dec = RefDecoder(cfg, params)
    return lambda toks: dec.forward(toks, KvState(cfg))


@torch.no_grad()
def seal(logits_fn, windows: torch.Tensor, path: str, top_k: int = TOP_K, meta: dict | None = None) -> dict:
    """windows [W, L] int64.  Writes the sealed file, returns its metadata."""
    W, L = windows.shape
    ids = torch.empty(W, L, top_k, dtype=torch.int32)
    lps = torch.empty(W, L, top_k, dtype=torch.float32)
    rest = torch.empty(W, L, dtype=torch.float32)
    for w in range(W):
        lp = torch.log_softmax(logits_fn(windows[w]).float(), dim=-1)
        k = min(top_k, lp.shape[-1] - 1)
        v, i = lp.topk(k, dim=-1)
        ids[w, :, :k], lps[w, :, :k] = i.to(torch.int32), v
        if k < top_k:
            ids[w, :, k:], lps[w, :, k:] = -1, float("-inf")
        rest[w] = torch.log((1.0 - v.exp().sum(-1)).clamp_min(1e-12))
    tensors = {"tokens": windows.to(torch.int32), "top_ids": ids, "top_logprobs": lps, "rest_logprob": rest}
    info = dict(meta or {}, windows=W, seq=L, top_k=top_k, digest=_digest(tensors))
    write_file(path, tensors, {"format": "pt", "fidelity": json.dumps(info)})
    return info


def load_sealed(path: str) -> tuple[dict[str, torch.Tensor], dict]:
    """Reads one sealed file (by its own header, whatever else the directory holds) and verifies its digest."""
    from ..loader.safetensors_io import DTYPES, read_header
    header, base = read_header(path)
    info = json.loads((header.pop("__metadata__", {}) or {}).get("fidelity", "{}"))
    tensors = {}
    with open(path, "rb") as f:
        for name in ("tokens", "top_ids", "top_logprobs", "rest_logprob"):
            if name not in header:
                raise ValueError(f"{path}: not a sealed window file (no {name})")
            b, e = header[name]["data_offsets"]
            f.seek(base + b)
            raw = bytearray(f.read(e - b))
            tensors[name] = torch.frombuffer(raw, dtype=DTYPES[header[name]["dtype"]][0]).view(header[name]["shape"]).clone()
    if info.get("digest") != _digest(tensors):
        raise ValueError(f"{path}: sealed windows do not match their digest")
    return tensors, info


@torch.no_grad()
def check(logits_fn, sealed: dict[str, torch.Tensor]) -> dict:
    toks = sealed["tokens"].long()
    W, L = toks.shape
    kls, agree, worst = [], [], 0.0
    per_window = []
    for w in range(W):
        lq = torch.log_softmax(logits_fn(toks[w]).float(), dim=-1)                      # [L, V]
        ids, lp, lrest = sealed["top_ids"][w].long(), sealed["top_logprobs"][w], sealed["rest_logprob"][w]
        valid = ids >= 0
        q_top = lq.gather(1, ids.clamp_min(0))
        q_top = torch.where(valid, q_top, torch.full_like(q_top, float("-inf")))
        q_rest = torch.log((1.0 - q_top.exp().sum(-1)).clamp_min(1e-12))
        p = torch.where(valid, lp.exp(), torch.zeros_like(lp))
        kl = (p * (torch.where(valid, lp, torch.zeros_like(lp)) - torch.where(valid, q_top, torch.zeros_like(lp)))).sum(-1)
        kl = kl + lrest.exp() * (lrest - q_rest)
        kl = kl.clamp_min(0.0)
        top1 = (lq.argmax(-1) == ids[:, 0]).float()
        kls.append(kl)
        agree.append(top1)
        worst = max(worst, float(kl.max()))
        per_window.append({"kl": round(float(kl.mean()), 6), "top1": round(float(top1.mean()), 4)})
    kl_all, a_all = torch.cat(kls), torch.cat(agree)
    return {"windows": W, "positions": int(kl_all.numel()), "kl_mean": float(kl_all.mean()), "kl_p99": float(kl_all.quantile(0.99)),
            "kl_max": worst, "top1": float(a_all.mean()), "per_window": per_window}


def random_windows(vocab: int, windows: int, seq: int, seed: int = 0) -> torch.Tensor:
    return torch.randint(0, vocab, (windows, seq), generator=torch.Generator().manual_seed(seed))


def run_cli(a) -> int:
    from ..loader.load import load_params
    cfg, params = load_params(a.snapshot)
    fn = logits_fn_for(cfg, params)
    if a.action == "seal":
        if a.tokens:
            from ..quant.calibrate import token_batches
            from ..serve.tokenizer import load_tokenizer
            tok = load_tokenizer(a.snapshot, cfg.vocab_size)
            rows = [t for t in token_batches(a.tokens, tok, cfg.vocab_size, a.windows * a.seq, a.seq) if t.numel() == a.seq]
            if not rows:
                raise SystemExit("the text file holds fewer tokens than one window")
            wins = torch.stack(rows[: a.windows])
        else:
            wins = random_windows(cfg.vocab_size, a.windows, a.seq, a.seed)
        print(json.dumps(seal(fn, wins, a.file, meta={"model": cfg.name})))
        return 0
    sealed, info = load_sealed(a.file)
    rep = check(fn, sealed)
    rep["reference"] = info.get("model")
    ok = rep["kl_mean"] <= a.max_kl and rep["top1"] >= a.min_top1
    print(json.dumps(dict({k: v for k, v in rep.items() if k != "per_window"}, ok=ok)))
    return 0 if ok else 1
