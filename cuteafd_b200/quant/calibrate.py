"""Calibration run for Hessian-aware quantisation: stream token batches through the oracle decoder and accumulate,
for every projection, H = sum over its input rows of x x^T.

    python -m cuteafd_b200.cli calibrate <snapshot> <out dir> --tokens calib.txt --rows 2048

The decoder calls an observer before every projection with the operand's prefix (``model.layers.3.self_attn.o_proj``,
``model.layers.5.mlp.experts.17.down_proj``, ...) and the rows the projection is about to consume; routed experts see
only the rows routed to them, the down projection sees the rounded SwiGLU activation.  Accumulation is float64 on the
host; the result is written as ``<prefix>.hessian`` tensors (float32, normalised by the row count so that experts
with few rows keep a comparable scale) plus ``<prefix>.rows`` counts, in safetensors shards of bounded size, which is
the layout ``quantize --hessians`` reads.

Operands that saw fewer rows than their input width get a ridge toward the mean diagonal (their Hessian is rank
deficient); the quantiser's own damping adds to that.

Counterpart: the calibration pass of the reference's quantisation pipeline (quantization/*.py, which captures layer
inputs with forward hooks on the exported reference model).
"""
from __future__ import annotations

import os

import torch

from ..config import ModelConfig
from ..loader.safetensors_io import write_file
from ..ref.model import KvState, RefDecoder


class HessianCollector:
    """Observer for ``RefDecoder.observe``."""

    def __init__(self, keep=None):
        self.h: dict[str, torch.Tensor] = {}
        self.rows: dict[str, int] = {}
        self.keep = keep                      # optional predicate on the operand prefix

    def __call__(self, prefix: str, x: torch.Tensor) -> None:
        if self.keep is not None and not self.keep(prefix):
            return
        xd = x.reshape(-1, x.shape[-1]).double()
        if prefix not in self.h:
            self.h[prefix] = torch.zeros(xd.shape[1], xd.shape[1], dtype=torch.float64)
            self.rows[prefix] = 0
        self.h[prefix].addmm_(xd.T, xd)
        self.rows[prefix] += xd.shape[0]

    def result(self, ridge: float = 0.01) -> dict[str, torch.Tensor]:
        out: dict[str, torch.Tensor] = {}
        for pre, h in self.h.items():
            n = self.rows[pre]
            hn = h / max(n, 1)
            if n < h.shape[0]:
                hn = hn + ridge * hn.diagonal().mean().clamp_min(1e-12) * torch.eye(h.shape[0], dtype=torch.float64)
            out[pre + ".hessian"] = hn.float()
            out[pre + ".rows"] = torch.tensor([n], dtype=torch.int64)
        return out


@torch.no_grad()
def collect(cfg: ModelConfig, params: dict[str, torch.Tensor], batches, keep=None) -> HessianCollector:
    """``batches``: an iterable of 1-D token tensors (one sequence each)."""
    dec = RefDecoder(cfg, params)
    col = HessianCollector(keep)
    dec.observe = col
    for toks in batches:
        dec.hidden_states(torch.as_tensor(toks, dtype=torch.long), KvState(cfg))
    return col


def save(col: HessianCollector, out_dir: str, shard_bytes: int = 2 << 30) -> list[str]:
    os.makedirs(out_dir, exist_ok=True)
    tensors = col.result()
    files, cur, size = [], {}, 0
    for name in sorted(tensors):
        t = tensors[name]
        nb = t.numel() * t.element_size()
        if cur and size + nb > shard_bytes:
            files.append(_flush(cur, out_dir, len(files)))
            cur, size = {}, 0
        cur[name] = t
        size += nb
    if cur:
        files.append(_flush(cur, out_dir, len(files)))
    return files


def _flush(tensors: dict, out_dir: str, i: int) -> str:
    name = f"hessians-{i:05d}.safetensors"
    write_file(os.path.join(out_dir, name), tensors, {"format": "pt"})
    return name


def token_batches(path: str | None, tokenizer, vocab: int, rows: int, seq: int, seed: int = 0):
    """Calibration sequences: lines of a text file through the tokenizer (cut / packed to ``seq``), or, with no file,
    uniform random ids (data-free fallback that still shapes the Hessian by the network's own statistics)."""
    if path is None:
        g = torch.Generator().manual_seed(seed)
        for _ in range(max(1, rows // seq)):
            yield torch.randint(0, vocab, (seq,), generator=g)
        return
    buf: list[int] = []
    done = 0
    with open(path, encoding="utf-8") as f:
        for line in f:
            buf.extend(t for t in tokenizer.encode(line) if t < vocab)
            while len(buf) >= seq and done < rows:
                yield torch.tensor(buf[:seq])
                buf, done = buf[seq:], done + seq
            if done >= rows:
                return
    if buf and done < rows:
        yield torch.tensor(buf)
