"""Exact full-vocabulary target sampling: the CPU oracle and the request-side parameter object.

Filter order: allowed-token mask -> temperature -> min_p -> top_k (exactly k, lowest id wins a
boundary tie) -> top_p (smallest descending prefix reaching the mass); the best token always
survives.  Greedy when temperature < 1e-5 or top_k == 1.  The uniform draw is a pure function of
(seed, absolute decode position), so batching, compaction and speculative row layout cannot
change a token.  Non-finite logits are a per-row error, never undefined behaviour.

Counterpart: rust/crates/cuteafd-core/src/target_sampling.rs:9-215 (semantics, SplitMix64 draw),
native/shared/cuda/sampling_gpu.h:82-120 (row status codes, 64-byte row parameters).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

GREEDY_EPS = 1.0e-5
MAX_TEMPERATURE = 2.0
MAX_UNIFORM = 0.99999994
_M64 = (1 << 64) - 1
STATUS_OK, STATUS_NONFINITE, STATUS_EMPTY_MASK, STATUS_BAD_PARAM = 0, 1, 2, 3


class SamplingError(ValueError):
    def __init__(self, status: int, msg: str):
        super().__init__(msg)
        self.status = status


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int | None = None
    min_p: float = 0.0
    seed: int = 0

    def __post_init__(self) -> None:
        if not (math.isfinite(self.temperature) and 0.0 <= self.temperature <= MAX_TEMPERATURE):
            raise SamplingError(STATUS_BAD_PARAM, "temperature must be in [0, 2]")
        if not (math.isfinite(self.top_p) and 0.0 < self.top_p <= 1.0):
            raise SamplingError(STATUS_BAD_PARAM, "top_p must be in (0, 1]")
        if self.top_k is not None and self.top_k < 1:
            raise SamplingError(STATUS_BAD_PARAM, "top_k must be at least 1")
        if not (math.isfinite(self.min_p) and 0.0 <= self.min_p <= 1.0):
            raise SamplingError(STATUS_BAD_PARAM, "min_p must be in [0, 1]")

    @property
    def greedy(self) -> bool:
        return self.temperature < GREEDY_EPS or self.top_k == 1

    def uniform(self, position: int) -> float:
        """SplitMix64 over (domain, seed, position) -> 24-bit uniform in [0, 1)."""
        x = (self.seed + 0x7F4A7C159E3779B9 + ((position * 0x9E3779B97F4A7C15) & _M64) + 0x9E3779B97F4A7C15) & _M64
        x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _M64
        x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _M64
        x ^= x >> 31
        return (x >> 40) * (1.0 / 16777216.0)


def select_token(logits: torch.Tensor, params: SamplingParams, position: int, mask: torch.Tensor | None = None,
                 uniform: float | None = None) -> int:
    """One row.  ``mask`` is a bool tensor of allowed tokens (None = all)."""
    if logits.numel() == 0:
        raise SamplingError(STATUS_BAD_PARAM, "empty vocabulary")
    x = logits.detach().float().cpu()
    allowed = torch.ones_like(x, dtype=torch.bool) if mask is None else mask.cpu().bool()
    if not allowed.any():
        raise SamplingError(STATUS_EMPTY_MASK, "the grammar allows no token")
    if not torch.isfinite(x[allowed]).all():
        raise SamplingError(STATUS_NONFINITE, "non-finite logit among the allowed tokens")
    x = torch.where(allowed, x, torch.full_like(x, float("-inf")))
    if params.greedy:
        best = x.max()
        return int(torch.nonzero(x == best)[0])          # lowest id among ties
    x = x / params.temperature
    if params.min_p > 0.0:
        x = torch.where(x >= x.max() + math.log(params.min_p), x, torch.full_like(x, float("-inf")))
    # descending by value, ascending id inside ties
    order = torch.sort(x, descending=True, stable=True).indices
    if params.top_k is not None and params.top_k < x.numel():
        order = order[: params.top_k]
    order = order[torch.isfinite(x[order])]
    probs = torch.softmax(x[order].double(), dim=0)
    if params.top_p < 1.0:
        cum = torch.cumsum(probs, 0)
        keep = int(torch.searchsorted(cum, torch.tensor(params.top_p, dtype=torch.float64)).item()) + 1
        keep = max(1, min(keep, order.numel()))
        order, probs = order[:keep], probs[:keep] / probs[:keep].sum()
    u = params.uniform(position) if uniform is None else uniform
    u = min(max(u, 0.0), MAX_UNIFORM)
    cum = torch.cumsum(probs, 0)
    pick = int(torch.searchsorted(cum, torch.tensor(u * float(cum[-1]), dtype=torch.float64), right=True).item())
    return int(order[min(pick, order.numel() - 1)])


def select_rows(logits: torch.Tensor, params: list[SamplingParams], positions: list[int],
                masks: list[torch.Tensor | None] | None = None) -> tuple[list[int], list[int]]:
    """Batch form: returns (tokens, per-row status).  A failing row yields token -1 and its status;
    other rows are unaffected."""
    toks, status = [], []
    for i in range(logits.shape[0]):
        try:
            toks.append(select_token(logits[i], params[i], positions[i], None if masks is None else masks[i]))
            status.append(STATUS_OK)
        except SamplingError as e:
            toks.append(-1)
            status.append(e.status)
    return toks, status


def accept_prefix(selected: list[int], draft: list[int]) -> tuple[int, int]:
    """Sample-match verification: rows 0..n of ``selected`` are the target's choice after the last
    committed token and after each draft token.  A draft is accepted iff it equals the target's
    choice at that row; the first mismatch (or the row after the last draft) supplies the bonus
    token.  Returns (accepted drafts, bonus token)."""
    n = 0
    for d, s in zip(draft, selected):
        if d != s:
            break
        n += 1
    return n, selected[n]


def row_hash(logits: torch.Tensor) -> str:
    """Hash of a logit row's bytes (probe for byte-exactness checks)."""
    import hashlib
    return hashlib.blake2b(logits.detach().float().contiguous().cpu().numpy().tobytes(), digest_size=16).hexdigest()
