"""Plain PyTorch fp32 restatements of every hot op: the oracle for the CUDA kernels.

Behaviour follows the reference's tiny readable references
(python/reference/cuteafd_reference/{rmsnorm,rope,router,moe,attention}_ref.py) and, where
those are silent, the contracts of its CUDA kernels: router bias is used for selection only and
ties go to the lowest expert id (native/shared/cuda/expert_router.cu:12-55); the MoE combine sums
routes in slot order in fp32 and rounds once (native/shared/cuda/route_reduce.cu:103-122).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    return (y * weight.float()).to(x.dtype)


def add_rmsnorm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6):
    """residual' = residual + x (rounded to the storage dtype), y = rmsnorm(residual')."""
    r = (residual.float() + x.float()).to(residual.dtype)
    return rmsnorm(r, weight, eps), r


def rope_angles(dim: int, positions: torch.Tensor, theta: float, inv_freq: torch.Tensor | None = None) -> torch.Tensor:
    inv = inv_freq.to(positions.device) if inv_freq is not None else \
        1.0 / (theta ** (torch.arange(0, dim, 2, device=positions.device).float() / dim))
    return torch.outer(positions.float(), inv)            # [T, dim/2]


def _yarn_mscale(factor: float, m: float) -> float:
    return 1.0 if factor <= 1.0 or m == 0.0 else 0.1 * m * math.log(factor) + 1.0


def rope_inv_freq(cfg, dim: int) -> torch.Tensor:
    """Rotation frequencies [dim / 2] (fp32) for the checkpoint's long-context scaling.  This table is the only thing
    the rope kernels read, so every scaling rule is host arithmetic:

    * ``linear``: every frequency divided by the factor (position interpolation).
    * ``llama3``: wavelengths above ``original_max / low_freq_factor`` are divided by the factor, those below
      ``original_max / high_freq_factor`` are kept, the band between is blended.
    * ``yarn``: per dimension a blend of the kept frequency (dimensions that rotate more than ``beta_fast`` times over
      the original context) and the interpolated one (fewer than ``beta_slow`` rotations), linear ramp between.
    """
    base = 1.0 / (cfg.rope_theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
    kind, f = cfg.rope_scaling, float(cfg.rope_factor)
    if kind in ("none", "default") or f == 1.0:
        return base
    if kind == "linear":
        return base / f
    if kind == "llama3":
        old = float(cfg.rope_original_max)
        lo_w, hi_w = old / cfg.rope_low_freq_factor, old / cfg.rope_high_freq_factor
        wavelen = 2 * math.pi / base
        scaled = torch.where(wavelen > lo_w, base / f, base)
        smooth = (old / wavelen - cfg.rope_low_freq_factor) / (cfg.rope_high_freq_factor - cfg.rope_low_freq_factor)
        blended = (1 - smooth) * scaled / f + smooth * scaled
        medium = ~(wavelen < hi_w) & ~(wavelen > lo_w)
        return torch.where(medium, blended, scaled)
    if kind == "yarn":
        def correction_dim(rotations: float) -> float:
            return dim * math.log(cfg.rope_original_max / (rotations * 2 * math.pi)) / (2 * math.log(cfg.rope_theta))
        low = max(math.floor(correction_dim(cfg.rope_beta_fast)), 0)
        high = min(math.ceil(correction_dim(cfg.rope_beta_slow)), dim - 1)
        if low == high:
            high += 0.001
        ramp = ((torch.arange(dim // 2, dtype=torch.float32) - low) / (high - low)).clamp(0, 1)
        keep = 1 - ramp
        return (base / f) * (1 - keep) + base * keep
    raise ValueError(f"unknown rope scaling {kind!r}")


def rope_magnitudes(cfg) -> tuple[float, float]:
    """(multiplier on cos / sin, multiplier on the softmax scale).  YaRN enlarges the logits to keep attention sharp
    over the longer context: DeepSeek-style configurations (``mscale_all_dim`` set) put ``mscale(all_dim)^2`` on the
    softmax scale and the ratio ``mscale / mscale(all_dim)`` on cos / sin (1 when the two are equal, as shipped);
    plain YaRN puts ``0.1 ln(factor) + 1`` on cos / sin."""
    if cfg.rope_scaling != "yarn" or cfg.rope_factor <= 1.0:
        return 1.0, 1.0
    if cfg.rope_mscale_all_dim:
        all_dim = _yarn_mscale(cfg.rope_factor, cfg.rope_mscale_all_dim)
        return _yarn_mscale(cfg.rope_factor, cfg.rope_mscale) / all_dim, all_dim * all_dim
    return _yarn_mscale(cfg.rope_factor, 1.0), 1.0


def apply_rope(x: torch.Tensor, positions: torch.Tensor, theta: float = 10000.0,
               interleaved: bool = True, inv_freq: torch.Tensor | None = None, magnitude: float = 1.0) -> torch.Tensor:
    """x: [T, heads, dim].  interleaved rotates pairs (2i, 2i+1); otherwise (i, i+dim/2).  ``inv_freq`` replaces the
    plain ``theta`` table (long-context scaling); ``magnitude`` multiplies cos and sin."""
    dim = x.shape[-1]
    rot = 2 * inv_freq.shape[0] if inv_freq is not None else dim
    if rot < dim:                      # partial rotary: the leading ``rot`` dims rotate, the rest pass through
        head = apply_rope(x[..., :rot], positions, theta, interleaved, inv_freq, magnitude)
        return torch.cat([head, x[..., rot:]], dim=-1)
    ang = rope_angles(dim, positions, theta, inv_freq)
    cos, sin = ang.cos()[:, None, :] * magnitude, ang.sin()[:, None, :] * magnitude
    xf = x.float()
    if interleaved:
        a, b = xf[..., 0::2], xf[..., 1::2]
        out = torch.empty_like(xf)
        out[..., 0::2] = a * cos - b * sin
        out[..., 1::2] = a * sin + b * cos
    else:
        a, b = xf[..., : dim // 2], xf[..., dim // 2:]
        out = torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1)
    return out.to(x.dtype)


def route_topk(logits: torch.Tensor, top_k: int, scoring: str = "softmax", bias: torch.Tensor | None = None,
               num_groups: int = 1, topk_groups: int = 1, normalize: bool = True,
               routed_scale: float = 1.0) -> tuple[torch.Tensor, torch.Tensor]:
    """Router selection.  Returns (indices int32 [T,k], weights fp32 [T,k]).

    softmax: full-denominator softmax, top-k by probability, optional renormalisation.
    sigmoid: scores = sigmoid(logits); selection on scores+bias; group-limited routing keeps the
    ``topk_groups`` groups whose top-2 (biased) scores sum highest; weights are the unbiased
    scores, normalised with +1e-20 and scaled.  Ties resolve to the lowest expert id.
    """
    lf = logits.float()
    T, E = lf.shape
    scores = torch.softmax(lf, dim=-1) if scoring == "softmax" else torch.sigmoid(lf)
    sel = scores + bias.float() if bias is not None else scores.clone()
    if num_groups > 1:
        g = sel.view(T, num_groups, E // num_groups)
        gscore = g.topk(2, dim=-1).values.sum(-1)                      # [T, G]
        keep = _stable_topk(gscore, topk_groups)[1]
        mask = torch.zeros(T, num_groups, dtype=torch.bool, device=lf.device)
        mask.scatter_(1, keep, True)
        sel = sel.masked_fill(~mask[:, :, None].expand_as(g).reshape(T, E), float("-inf"))
    idx = _stable_topk(sel, top_k)[1]
    w = scores.gather(1, idx)
    if normalize:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return idx.to(torch.int32), (w * routed_scale).float()


def _stable_topk(x: torch.Tensor, k: int) -> tuple[torch.Tensor, torch.Tensor]:
    """top-k, value descending, ties to the lowest index (torch.topk leaves tie order open)."""
    order = torch.sort(x, dim=-1, descending=True, stable=True)
    return order.values[..., :k], order.indices[..., :k]


def swiglu_mlp(x: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    xf = x.float()
    h = F.silu(xf @ gate.float().T) * (xf @ up.float().T)
    return h.to(x.dtype).float() @ down.float().T           # intermediate rounded like the kernels do


def moe_forward(x: torch.Tensor, idx: torch.Tensor, w: torch.Tensor, gate: torch.Tensor, up: torch.Tensor,
                down: torch.Tensor, expert_base: int = 0) -> torch.Tensor:
    """Routed experts for the experts held locally: gate/up [E_local, I, H], down [E_local, H, I].

    Returns fp32 [T, k, H]: per-(token, slot) weighted contribution, zero where the slot's expert
    is not local.  The caller sums the slots in slot order.
    """
    T, k = idx.shape
    out = torch.zeros(T, k, x.shape[-1], dtype=torch.float32, device=x.device)
    e_local = gate.shape[0]
    for e in range(e_local):
        hit = (idx == e + expert_base)
        if not hit.any():
            continue
        rows, slots = hit.nonzero(as_tuple=True)
        y = swiglu_mlp(x[rows], gate[e], up[e], down[e])
        out[rows, slots] = y.to(x.dtype).float() * w[rows, slots][:, None]
    return out


def combine_slots(parts: torch.Tensor, shared: torch.Tensor | None, residual: torch.Tensor | None,
                  dtype: torch.dtype) -> torch.Tensor:
    """Ordered fp32 sum over slots, then the shared expert, then the residual; one rounding."""
    acc = torch.zeros_like(parts[:, 0])
    for s in range(parts.shape[1]):
        acc = acc + parts[:, s]
    if shared is not None:
        acc = acc + shared.float()
    if residual is not None:
        acc = acc + residual.float()
    return acc.to(dtype)


def index_select(q_idx: torch.Tensor, k_idx: torch.Tensor, head_w: torch.Tensor, q_start: int, top_k: int) -> torch.Tensor:
    """Lightning-indexer selection.  q_idx [Tq, Hi, Di], k_idx [Tk, Di], head_w [Tq, Hi] (fp32).  Returns a bool
    mask [Tq, Tk]: the top_k visible positions by sum_h w * relu(q . k), ties to the lower position; every
    visible position when there are at most top_k."""
    s = torch.einsum("th,thl->tl", head_w.float(), torch.relu(torch.einsum("thd,ld->thl", q_idx.float(), k_idx.float())))
    Tq, Tk = s.shape
    allowed = torch.zeros(Tq, Tk, dtype=torch.bool)
    for i in range(Tq):
        n = min(Tk, q_start + i + 1)
        if n <= top_k:
            allowed[i, :n] = True
        else:
            order = torch.sort(s[i, :n], descending=True, stable=True).indices[:top_k]
            allowed[i, order] = True
    return allowed


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_start: int, scale: float | None = None,
                     allowed: torch.Tensor | None = None, window: int = 0) -> torch.Tensor:
    """q [Tq, Hq, D], k [Tk, Hk, D], v [Tk, Hk, Dv]; query row i sits at position q_start+i.  ``allowed`` [Tq, Tk]
    further restricts the visible positions (sparse attention); ``window`` > 0 keeps keys (t - window, t] only."""
    Tq, Hq, D = q.shape
    Tk, Hk, _ = k.shape
    rep = Hq // Hk
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    kf = k.float().repeat_interleave(rep, dim=1)
    vf = v.float().repeat_interleave(rep, dim=1)
    s = torch.einsum("qhd,khd->hqk", q.float(), kf) * scale
    qpos = torch.arange(Tq, device=q.device)[:, None] + q_start
    kpos = torch.arange(Tk, device=q.device)[None, :]
    s = s.masked_fill((kpos > qpos)[None], float("-inf"))
    if window > 0:
        s = s.masked_fill((kpos <= qpos - window)[None], float("-inf"))
    if allowed is not None:
        s = s.masked_fill(~allowed.to(s.device)[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hqk,khd->qhd", p, vf).to(q.dtype)


def greedy_verify(target_logits: torch.Tensor, draft: torch.Tensor) -> tuple[int, int]:
    """Sample-match verification for greedy rows: accepted prefix length and the bonus token
    (python/reference/cuteafd_reference/mtp_protocol_ref.py:6-15)."""
    pred = target_logits.argmax(-1).tolist()
    n = 0
    for p, d in zip(pred, draft.tolist()):
        if p != d:
            break
        n += 1
    return n, pred[n]


def fp8_latent_roundtrip(latent: torch.Tensor, group: int = 128) -> torch.Tensor:
    """Latents as the FP8 cache record stores them: per 128 values one fp32 scale amax / 448, values rounded to E4M3,
    decoded back to the input dtype (reference record: native/shared/cuda/mla_indexing.cu, fp8_ds_mla pack)."""
    T, D = latent.shape
    if D % group:
        group = D
    v = latent.float().view(T, D // group, group)
    scale = v.abs().amax(dim=-1, keepdim=True).clamp_min(1e-12) * (1.0 / 448.0)
    q = (v * (1.0 / scale)).to(torch.float8_e4m3fn).float()
    return (q * scale).view(T, D).to(latent.dtype)
