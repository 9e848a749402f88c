"""Host-side codebook fit ("distribution fit") for ARCQ quantizers.

One-off work per tensor: from a sample of normalised residuals t = (x - mean)/scale
produce the sorted non-uniform codebook of 2**bits levels that all groups of the
tensor share, and its thresholds (midpoints).  Only these two small vectors enter
the CUDA kernels.  Same procedure as the reference's
``ARCQQuantizer._build_codebook_from_flat`` with its moment tables
(methods/fair_qat_framework/quant/dcarcq.py:24-105, :155-290): kurtosis ->
generalised-Gaussian shape beta -> clip point tau -> share of levels for the
negative and positive side proportional to p^(1/3) * sigma^(2/3) -> two linear
ramps around an exact zero level, each reaching min(mean + 3*std, 1.2*tau) of its
side.  Scalars are evaluated on the host; tensors may live on any device.
"""
from __future__ import annotations

import math
from functools import lru_cache

import torch

N_BETA = 512
N_U = 4096


@lru_cache(maxsize=None)
def _beta_kappa():
    beta = torch.linspace(0.75, 8.0, N_BETA)
    kappa = torch.tensor([math.exp(math.lgamma(5.0 / b) + math.lgamma(1.0 / b) - 2.0 * math.lgamma(3.0 / b))
                          for b in beta.tolist()], dtype=torch.float32)
    return beta, kappa


@lru_cache(maxsize=None)
def _tau_table(bits: int) -> torch.Tensor:
    """tau(beta): the point where the generalised-Gaussian |t| CDF reaches 1 - 1/(2 L^2)."""
    beta, _ = _beta_kappa()
    L = 2 ** bits
    target = 1.0 - 1.0 / (2.0 * L * L)
    out = torch.full((N_BETA,), 8.0)
    for i, b in enumerate(beta.tolist()):
        alpha = math.sqrt(math.exp(math.lgamma(1.0 / b) - math.lgamma(3.0 / b)))
        Z = math.exp(math.log(b) - math.log(alpha) - math.lgamma(1.0 / b))
        u_max = 8.0
        for _ in range(6):
            u = torch.linspace(0.0, u_max, N_U)
            cdf = torch.cumsum((b / Z) * torch.exp(-((u / alpha) ** b)), dim=0)
            cdf = cdf / cdf[-1]
            if cdf[-1] >= target:
                break
            u_max *= 2.0
        hit = (cdf >= target).nonzero()
        if hit.numel():
            out[i] = u[hit[0, 0]]
    return out


def shape_and_clip(kurtosis: float, bits: int):
    """(beta, tau) for a sample kurtosis."""
    beta_grid, kappa = _beta_kappa()
    k = min(max(float(kurtosis), float(kappa.min())), float(kappa.max()))
    beta = float(beta_grid[(kappa - k).abs().argmin()])
    if bits in (1, 2, 3, 4, 5, 6, 8):
        tau = float(_tau_table(bits)[(beta_grid - beta).abs().argmin()])
        tau = min(max(tau, 0.5), 8.0)
    else:
        tau = 2.5
    return beta, tau


def _reach(side: torch.Tensor, tau: float) -> float:
    if side.numel() < 2:
        return tau
    return min(side.mean().item() + 3.0 * side.std().item(), 1.2 * tau)


@torch.no_grad()
def fit_codebook(t_flat: torch.Tensor, bits: int, eps: float = 1e-6) -> torch.Tensor:
    """Sorted fp32 codebook of 2**bits levels fitted to the sample t_flat (1-D)."""
    if bits < 2:
        raise ValueError("bits must be >= 2")
    t = t_flat.detach().float().flatten()
    L = 2 ** bits
    sq = t * t
    m2, m4 = sq.mean().item(), (sq * sq).mean().item()
    _, tau = shape_and_clip(m4 / max(m2 * m2, eps), bits)
    ts = t.clamp(-tau, tau) if bits >= 3 else t
    pos, neg = ts[ts > 1e-8], ts[ts < -1e-8]
    p_pos, p_neg = pos.numel() / ts.numel(), neg.numel() / ts.numel()
    s_pos = pos.std().item() if pos.numel() else 1.0
    s_neg = neg.abs().std().item() if neg.numel() else 1.0
    w_pos = max(p_pos, 1e-8) ** (1 / 3) * s_pos ** (2 / 3)
    w_neg = max(p_neg, 1e-8) ** (1 / 3) * s_neg ** (2 / 3)
    share = w_pos / (w_pos + w_neg + 1e-8)
    reach_pos = _reach(pos, tau) if pos.numel() else tau
    reach_neg = _reach(-neg, tau) if neg.numel() else tau
    dev = t.device
    if bits == 2:      # four levels, none at zero
        n_pos = max(1, round(L * share))
        n_neg = L - n_pos
        if n_neg < 1:
            n_neg, n_pos = 1, L - 1
        levels = torch.cat([-torch.linspace(0.05, reach_neg, n_neg, device=dev).flip(0),
                            torch.linspace(0.05, reach_pos, n_pos, device=dev)])
    else:              # one level pinned at zero, the rest shared between the sides
        n_pos = max(1, round(L * share))
        n_neg = L - n_pos - 1
        if n_neg < 1:
            n_neg = 1
            n_pos = L - 2
        levels = torch.cat([-torch.linspace(0.0, reach_neg, n_neg + 1, device=dev)[1:].flip(0),
                            torch.zeros(1, device=dev),
                            torch.linspace(0.0, reach_pos, n_pos + 1, device=dev)[1:]])
    return levels[:L].sort()[0].float()


def thresholds_from_codebook(codebook: torch.Tensor) -> torch.Tensor:
    """Decision thresholds: midpoints of adjacent levels (reference: quant/dcarcq.py:483)."""
    return (codebook[:-1] + codebook[1:]) / 2.0


@torch.no_grad()
def normalized_residuals(x: torch.Tensor, group_size: int = 64, eps: float = 1e-6) -> torch.Tensor:
    """[..., C] -> [n_groups, group_size] of (x - mean) / sqrt(mean(r^2) + eps), fp32."""
    x3 = x.detach().float().reshape(-1, x.shape[-1] // group_size, group_size)
    r = x3 - x3.mean(dim=-1, keepdim=True)
    s = (r.square().mean(dim=-1, keepdim=True) + eps).sqrt()
    return (r / s).reshape(-1, group_size)


@torch.no_grad()
def calibrate_codebook(x: torch.Tensor, bits: int, group_size: int = 64, eps: float = 1e-6,
                       stats_sample_groups: int = 4096):
    """One codebook compile on tensor x: subsample every step-th group when there are more
    than ``stats_sample_groups`` of them (reference: quant/dcarcq.py:474-484), fit, and
    return (codebook, thresholds)."""
    t = normalized_residuals(x, group_size, eps)
    if t.shape[0] > stats_sample_groups:
        t = t[:: max(1, t.shape[0] // stats_sample_groups)]
    cb = fit_codebook(t.flatten(), bits, eps)
    return cb, thresholds_from_codebook(cb)
