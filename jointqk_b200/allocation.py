"""Reverse water-filling and the integer bit allocation used by the key compressor.

Public names follow the reference toolkit:

* ``water_fill(variances, total_bits, max_bits=16.0)``
      -- experiments/stage1/toolkit/metric_transform.py:156-213 (row solver :131-153)
* ``round_bits_to_integer(bits, total_bits=None)``
      -- experiments/stage1/toolkit/per_coord_quantization.py:236-258
* ``allocate_bits(scores, bits, max_coord_bits)``
      -- experiments/stage1/calibration/analyze_bases.py:140-185, the same tail as
         per_coord_quantization.py:360-379 (cap, then hand the excess to the coordinates
         holding the smallest allocation, lowest index first)

All arithmetic is fp32 on the CPU in the same operation order as the reference so that
the integer allocations are identical on identical inputs (golden-vector tests).
"""

from __future__ import annotations

import torch


def _water_level_row(log2_var: torch.Tensor, total_bits: float) -> torch.Tensor:
    """Unconstrained reverse water-fill of one row given log2 variances; bits >= 0."""
    d = log2_var.shape[0]
    ordered, order = torch.sort(log2_var, descending=True)
    prefix = torch.cumsum(ordered, dim=0)
    solved: torch.Tensor | None = None
    for k in range(1, d + 1):
        level = prefix[k - 1] / k - 2.0 * total_bits / k
        if ordered[k - 1] <= level:
            continue
        if k < d and ordered[k] > level:
            continue
        solved = (0.5 * (ordered - level)).clamp_min(0.0)
        break
    if solved is None:
        solved = torch.full_like(ordered, total_bits / d).clamp_min(0.0)
    out = torch.zeros_like(solved)
    out[order] = solved
    return out


def water_fill(variances: torch.Tensor, total_bits: float, max_bits: float = 16.0) -> torch.Tensor:
    """Continuous allocation ``b_j = max(0, 0.5*log2(v_j/theta))`` with ``sum b_j = total_bits``.

    Coordinates whose unconstrained share reaches ``max_bits`` are pinned there and the
    remainder is re-solved on the rest (at most d+1 rounds).  Accepts ``(d,)`` or ``(H, d)``.
    """
    v = variances.float().clamp_min(1e-30)
    squeeze = v.dim() == 1
    if squeeze:
        v = v.unsqueeze(0)
    n_rows, d = v.shape
    budget_cap = min(float(total_bits), d * float(max_bits))
    log2_v = torch.log2(v)
    out = torch.zeros_like(v)
    for h in range(n_rows):
        live = torch.ones(d, dtype=torch.bool, device=v.device)
        row = torch.zeros(d, dtype=v.dtype, device=v.device)
        left = budget_cap
        done = False
        for _ in range(d + 1):
            if int(live.sum().item()) == 0 or left <= 0:
                done = True
                break
            idx = torch.nonzero(live, as_tuple=True)[0]
            part = _water_level_row(log2_v[h, idx], left)
            full = part >= max_bits
            if not full.any():
                row[idx] = part.clamp_max(max_bits)
                done = True
                break
            pinned = idx[full]
            row[pinned] = max_bits
            live[pinned] = False
            left -= int(full.sum().item()) * float(max_bits)
        if not done:
            raise RuntimeError("water_fill iterative loop did not converge")
        out[h] = row
    return out.squeeze(0) if squeeze else out


def round_bits_to_integer(bits: torch.Tensor, total_bits: int | None = None) -> torch.Tensor:
    """Non-negative integer bits; with ``total_bits`` the row sum is preserved by giving the
    floor deficit to the largest fractional parts (``torch.topk`` order, as the reference)."""
    bits = bits.clamp_min(0.0)
    if total_bits is None:
        return bits.round().to(torch.long)
    lead = bits.shape[:-1]
    flat = bits.reshape(-1, bits.shape[-1])
    base = flat.floor()
    frac = flat - base
    want = int(total_bits)
    out = base.clone()
    for i in range(flat.shape[0]):
        short = want - int(out[i].sum().item())
        if short <= 0:
            continue
        _, pick = torch.topk(frac[i], k=short)
        out[i, pick] += 1
    return out.reshape(lead + (flat.shape[-1],)).to(torch.long)


def cap_and_redistribute(bits_int: torch.Tensor, max_coord_bits: int) -> torch.Tensor:
    """Clamp one row at ``max_coord_bits`` and re-seat the removed bits one round at a time on
    the coordinates that currently hold the minimum allocation below the cap (lowest index
    first).  Same loop as per_coord_quantization.py:367-379 with the cap as a parameter."""
    out = bits_int.clone()
    spare = int((out - max_coord_bits).clamp_min(0).sum().item())
    out.clamp_(max=max_coord_bits)
    while spare > 0:
        below = (out < max_coord_bits).nonzero(as_tuple=True)[0]
        if below.numel() == 0:
            break
        low = out[below].min()
        cand = below[out[below] == low]
        take = min(int(cand.numel()), spare)
        out[cand[:take]] += 1
        spare -= take
    return out


def allocate_bits_for_budget(scores: torch.Tensor, total_bits: float, max_coord_bits: int) -> torch.Tensor:
    """Integer allocation for an arbitrary (possibly fractional) budget.

    ``total_bits = b_avg * d`` feeds the continuous water-fill as a float and the rounding
    step as ``int(total_bits)`` (per_coord_quantization.py:286,363-364)."""
    lead = scores.shape[:-1]
    d = int(scores.shape[-1])
    flat = scores.detach().float().cpu().reshape(-1, d).clamp_min(1e-30)
    cont = water_fill(flat, total_bits=float(total_bits))
    ints = round_bits_to_integer(cont, total_bits=int(total_bits))
    rows = [cap_and_redistribute(ints[i], int(max_coord_bits)) for i in range(ints.shape[0])]
    return torch.stack(rows, 0).reshape(lead + (d,)).to(scores.device)


def allocate_bits(scores: torch.Tensor, bits: int, max_coord_bits: int = 8) -> torch.Tensor:
    """Reference signature: integer average ``bits`` per coordinate, budget ``bits * d``."""
    return allocate_bits_for_budget(scores, float(int(bits) * int(scores.shape[-1])), max_coord_bits)
