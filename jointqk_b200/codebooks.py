"""Gaussian Lloyd-Max codebooks and the seeded rotation used by the synthetic configs.

Mirrors the reference toolkit's public names:

* ``solve_lloyd_max(d, bits)``        -- experiments/stage1/toolkit/quantization.py:18-50
* ``unit_gaussian_centroids(bits)``   -- experiments/stage1/toolkit/per_coord_quantization.py:25-40
* ``generate_rotation_matrix(d, seed)`` -- experiments/stage1/toolkit/quantization.py:53-62

The reference integrates the Gaussian cell moments numerically (scipy ``quad``).  Both
integrals have closed forms, so this module evaluates them with ``math.erf``/``math.exp``
in float64 and iterates the same Lloyd sweep (same initialisation, same outer edges, same
stopping rule).  After the final cast to fp32 the tables agree bit for bit with the
reference for 1..8 bits (asserted by the golden-vector test).
"""

from __future__ import annotations

import math

import torch

_LLOYD_MAX_CACHE: dict[tuple[int, int], tuple[torch.Tensor, torch.Tensor]] = {}
_UNIT_GAUSSIAN_CACHE: dict[int, torch.Tensor] = {}

_SQRT2 = math.sqrt(2.0)
_INV_SQRT_2PI = 1.0 / math.sqrt(2.0 * math.pi)


def _cell_mass_and_first_moment(a: float, b: float, sigma: float) -> tuple[float, float]:
    """Mass and first moment of N(0, sigma^2) restricted to [a, b] (closed form)."""
    za, zb = a / sigma, b / sigma
    # Mass via erf differences; for cells far in one tail use erfc to keep precision.
    if za > 0.0:
        mass = 0.5 * (math.erfc(za / _SQRT2) - math.erfc(zb / _SQRT2))
    elif zb < 0.0:
        mass = 0.5 * (math.erfc(-zb / _SQRT2) - math.erfc(-za / _SQRT2))
    else:
        mass = 0.5 * (math.erf(zb / _SQRT2) - math.erf(za / _SQRT2))
    first = sigma * _INV_SQRT_2PI * (math.exp(-0.5 * za * za) - math.exp(-0.5 * zb * zb))
    return mass, first


def solve_lloyd_max(d: int, bits: int, max_iter: int = 200, tol: float = 1e-10) -> tuple[torch.Tensor, torch.Tensor]:
    """Lloyd-Max quantiser for N(0, 1/d) with ``2**bits`` levels.

    Returns ``(centroids, boundaries)`` as fp32 tensors, ascending.  Follows the reference
    sweep: centroids start at the midpoints of ``2**bits`` equal cells of [-3.5s, 3.5s],
    cell edges are midpoints of neighbouring centroids with outer edges at +-10.5s, a cell
    whose mass is below 1e-15 keeps its centroid, and iteration stops when the largest
    move is below ``tol`` or after ``max_iter`` sweeps.
    """
    key = (int(d), int(bits))
    hit = _LLOYD_MAX_CACHE.get(key)
    if hit is not None:
        return hit[0].clone(), hit[1].clone()

    levels = 2 ** int(bits)
    sigma = 1.0 / math.sqrt(d)
    lo, hi = -3.5 * sigma, 3.5 * sigma
    cents = [lo + (hi - lo) * (i + 0.5) / levels for i in range(levels)]
    for _ in range(max_iter):
        mids = [(cents[i] + cents[i + 1]) / 2.0 for i in range(levels - 1)]
        edges = [lo * 3] + mids + [hi * 3]
        new = []
        for i in range(levels):
            mass, first = _cell_mass_and_first_moment(edges[i], edges[i + 1], sigma)
            new.append(first / mass if mass > 1e-15 else cents[i])
        shift = max(abs(new[i] - cents[i]) for i in range(levels))
        cents = new
        if shift < tol:
            break
    mids = [(cents[i] + cents[i + 1]) / 2.0 for i in range(levels - 1)]
    c = torch.tensor(cents, dtype=torch.float32)
    b = torch.tensor(mids, dtype=torch.float32)
    _LLOYD_MAX_CACHE[key] = (c.clone(), b.clone())
    return c, b


def unit_gaussian_centroids(bits: int) -> torch.Tensor:
    """Lloyd-Max centroids of a unit-variance Gaussian; ``zeros(1)`` for ``bits <= 0``.

    Computed as ``solve_lloyd_max(64, bits)[0] * 8`` exactly like the reference (the scale
    is a power of two, so the fp32 product is exact).
    """
    if bits <= 0:
        return torch.zeros(1)
    hit = _UNIT_GAUSSIAN_CACHE.get(int(bits))
    if hit is not None:
        return hit.clone()
    cents, _ = solve_lloyd_max(64, int(bits))
    cents = cents * math.sqrt(64)
    _UNIT_GAUSSIAN_CACHE[int(bits)] = cents.clone()
    return cents


def generate_rotation_matrix(d: int, seed: int | None = None, device: str | torch.device = "cpu") -> torch.Tensor:
    """Seeded Haar-like orthogonal matrix: QR of a CPU-generated Gaussian, column signs fixed
    so that diag(R) > 0 (reference: quantization.py:53-62)."""
    gen = torch.Generator(device="cpu")
    if seed is not None:
        gen.manual_seed(seed)
    g = torch.randn(d, d, generator=gen)
    q, r = torch.linalg.qr(g)
    s = torch.sign(torch.diag(r))
    s[s == 0] = 1.0
    return (q * s.unsqueeze(0)).to(device)
