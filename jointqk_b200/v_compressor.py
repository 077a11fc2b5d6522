"""Value-side compressors with the reference toolkit's interface.

Drop-in for ``CenteredCompressor`` / ``build_v_compressor`` / ``V_METHOD_NAMES`` of
experiments/stage1/toolkit/v_compressor_adapter.py for the methods built on the per-coordinate
quantiser: ``v_eigen_waterfill`` (eigenbasis of Cov[V], reverse water-fill on its eigenvalues),
``v_eigen_uniform`` and ``v_random`` (same bits on every coordinate).  For values the distortion
target is plain reconstruction error, so the water-fill weights are the variances alone (:190-196).
``v_turboquant`` wraps a third-party compressor that is outside this path and raises.

The arithmetic runs in the same CUDA kernels as the key side: a centred compressor uploads its
mean with the head tables, the compress kernel subtracts it from every row in fp32 before the
transform and the decompress kernel adds it back, as ``CenteredCompressor.roundtrip`` does (:64-72).
"""

from __future__ import annotations

import torch

from . import paged
from .allocation import cap_and_redistribute, round_bits_to_integer, water_fill
from .compressor import PerCoordCompressor, _cuda_device
from .tables import HeadTables

V_METHOD_NAMES = ("v_random", "v_eigen_uniform", "v_eigen_waterfill", "v_turboquant")


class CenteredCompressor:
    """Wraps a per-coordinate compressor with mean centring: subtract ``mu`` before quantising, add it
    back after (reference :46-72).  ``roundtrip`` keeps the reference's contract; ``compress`` /
    ``decompress`` expose the packed pages in between."""

    def __init__(self, inner: PerCoordCompressor, mu: torch.Tensor) -> None:
        self.inner = inner
        self.mu = mu                      # (d,) in original (un-rotated) coordinates
        self._tables: HeadTables | None = None
        self._dense = None

    @property
    def d(self) -> int:
        return self.inner.d

    def to(self, device) -> "CenteredCompressor":
        self.inner.to(device)
        if self.mu.device != torch.device(device):
            self.mu = self.mu.to(device)
        return self

    def head_tables(self, device: torch.device | None = None) -> HeadTables:
        dev = _cuda_device(device)
        if not self.inner.packable:
            self.inner.head_tables(dev)   # raises with the explanation
        if self._tables is None or self._tables.device != dev:
            self._tables = HeadTables.from_compressors([self.inner], device=dev, center=self.mu.reshape(1, -1))
        return self._tables

    @torch.no_grad()
    def compress(self, states: torch.Tensor) -> paged.PackedKeys:
        if states.shape[-1] != self.d:
            raise ValueError(f"states last-dim {states.shape[-1]} != compressor.d {self.d}")
        dev = _cuda_device(states.device)
        flat = states.reshape(-1, self.d)
        if flat.dtype not in (torch.float32, torch.bfloat16, torch.float16):
            flat = flat.float()
        packed = paged.compress(self.head_tables(dev), flat.to(dev).contiguous().view(1, 1, flat.shape[0], self.d))
        packed.leading_shape = tuple(states.shape[:-1])
        return packed

    @torch.no_grad()
    def decompress(self, packed: paged.PackedKeys) -> torch.Tensor:
        return paged.decompress(packed).reshape(tuple(packed.leading_shape) + (self.d,))

    @torch.no_grad()
    def roundtrip(self, states: torch.Tensor) -> torch.Tensor:
        if not self.inner.packable and int(self.inner.bits_int.max()) <= 8:
            # beyond the packed record: the same arithmetic without one (jqk_roundtrip_dense)
            from .dense import DenseTables

            dev = _cuda_device(states.device)
            if self._dense is None or self._dense.device != dev:
                self._dense = DenseTables(self.inner.forward_map.unsqueeze(0), self.inner.inverse_map.unsqueeze(0),
                                          self.inner.codebooks_padded.unsqueeze(0), dev, center=self.mu.reshape(1, -1))
            out, _ = self._dense.roundtrip(states.reshape(1, -1, self.d))
            return out.reshape(tuple(states.shape)).to(states.device)
        return self.decompress(self.compress(states)).to(states.device)


def _seeded_rotation(d: int, seed: int) -> torch.Tensor:
    """Orthogonal (d, d) from the QR of a seeded Gaussian matrix (reference :107-119)."""
    g = torch.Generator().manual_seed(seed)
    q, _ = torch.linalg.qr(torch.randn(d, d, generator=g))
    return q.float()


def build_v_compressor(method: str, cov_v_for_head: torch.Tensor | None = None, head_dim: int = 0, bits: int = 0,
                       seed: int = 42, mu_v_for_head: torch.Tensor | None = None, *,
                       sigma_v_for_head: torch.Tensor | None = None, max_bits: int = 8):
    """Reference signature (:122-134) plus ``max_bits``: the cap of the water-fill tail, 8 in the
    reference (:202); pass 4 for allocations the packed GPU format can store.  Returns a
    ``PerCoordCompressor`` or, with ``mu_v_for_head``, a ``CenteredCompressor`` around it."""
    if cov_v_for_head is None and sigma_v_for_head is not None:
        cov_v_for_head = sigma_v_for_head
    if method == "v_turboquant":
        raise ValueError("v_turboquant wraps a third-party compressor that is not part of this build")
    if cov_v_for_head is None:
        raise ValueError(f"{method} requires cov_v_for_head (or sigma_v_for_head)")
    cov = cov_v_for_head.detach().float().cpu()
    if method == "v_random":
        forward_map = _seeded_rotation(head_dim, seed)
    elif method.startswith("v_eigen_"):
        vals, vecs = torch.linalg.eigh(cov)
        forward_map = vecs[:, torch.argsort(vals, descending=True)].float()
    else:
        raise ValueError(f"Unknown V method: {method!r}")
    inverse_map = forward_map.transpose(-1, -2)
    var = (forward_map.transpose(-1, -2) @ cov @ forward_map).diagonal(dim1=-2, dim2=-1).clamp_min(1e-30)
    total_bits = int(bits) * head_dim
    if method.endswith("_random") or method.endswith("_uniform"):
        bits_int = torch.full((head_dim,), int(bits), dtype=torch.long)
        how = "uniform"
    elif method.endswith("_waterfill"):
        cont = water_fill(var.unsqueeze(0), total_bits=total_bits).squeeze(0)
        ints = round_bits_to_integer(cont.unsqueeze(0), total_bits=total_bits).squeeze(0)
        bits_int = cap_and_redistribute(ints, int(max_bits))
        how = f"capped_tail(max_bits={int(max_bits)})"
    else:
        raise ValueError(f"Unknown allocation in V method: {method!r}")
    inner = PerCoordCompressor(bits_int, torch.sqrt(var.float()), forward_map=forward_map.float(),
                               inverse_map=inverse_map.float())
    inner.allocation = how
    if mu_v_for_head is not None:
        return CenteredCompressor(inner, mu_v_for_head.detach().float())
    return inner
