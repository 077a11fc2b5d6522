"""Round trip on the GPU without a packed record.

The packed record holds 0..8 bits per coordinate with at most ``MAX_WIDE`` coordinates above 4 bits
and 512 bits per key.  The reference's default recipe (water-fill tail capped at 8 bits,
experiments/stage1/toolkit/per_coord_quantization.py:365-379) leaves that range from budgets of about
3.5 bits per coordinate on, and its ``roundtrip`` (:123-165) never needs a record.  ``DenseTables``
holds what one launch of ``jqk_roundtrip_dense`` needs for such objects: the maps, the exact fp32
decision thresholds of every coordinate (``layout.decision_thresholds``, 255 per coordinate) and its
levels.  Keys stay unpacked on this path, so there is no cache to attend over: it serves
``roundtrip`` / ``codes`` / ``batched_roundtrip`` and the evaluation scores, which is all the
reference does with a compressor.
"""

from __future__ import annotations

import numpy as np
import torch

from . import _native
from .layout import decision_thresholds

MAX_DENSE_BITS = 8


class DenseTables:
    """forward_maps / inverse_maps (H, d, d), codebooks (H, d, K) +inf padded (K <= 256); ``center`` (H, d) or None."""

    def __init__(self, forward_maps: torch.Tensor, inverse_maps: torch.Tensor, codebooks: torch.Tensor, device,
                 center: torch.Tensor | None = None) -> None:
        fwd = forward_maps.detach().float().cpu().contiguous()
        inv = inverse_maps.detach().float().cpu().contiguous()
        cb = codebooks.detach().float().cpu().contiguous()
        H, d, K = cb.shape
        if fwd.shape != (H, d, d) or inv.shape != (H, d, d):
            raise ValueError(f"maps must be ({H}, {d}, {d}), got {tuple(fwd.shape)} and {tuple(inv.shape)}")
        if d > 128:
            raise ValueError(f"head_dim must be at most 128, got {d}")
        lengths = torch.isfinite(cb).sum(-1)
        if int(lengths.min()) < 1 or not bool(((lengths & (lengths - 1)) == 0).all()):
            raise ValueError("every codebook row needs 2^b finite levels")
        if int(lengths.max()) > 2 ** MAX_DENSE_BITS:
            raise ValueError(f"at most {MAX_DENSE_BITS} bits per coordinate, got a row of {int(lengths.max())} levels")
        widths = torch.log2(lengths.float()).round().to(torch.int32)
        rows = np.zeros((H * d, 256), np.float32)
        kk = min(K, 256)
        flat = cb.reshape(H * d, K).numpy()
        rows[:, :kk] = np.where(np.isfinite(flat[:, :kk]), flat[:, :kk], 0.0)
        thr = decision_thresholds(rows, widths.reshape(-1).numpy(), max_levels=256)          # (H d, 255), +inf padded
        self.n_heads, self.d = H, d
        self.device = torch.device(device)
        up = lambda a: a.to(self.device).contiguous()
        self.fwd, self.inv = up(fwd), up(inv)
        self.thresholds = up(torch.from_numpy(thr).reshape(H, d, 255))
        self.levels = up(torch.from_numpy(rows).reshape(H, d, 256))
        self.widths = up(widths)
        self.center = None if center is None else up(center.detach().float().cpu().reshape(H, d))

    @torch.no_grad()
    def roundtrip(self, rows: torch.Tensor, want_out: bool = True, want_codes: bool = False):
        """rows (H, N, d) fp32 / bf16 / fp16 on this device -> (fp32 reconstruction or None, uint8 codes or None)."""
        H, N, d = rows.shape
        if H != self.n_heads or d != self.d:
            raise ValueError(f"rows must be ({self.n_heads}, N, {self.d}), got {tuple(rows.shape)}")
        if rows.dtype not in (torch.float32, torch.bfloat16, torch.float16):
            rows = rows.float()
        rows = rows.to(self.device)
        if rows.stride(2) != 1:
            rows = rows.contiguous()
        out = torch.empty((H, N, d), dtype=torch.float32, device=self.device) if want_out else None
        codes = torch.empty((H, N, d), dtype=torch.uint8, device=self.device) if want_codes else None
        if N:
            _native.check(_native.lib.jqk_roundtrip_dense(
                self.fwd.data_ptr(), self.inv.data_ptr(), self.thresholds.data_ptr(), self.levels.data_ptr(),
                self.widths.data_ptr(), None if self.center is None else self.center.data_ptr(), H, d, rows.data_ptr(),
                _native.torch_dtype_code(rows.dtype), rows.stride(0), rows.stride(1), N,
                None if out is None else out.data_ptr(), None if codes is None else codes.data_ptr(),
                torch.cuda.current_stream(self.device).cuda_stream))
        return out, codes
