"""Device tables of one layer's kv heads: what the kernels read besides keys, values and pages.

Built on the host from the same three tensors the reference's batched path consumes --
``forward_maps (H,d,d)``, ``inverse_maps (H,d,d)`` and ``codebooks (H,d,K)`` with ``+inf`` in
unused slots (``stack_per_head``, experiments/stage1/toolkit/per_coord_quantization.py:219-233)
-- and uploaded once.  The per-coordinate bit width is read off the codebook row length.
"""

from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import _native
from .codebooks import unit_gaussian_centroids
from .layout import MAX_TABLES, MAX_VALUE_WIDE_LEVELS, MAX_WIDE, KeyLayout, decision_thresholds, plan_key_layout, unit_quantiser_tables

DESC_INTS = 32
MAX_COLS = 128


def split_bf16_limbs(x: torch.Tensor, n_limbs: int = 3) -> torch.Tensor:
    """Split fp32 ``x`` into ``n_limbs`` bf16 tensors whose sum reproduces ``x`` to ~2^-24.

    Each limb is the round-to-nearest bf16 of the residual left by the previous limbs, so
    bf16 x bf16 products against bf16 keys are exact in fp32 and only the accumulation order
    differs from a plain fp32 dot product."""
    res = x.float().clone()
    limbs = []
    for _ in range(n_limbs):
        l = res.to(torch.bfloat16)
        limbs.append(l)
        res = res - l.float()
    return torch.stack(limbs, 0)


class HeadTables:
    """Stacked tables for ``H`` heads; owns the device tensors and the ctypes struct."""

    def __init__(self, forward_maps: torch.Tensor | None, inverse_maps: torch.Tensor | None,
                 codebooks: torch.Tensor, device: torch.device | str = "cuda",
                 center: torch.Tensor | None = None) -> None:
        cb = codebooks.detach().float().cpu()
        if cb.dim() != 3:
            raise ValueError("codebooks must be (H, d, K)")
        H, d, K = cb.shape
        eye = torch.eye(d).expand(H, d, d)
        fwd = eye if forward_maps is None else forward_maps.detach().float().cpu()
        inv = fwd.transpose(-1, -2) if inverse_maps is None else inverse_maps.detach().float().cpu()
        if tuple(fwd.shape) != (H, d, d) or tuple(inv.shape) != (H, d, d):
            raise ValueError(f"maps must be (H, d, d) = ({H}, {d}, {d})")
        lengths = torch.isfinite(cb).sum(-1)                       # (H, d)
        if not bool(((lengths & (lengths - 1)) == 0).all()) or int(lengths.min()) < 1:
            raise ValueError("each codebook row must hold a power-of-two number of finite levels")
        if int(lengths.max()) > 256:
            raise ValueError(
                f"the packed GPU path stores at most 8 bits per coordinate; a codebook row has "
                f"{int(lengths.max())} levels")
        bits = torch.log2(lengths.float()).round().long()
        zero_rows = cb[..., 0][bits == 0]
        if zero_rows.numel() and float(zero_rows.abs().max()) != 0.0:
            raise ValueError("a 0-bit coordinate must reconstruct to 0.0")

        self.n_heads, self.d = H, d
        self.bits = bits.clone()
        self.layouts: list[KeyLayout] = [plan_key_layout(bits[h].numpy()) for h in range(H)]
        self.words_per_record = max(l.n_words for l in self.layouts)

        desc = np.zeros((H, DESC_INTS), np.int32)
        col_meta = np.zeros((H, MAX_COLS), np.int32)
        col_meta[:] = 255 << 16
        fields = np.full((H, MAX_TABLES, 4), -1, np.int32)
        fwd_cols = np.zeros((H, d, MAX_COLS), np.float32)
        qproj = np.zeros((H, d, MAX_COLS), np.float32)
        inv_rows = np.zeros((H, MAX_COLS, d), np.float32)
        thr = np.full((H, MAX_COLS, 16), np.inf, np.float32)
        cb_cols = np.zeros((H, MAX_COLS, 16), np.float32)
        # columns of 5..8 bits: their own 256-entry rows, indexed by column - wide_first
        self.n_wide = max(l.n_wide for l in self.layouts)
        self.decodable = all(l.decodable for l in self.layouts)     # every head's lookups fit the decode kernels' table memory
        # as value tables: the kernel holds the levels of a head's wide columns as they are
        self.value_decodable = all(int(sum(1 << int(w) for w in l.col_width[l.wide_first:l.wide_first + l.n_wide]))
                                   <= MAX_VALUE_WIDE_LEVELS for l in self.layouts)
        wide_thr = np.full((H, MAX_WIDE, 256), np.inf, np.float32)
        wide_cb = np.zeros((H, MAX_WIDE, 256), np.float32)
        col_scale = np.ones((H, MAX_COLS), np.float32)     # 1 / sigma of the column's coordinate
        unit = {b: unit_gaussian_centroids(b).numpy() for b in range(1, 9 if self.n_wide else 5)}
        scaled_ok = True
        cb_np, fwd_np, inv_np = cb.numpy(), fwd.numpy(), inv.numpy()
        for h, lay in enumerate(self.layouts):
            desc[h, :8] = lay.descriptor()
            desc[h, 8:8 + lay.n_words + 1] = lay.word_col_begin
            desc[h, 30], desc[h, 31] = lay.wide_first, lay.n_wide
            n = lay.n_active
            coords = lay.col_coord[:n]
            col_meta[h, :n] = lay.col_width[:n] | (lay.col_bitpos[:n] << 4) | (coords << 16)
            if len(lay.table_fields):
                fields[h, :len(lay.table_fields)] = lay.table_fields
            fwd_cols[h, :, :n] = fwd_np[h][:, coords]
            qproj[h, :, :n] = inv_np[h][coords, :].T
            inv_rows[h, :n, :] = inv_np[h][coords, :]
            rows = np.zeros((n, 16), np.float32)
            kk = min(K, 16)
            rows[:, :kk] = np.where(np.isfinite(cb_np[h][coords, :kk]), cb_np[h][coords, :kk], 0.0)
            narrow = lay.col_width[:n] <= 4
            rows[~narrow] = 0.0
            cb_cols[h, :n] = rows
            thr[h, :n, :15] = decision_thresholds(rows, np.where(narrow, lay.col_width[:n], 0))
            if lay.n_wide:
                wc = np.arange(lay.wide_first, lay.wide_first + lay.n_wide)
                wrows = np.zeros((lay.n_wide, 256), np.float32)
                kw = min(K, 256)
                wrows[:, :kw] = np.where(np.isfinite(cb_np[h][coords[wc], :kw]), cb_np[h][coords[wc], :kw], 0.0)
                wide_cb[h, :lay.n_wide] = wrows
                wide_thr[h, :lay.n_wide, :255] = decision_thresholds(wrows, lay.col_width[wc], max_levels=256)
            # the codebook row is unit levels x sigma (per_coord_quantization.py:107): the ratio of the
            # top levels gives 1 / sigma back to an ulp, which is all the scaled transform needs
            for c in range(n):
                w = int(lay.col_width[c])
                top = float(rows[c, (1 << w) - 1]) if w <= 4 else float(wide_cb[h, c - lay.wide_first, (1 << w) - 1])
                if not (top > 1e-30 and np.isfinite(top)):
                    scaled_ok = False
                else:
                    col_scale[h, c] = np.float32(float(unit[w][-1]) / top)
        self.device = torch.device(device)
        if self.device.type == "cuda" and self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        up = lambda a: torch.from_numpy(a).to(self.device)
        self.desc, self.col_meta, self.table_fields = up(desc), up(col_meta), up(fields)
        self.fwd_cols, self.qproj_cols, self.inv_rows = up(fwd_cols), up(qproj), up(inv_rows)
        self.thresholds, self.cb_cols = up(thr), up(cb_cols)
        self.wide_thr = self.wide_cb = None
        if self.n_wide:
            self.wide_thr, self.wide_cb = up(wide_thr), up(wide_cb)
        # Tensor-core transform: the basis columns scaled by 1 / sigma of their coordinate, so that every
        # transformed value is quantised against the unit levels of its width (one shared set of tables,
        # layout.unit_quantiser_tables), split into three bf16 limbs, [H][3][col][dim] (column-major =
        # K-major B operand).  Absent when a codebook is degenerate; the CUDA-core kernel then runs.
        u_thr, u_pre, u_aff = unit_quantiser_tables(unit)
        self.unit_thr, self.unit_aff = u_thr, u_aff
        self.unit_pre = up(u_pre)
        # unit thresholds of the widths 5..8, a 256-entry row each (+inf padded): the tensor-core kernel
        # finds a wide column's code by binary search over the row of its width
        self.unit_wide_thr = None
        if self.n_wide:
            uw = np.full((4, 256), np.inf, np.float32)
            for b in range(5, 9):
                rows_b = np.zeros((1, 256), np.float32)
                rows_b[0, : 2 ** b] = unit[b]
                uw[b - 5, :255] = decision_thresholds(rows_b, np.array([b]), max_levels=256)[0]
            self.unit_wide_thr = up(uw)
        self.fwd_limbs = None
        if scaled_ok:
            scaled = torch.from_numpy(fwd_cols * col_scale[:, None, :])
            self.fwd_limbs = split_bf16_limbs(scaled.transpose(1, 2).contiguous(), 3) \
                .permute(1, 0, 2, 3).contiguous().to(self.device)
        # optional per-head mean, subtracted before the transform and added back after reconstruction
        self.center = self.center_cols = None
        if center is not None:
            c = center.detach().float().cpu().reshape(H, d).contiguous()
            self.center = c.to(self.device)
            if self.fwd_limbs is not None:
                # the mean in column space, through exactly the basis the tensor cores multiply by (the
                # sum of the three limbs), in fp64: transform(raw row) - this = transform(row - mean)
                basis = self.fwd_limbs.float().cpu().double().sum(1)                # [H][col][dim]
                self.center_cols = torch.einsum("hd,hcd->hc", c.double(), basis).float().contiguous().to(self.device)
        self.struct = _native.JqkHeadTables(
            n_heads=H, d=d, words_per_record=self.words_per_record, n_wide=self.n_wide,
            desc=self.desc.data_ptr(), col_meta=self.col_meta.data_ptr(),
            table_fields=self.table_fields.data_ptr(), fwd_cols=self.fwd_cols.data_ptr(),
            thresholds=self.thresholds.data_ptr(), cb_cols=self.cb_cols.data_ptr(),
            qproj_cols=self.qproj_cols.data_ptr(), inv_rows=self.inv_rows.data_ptr(),
            fwd_limbs=None if self.fwd_limbs is None else self.fwd_limbs.data_ptr(),
            unit_pre=self.unit_pre.data_ptr(),
            center=None if self.center is None else self.center.data_ptr(),
            center_cols=None if self.center_cols is None else self.center_cols.data_ptr(),
            unit_thr=(C.c_float * 64)(*[float(x) for x in u_thr.reshape(-1)]),
            unit_aff=(C.c_float * 2)(float(u_aff[0]), float(u_aff[1])),
            wide_thr=None if self.wide_thr is None else self.wide_thr.data_ptr(),
            wide_cb=None if self.wide_cb is None else self.wide_cb.data_ptr(),
            unit_wide_thr=None if self.unit_wide_thr is None else self.unit_wide_thr.data_ptr(),
            decodable=int(self.decodable), value_decodable=int(self.value_decodable))

    @property
    def ref(self):
        return C.byref(self.struct)

    def require_value_decodable(self, what: str) -> None:
        """Decode over packed values keeps the levels of a head's columns of 5..8 bits in shared memory."""
        if not self.value_decodable:
            raise ValueError(
                f"{what}: the levels of a head's columns above 4 bits exceed the {MAX_VALUE_WIDE_LEVELS} entries the decode "
                f"kernel holds ({self.n_wide} such columns).  Fit the values with a lower cap, e.g. max_bits=4 or 6")

    def require_decodable(self, what: str) -> None:
        """The decode and score kernels keep every lookup table of a head in shared memory: 208 slots of
        16 entries, a column of w = 5..8 bits taking 2^(w-4) of them."""
        if not self.decodable:
            raise ValueError(
                f"{what}: the lookup tables of a head exceed the kernels' table memory ({self.n_wide} columns above 4 bits "
                "take 2..16 table slots each).  Fit with a lower cap, e.g. max_bits=4, for packed decode attention; "
                "compress, unpack, decompress, roundtrip and the evaluation scores work as they are")

    @property
    def record_bytes(self) -> int:
        return 4 * self.words_per_record

    @property
    def payload_bytes_per_key(self) -> float:
        """Algorithmic code bytes per key and head (sum of bits / 8, averaged over heads)."""
        return float(np.mean([l.payload_bits for l in self.layouts])) / 8.0

    @classmethod
    def from_compressors(cls, comps, device="cuda", center: torch.Tensor | None = None) -> "HeadTables":
        d = comps[0].d
        k_max = max(int(c.codebooks_padded.shape[1]) for c in comps)
        cb = torch.full((len(comps), d, k_max), float("inf"))
        for h, c in enumerate(comps):
            cb[h, :, : c.codebooks_padded.shape[1]] = c.codebooks_padded.detach().float().cpu()
        eye = torch.eye(d)
        fwd = torch.stack([(c.forward_map if c.forward_map is not None else eye).detach().float().cpu() for c in comps])
        inv = torch.stack([(c.inverse_map if c.inverse_map is not None else eye).detach().float().cpu() for c in comps])
        return cls(fwd, inv, cb, device=device, center=center)
