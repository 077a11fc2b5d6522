"""Packed record layout for per-coordinate codes of 0..4 bits, and of 5..8 bits as whole bytes
(the reference keeps dequantised floats and models no storage, per_coord_quantization.py:8).

One *record* holds the codes of one key.  Its bit string is ``32 * n_words`` long:

* the **A region** grows from bit 0: nibble-aligned *slots* of 4 bits.  A slot carries one
  4-bit code, a (3,1) pair, a (2,2) pair, (2,1,1), (1,1,1,1) or, once per record, a
  partially filled leftover.  Slot ``s`` sits at bits ``[4s, 4s+4)``.
* the **C region** grows from the last byte downwards: bytes holding two 3-bit codes and
  one 2-bit code (or two 1-bit codes) at bits 0-2, 3-5 and 6-7 of the byte.  It absorbs
  3-bit coordinates that have no 1-bit partner, so a 3.0-bit budget still packs into
  exactly 48 bytes.  C byte ``i`` is physical byte ``4*n_words - 1 - i``.

Both regions have compile-time bit positions relative to a record end, which is what lets
the decode kernel keep a record in registers and extract every lookup index with a static
shift and mask.  Each slot / sub-byte field is one *lookup*: the decode kernel turns it into
one read of a 16-entry shared-memory table holding the summed score contribution of the
coordinates in the lookup.  Lookups are numbered by physical position:

    table id = 8*w + k                      A word w (0..n_a_words-1), nibble k
    table id = 8*n_a_words + 12*iw + 3*pb + sub
                                            C word iw counted from the end (physical word
                                            n_words-1-iw), physical byte pb, sub-field 0..2

A word that is shared by the two regions is scanned by both loops; the lookups that fall
on the other region's bytes get all-zero tables.

* **Wide words** (only when some coordinate carries 5..8 bits, what the reference's default cap of
  8 gives outlier channels, per_coord_quantization.py:365-379): such a coordinate takes one byte,
  four to a word, in whole words between the A region and the C region, which then share no word.
  The decode kernels give it a table of 2^width entries behind the 16-entry ones and scan these
  words first.

*Columns* are the coordinates with >0 bits listed in ascending physical bit position, padded
with empty columns to a multiple of 16 (the tensor-core N granularity of the transform).
The compress kernel quantises column after column and appends the codes to the record in
that order; basis columns, decision thresholds and codebooks are stored in column order.

Within a page of 16 keys the records are stored word-major: word ``w`` of key ``t`` is the
uint32 at ``page_base + 4*(16*w + t)`` so that a warp reading or writing one word of 32
consecutive keys touches two full 64-byte segments.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

PAGE_TOKENS = 16
MAX_CODE_BITS = 4       # widths that share slots and 16-entry tables; wider codes take a byte each
MAX_STORED_BITS = 8     # widths a record can hold: 5..8-bit codes take a byte each ("wide" columns)
MAX_WIDE = 32           # wide columns per head
MAX_VALUE_WIDE_LEVELS = 6144   # sum of 2^width over a head's wide columns that decode over packed VALUES holds
MAX_WORDS = 16          # 128 coordinates x 4 bits
MAX_TABLES = 208        # (MAX_WORDS + 1 shared word) * 12 rounded up to a multiple of 8
TABLE_FIELDS = 4        # a lookup combines at most four coordinates (1,1,1,1)


@dataclass
class KeyLayout:
    """Everything the kernels need to know about one head's record format."""

    d: int
    bits: np.ndarray                 # (d,) int32, 0..8, coordinate order
    n_cols: int                      # active columns rounded up to a multiple of 16
    n_active: int                    # coordinates with >0 bits
    col_coord: np.ndarray            # (n_cols,) int32, -1 for padding columns
    col_width: np.ndarray            # (n_cols,) int32, 0 for padding columns
    col_bitpos: np.ndarray           # (n_cols,) int32 absolute bit position in the record
    n_words: int
    n_a_words: int                   # words scanned as nibble words
    n_c_words: int                   # words scanned as (3,3,2)-byte words, from the end
    n_tables: int
    # (n_tables, TABLE_FIELDS) int32; a field is col | width << 8 | shift << 12, or -1
    table_fields: np.ndarray
    payload_bits: int                # sum of bits
    waste_bits: int                  # pad bits inside slots / bytes (not word rounding)
    word_col_begin: np.ndarray = field(default=None)  # (n_words + 1,) first column of each word
    n_wide: int = 0                  # columns of 5..8 bits, one byte each, in whole words between the A and C regions
    wide_first: int = 0              # column index of the first of them
    decodable: bool = True           # the decode kernels' table memory holds all lookups (2^(width-4) table slots per wide column)

    @property
    def record_bytes(self) -> int:
        return 4 * self.n_words

    @property
    def page_bytes(self) -> int:
        return PAGE_TOKENS * self.record_bytes

    def descriptor(self) -> np.ndarray:
        """int32 header consumed by the C ABI: [d, n_cols, n_active, n_words, n_a_words,
        n_c_words, n_tables, payload_bits]."""
        return np.array([self.d, self.n_cols, self.n_active, self.n_words, self.n_a_words,
                         self.n_c_words, self.n_tables, self.payload_bits], dtype=np.int32)


def plan_key_layout(bits) -> KeyLayout:
    """Compose slots and bytes from a per-coordinate bit allocation (values 0..8).

    Coordinates of 5..8 bits ("wide", what the reference's cap of 8 gives outlier channels,
    per_coord_quantization.py:365-379) take one byte each, four to a word, in whole words between
    the A region and the C region; the two regions then share no word.  The decode kernels read a
    wide column through a table of 2^width entries, 2^(width - 4) of their ``MAX_TABLES`` slots of 16
    entries (``decodable``: the slots of all columns fit).  Raises ``ValueError`` when the record
    does not hold the allocation: more than ``MAX_WIDE`` wide coordinates, or more than 16 words."""
    bits = np.asarray(bits).astype(np.int64).reshape(-1)
    d = int(bits.shape[0])
    if d % 16 != 0 or d > 128:
        raise ValueError(f"head_dim must be a multiple of 16 and at most 128, got {d}")
    if bits.min() < 0 or bits.max() > MAX_STORED_BITS:
        raise ValueError(
            f"the packed GPU path stores 0..{MAX_STORED_BITS} bits per coordinate, got range "
            f"[{int(bits.min())}, {int(bits.max())}]")
    wide = [int(j) for j in np.nonzero(bits > MAX_CODE_BITS)[0]]
    if len(wide) > MAX_WIDE:
        raise ValueError(f"{len(wide)} coordinates carry more than {MAX_CODE_BITS} bits; a record holds at most {MAX_WIDE} such")
    by_width = {w: [int(j) for j in np.nonzero(bits == w)[0]] for w in (1, 2, 3, 4)}
    l4, l3, l2, l1 = by_width[4], by_width[3], by_width[2], by_width[1]

    a_slots: list[list[tuple[int, int]]] = []
    c_bytes: list[list[tuple[int, int]]] = []
    for j in l4:
        a_slots.append([(j, 4)])
    while l3 and l1:                                   # (3,1) pairs
        a_slots.append([(l3.pop(0), 3), (l1.pop(0), 1)])
    while len(l3) >= 2 and (l2 or len(l1) >= 2):        # (3,3,2) or (3,3,1,1) bytes
        byte = [(l3.pop(0), 3), (l3.pop(0), 3)]
        if l2:
            byte.append((l2.pop(0), 2))
        else:
            byte.extend([(l1.pop(0), 1), (l1.pop(0), 1)])
        c_bytes.append(byte)
    for j in l3:                                       # 3-bit codes nothing can complete
        a_slots.append([(j, 3)])
    l3 = []
    while len(l2) >= 2:
        a_slots.append([(l2.pop(0), 2), (l2.pop(0), 2)])
    if l2:
        slot = [(l2.pop(0), 2)]
        while l1 and sum(w for _, w in slot) < 4:
            slot.append((l1.pop(0), 1))
        a_slots.append(slot)
    while l1:
        slot = []
        while l1 and len(slot) < 4:
            slot.append((l1.pop(0), 1))
        a_slots.append(slot)

    n_a, n_c = len(a_slots), len(c_bytes)
    n_a_words = -(-n_a // 8)
    n_c_words = -(-n_c // 4)
    n_w_words = -(-len(wide) // 4)
    n_words = max(1, -(-(4 * n_a + 8 * n_c) // 32)) if not wide else n_a_words + n_w_words + n_c_words
    if n_words > MAX_WORDS:
        raise ValueError("record exceeds 16 words")
    n_tables = 8 * n_a_words + 12 * n_c_words
    rec_bytes = 4 * n_words

    cols: list[tuple[int, int, int]] = []             # (coord, width, bitpos) ascending bitpos
    table_fields = np.full((max(n_tables, 1), TABLE_FIELDS), -1, dtype=np.int32)
    for s, slot in enumerate(a_slots):
        shift = 0
        for f, (j, w) in enumerate(slot):
            table_fields[s, f] = len(cols) | (w << 8) | (shift << 12)
            cols.append((j, w, 4 * s + shift))
            shift += w
    wide_first = len(cols)
    for i, j in enumerate(wide):                       # one byte each, from the first word after the A region
        cols.append((j, int(bits[j]), 32 * n_a_words + 8 * i))
    for i in range(n_c - 1, -1, -1):                   # ascending physical byte
        phys_byte = rec_bytes - 1 - i
        iw, pb = (n_words - 1) - phys_byte // 4, phys_byte % 4
        base_tab = 8 * n_a_words + 12 * iw + 3 * pb
        byte = c_bytes[i]
        subs = [[byte[0]], [byte[1]], byte[2:]]
        for sub, (fields, off) in enumerate(zip(subs, (0, 3, 6))):
            shift = 0
            for f, (j, w) in enumerate(fields):
                table_fields[base_tab + sub, f] = len(cols) | (w << 8) | (shift << 12)
                cols.append((j, w, 8 * phys_byte + off + shift))
                shift += w
    n_active = len(cols)
    assert n_active == int((bits > 0).sum())
    n_cols = max(16, -(-n_active // 16) * 16)
    col_coord = np.full(n_cols, -1, dtype=np.int32)
    col_width = np.zeros(n_cols, dtype=np.int32)
    col_bitpos = np.zeros(n_cols, dtype=np.int32)
    for c, (j, w, p) in enumerate(cols):
        col_coord[c], col_width[c], col_bitpos[c] = j, w, p
    if n_active:
        assert np.all(np.diff(col_bitpos[:n_active]) > 0), "columns must ascend in bit position"
        col_bitpos[n_active:] = 32 * n_words
    word_col_begin = np.searchsorted(col_bitpos[:n_active], 32 * np.arange(n_words + 1)).astype(np.int32)
    payload = int(bits.sum())
    # a wide column's table of 2^width entries takes the room of 2 .. 16 of the 16-entry ones, behind them
    n_tables_all = n_tables + sum(1 << (int(bits[j]) - 4) for j in wide)
    decodable = n_tables_all <= MAX_TABLES
    return KeyLayout(
        d=d, bits=bits.astype(np.int32), n_cols=n_cols, n_active=n_active, col_coord=col_coord,
        col_width=col_width, col_bitpos=col_bitpos, n_words=n_words, n_a_words=n_a_words,
        n_c_words=n_c_words, n_tables=n_tables_all if decodable else n_tables, decodable=decodable,
        table_fields=table_fields[:max(n_tables, 1)],
        payload_bits=payload, waste_bits=4 * n_a + 8 * n_c + 8 * len(wide) - payload, word_col_begin=word_col_begin,
        n_wide=len(wide), wide_first=wide_first)


def decision_thresholds(codebook_rows: np.ndarray, widths: np.ndarray, max_levels: int = 16) -> np.ndarray:
    """Exact fp32 decision thresholds of the reference's nearest-centroid rule.

    The reference picks ``argmin_l |x - cb[l]|`` in fp32 with the first index winning ties
    (per_coord_quantization.py:156-157).  Between two neighbouring centroids ``a < b`` the
    fp32 predicate ``|x - b| < |x - a|`` is monotone in ``x`` (one rounded difference never
    decreases, the other never increases), so there is a smallest fp32 ``x`` for which the
    upper centroid wins.  That value is found by bisection over fp32 bit patterns, which
    makes ``code = #{l : x >= thr[l]}`` reproduce the reference code for every finite ``x``
    whose distances to the centroids are distinguishable in fp32.

    ``codebook_rows``: (n, L) fp32 ascending centroids (unused tail arbitrary), L = ``max_levels``
    (16, or 256 for the wide columns); ``widths``: (n,) code widths.  Returns (n, L - 1) fp32,
    unused entries ``+inf``.
    """
    L = int(max_levels)
    cb = np.asarray(codebook_rows, dtype=np.float32)
    widths = np.asarray(widths).astype(np.int64).reshape(-1)
    n = cb.shape[0]
    levels = (1 << widths)[:, None]                           # (n, 1)
    valid = np.arange(L - 1)[None, :] < (levels - 1)          # (n, L - 1)
    if cb.shape[1] < L:
        cb = np.concatenate([cb, np.zeros((n, L - cb.shape[1]), np.float32)], axis=1)
    a = np.where(valid, cb[:, :L - 1], np.float32(0.0)).astype(np.float32)
    b = np.where(valid, cb[:, 1:L], np.float32(1.0)).astype(np.float32)

    def to_ord(x: np.ndarray) -> np.ndarray:                  # monotone int64 key of fp32 values
        u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.int64)
        return np.where(u & 0x80000000, 0x80000000 - u, u)

    def from_ord(o: np.ndarray) -> np.ndarray:
        u = np.where(o < 0, 0x80000000 - o, o).astype(np.uint32)
        return u.view(np.float32)

    lo, hi = to_ord(a), to_ord(b)                             # pred(lo) False, pred(hi) True
    while np.any(hi - lo > 1):
        mid = (lo + hi) // 2
        x = from_ord(mid)
        with np.errstate(invalid="ignore", over="ignore"):
            pred = np.abs(x - b) < np.abs(x - a)
        hi = np.where(pred, mid, hi)
        lo = np.where(pred, lo, mid)
    return np.where(valid, from_ord(hi), np.float32(np.inf)).astype(np.float32)


BUCKETS = 128


def unit_quantiser_tables(unit_centroids: dict):
    """Shared quantiser tables of the tensor-core compress kernel, one set for all columns.

    The kernel transforms keys with basis columns scaled by 1 / sigma_c, so every transformed
    coordinate is quantised against the *unit* Lloyd-Max levels of its width: the decision thresholds
    of a column, sigma_c * u_l up to a rounding, become u_l for every column of that width (the
    change moves a code only when the value lies within ~1e-7 relative of a threshold).  Returns

    * ``thr``  float32 (4, 16): exact fp32 decision thresholds of the unit codebook of width 1..4
      (``decision_thresholds``), ``+inf`` padded;
    * ``pre``  uint8 (4, 128): for one common grid of 128 cells over the value axis, a lower bound of
      the code (at most one short) with ``16 * (width - 1)`` added, i.e. the index into ``thr``
      flattened at which the one exact comparison is made;
    * ``aff``  float32 (2,): the kernel maps a value to one of ``BUCKETS`` equal cells with one fused
      multiply-add, ``y = x * aff[0] + aff[1]`` (aff[1] carries the 2**23 bias that leaves the cell index
      in the low mantissa bits, after clamping).  The lower bound read from ``pre`` is valid because
      neighbouring thresholds are at least three cells apart: one cell of slack on either side absorbs
      any rounding difference between this host arithmetic and the device's.

    ``unit_centroids[b]`` are the unit-variance centroids of width b (ascending)."""
    thr = np.full((4, 16), np.inf, np.float32)
    for b in range(1, 5):
        rows = np.zeros((1, 16), np.float32)
        rows[0, : 2 ** b] = np.asarray(unit_centroids[b], dtype=np.float32)
        thr[b - 1, : 2 ** b - 1] = decision_thresholds(rows, np.array([b]))[0, : 2 ** b - 1]
    t4 = thr[3, :15].astype(np.float64)
    step = (t4[-1] - t4[0]) / (BUCKETS - 8)
    inv_step = np.float32(1.0 / step)
    off = np.float32(-(t4[0] - 4.0 * step) * float(inv_step) + 2.0 ** 23)
    pre = np.zeros((4, BUCKETS), np.uint8)
    cells = np.arange(BUCKETS)
    for b in range(1, 5):
        n_thr = 2 ** b - 1
        y = np.float32(thr[b - 1, :n_thr].astype(np.float64) * float(inv_step) + float(off))
        y = np.minimum(np.maximum(y, np.float32(2.0 ** 23)), np.float32(2.0 ** 23 + BUCKETS - 1))
        cell = y.view(np.uint32).astype(np.int64) & (BUCKETS - 1)
        if n_thr > 1 and np.any(np.diff(cell) < 3):
            raise AssertionError("unit thresholds too close for the cell grid")
        lower = (cell[None, :] <= (cells[:, None] - 2)).sum(-1)          # thresholds safely below the cell
        pre[b - 1] = (16 * (b - 1) + np.minimum(lower, n_thr - 1 if n_thr > 1 else 0)).astype(np.uint8)
    return thr, pre, np.array([inv_step, off], np.float32)
