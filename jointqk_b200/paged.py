"""Paged storage for packed keys and bf16 values, and the calls that fill and read it.

Everything here is plumbing around the C ABI: torch owns the device memory and the stream,
the kernels do the work.  The reference has no counterpart for the storage itself (it keeps
dequantised floats in the HF cache, experiments/stage1/toolkit/jointqk_press.py:306-307).
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _native
from .layout import PAGE_TOKENS
from .tables import HeadTables


def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def pages_for(n_tokens: int) -> int:
    return (int(n_tokens) + PAGE_TOKENS - 1) // PAGE_TOKENS


@dataclass
class PackedKeys:
    """Result of ``compress``: packed code pages plus the page table that orders them."""

    tables: HeadTables
    k_pool: torch.Tensor        # uint32 (int32 storage) [n_pages, H, words_per_record, 16]
    page_table: torch.Tensor    # int32 [n_seqs, max_pages]
    n_tokens: torch.Tensor      # int32 [n_seqs] on device
    lengths: list[int]          # host copy of n_tokens
    status: torch.Tensor        # int32 [1] device status word
    leading_shape: tuple = ()   # shape to restore on decompress (compressor API)

    @property
    def n_seqs(self) -> int:
        return len(self.lengths)

    @property
    def max_tokens(self) -> int:
        return max(self.lengths) if self.lengths else 0

    @property
    def n_pages(self) -> int:
        return int(self.k_pool.shape[0])

    def nbytes_payload(self) -> int:
        return int(sum(self.lengths) * self.tables.n_heads * self.tables.payload_bytes_per_key)


def alloc_k_pool(tables: HeadTables, n_pages: int) -> torch.Tensor:
    return torch.zeros((n_pages, tables.n_heads, tables.words_per_record, PAGE_TOKENS),
                       dtype=torch.int32, device=tables.device)


def alloc_v_pool(tables: HeadTables, n_pages: int) -> torch.Tensor:
    """bf16 value pool, (n_pages, H, d * 16): a (page, head) block is dims-major, see ``v_slot_offsets``."""
    return torch.zeros((n_pages, tables.n_heads, tables.d * PAGE_TOKENS), dtype=torch.bfloat16,
                       device=tables.device)


_V_OFFSETS: dict = {}


def v_slot_offsets(d: int, device) -> torch.Tensor:
    """int64 (16, d): element offset of (slot, dim) inside a (page, head) block of the V pool.

    The block is stored dims-major -- 32 bytes (16 keys) per dim -- because that is the operand
    layout of the decode kernel's tensor-core product: a 16-dim x 16-key tile is one ldmatrix.
    The two 16-byte halves of a row are swapped on dims 4..7 (mod 8) so that the eight rows an
    ldmatrix phase touches fall into eight different shared-memory bank groups."""
    key = (d, str(device))
    if key not in _V_OFFSETS:
        slot = torch.arange(PAGE_TOKENS).view(PAGE_TOKENS, 1)
        dim = torch.arange(d).view(1, d)
        off = dim * PAGE_TOKENS + ((((slot >> 3) ^ ((dim >> 2) & 1)) << 3) + (slot & 7))
        _V_OFFSETS[key] = off.to(device)
    return _V_OFFSETS[key]


def sequential_page_table(lengths: list[int], device, first_page: int = 0) -> tuple[torch.Tensor, int]:
    """Page table that lays the sequences out one after another; returns (table, pages used)."""
    counts = [pages_for(n) for n in lengths]
    width = max(1, max(counts) if counts else 1)
    table = torch.zeros((max(1, len(lengths)), width), dtype=torch.int32)
    nxt = first_page
    for s, c in enumerate(counts):
        table[s, :c] = torch.arange(nxt, nxt + c, dtype=torch.int32)
        nxt += c
    return table.to(device), nxt - first_page


def check_status(status: torch.Tensor) -> None:
    """Raise if a kernel flagged a bad page index, an over-long length or an expired wait
    (synchronises)."""
    v = int(status.item())
    if v & _native.STATUS_BAD_PAGE:
        raise RuntimeError("jointqk_b200: page table holds an index outside the pool")
    if v & _native.STATUS_BAD_LENGTH:
        raise RuntimeError("jointqk_b200: a sequence length reaches past what the call was sized for")
    if v & _native.STATUS_WAIT_EXPIRED:
        raise RuntimeError("jointqk_b200: a bounded device-side wait expired")


def store_values_into(values: torch.Tensor, n_tokens: torch.Tensor, max_tokens: int, page_table: torch.Tensor,
                      v_pool: torch.Tensor, status: torch.Tensor, seq_starts: torch.Tensor | None = None) -> None:
    """values (n_seqs, H, S, d) with d contiguous -> bf16 V pages (one kernel pass, no torch indexing)."""
    if values.dim() != 4 or values.stride(3) != 1:
        values = values.contiguous()
    if values.dtype not in (torch.float32, torch.bfloat16, torch.float16):
        values = values.float()
    n_seqs, H, _, d = values.shape
    if v_pool.dtype != torch.bfloat16 or v_pool.shape[1] != H or v_pool.shape[2] != d * PAGE_TOKENS:
        raise ValueError(f"v_pool must be bf16 (n_pages, {H}, {d * PAGE_TOKENS})")
    _native.check(_native.lib.jqk_store_values_paged(
        values.data_ptr(), _native.torch_dtype_code(values.dtype), values.stride(0), values.stride(1),
        values.stride(2), n_seqs, H, d, n_tokens.data_ptr(), _ptr(seq_starts), int(max_tokens),
        page_table.data_ptr(), page_table.stride(0), int(v_pool.shape[0]), v_pool.data_ptr(),
        status.data_ptr(), _stream_ptr(v_pool.device)))


def compress_into(tables: HeadTables, keys: torch.Tensor, n_tokens: torch.Tensor, max_tokens: int,
                  page_table: torch.Tensor, k_pool: torch.Tensor, status: torch.Tensor,
                  seq_starts: torch.Tensor | None = None) -> None:
    """keys: (n_seqs, H, S, d) with d contiguous; writes packed records into ``k_pool``."""
    if keys.dim() != 4 or keys.shape[1] != tables.n_heads or keys.shape[3] != tables.d:
        raise ValueError(f"keys must be (n_seqs, {tables.n_heads}, S, {tables.d}), got {tuple(keys.shape)}")
    if keys.stride(3) != 1:
        keys = keys.contiguous()
    if keys.device != tables.device:
        raise ValueError("keys and tables live on different devices")
    _native.check(_native.lib.jqk_compress_paged(
        tables.ref, keys.data_ptr(), _native.torch_dtype_code(keys.dtype),
        keys.stride(0), keys.stride(1), keys.stride(2), keys.shape[0], n_tokens.data_ptr(),
        _ptr(seq_starts), int(max_tokens), page_table.data_ptr(), page_table.stride(0),
        int(k_pool.shape[0]), k_pool.data_ptr(), status.data_ptr(), _stream_ptr(tables.device)))


def compress(tables: HeadTables, keys: torch.Tensor, lengths: list[int] | None = None) -> PackedKeys:
    """Compress (n_seqs, H, S, d) keys into freshly allocated sequential pages."""
    n_seqs, _, S, _ = keys.shape
    lengths = [S] * n_seqs if lengths is None else [int(x) for x in lengths]
    dev = tables.device
    page_table, used = sequential_page_table(lengths, dev)
    k_pool = alloc_k_pool(tables, max(1, used))
    n_tok = torch.tensor(lengths if lengths else [0], dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    if n_seqs and max(lengths) > 0:
        compress_into(tables, keys, n_tok, max(lengths), page_table, k_pool, status)
    return PackedKeys(tables, k_pool, page_table, n_tok, lengths, status)


def decompress(packed: PackedKeys) -> torch.Tensor:
    """fp32 (n_seqs, H, max_tokens, d) reconstruction; rows past a sequence's length are 0."""
    t = packed.tables
    out = torch.zeros((packed.n_seqs, t.n_heads, packed.max_tokens, t.d), dtype=torch.float32, device=t.device)
    if packed.n_seqs and packed.max_tokens:
        _native.check(_native.lib.jqk_decompress_paged(
            t.ref, packed.n_seqs, packed.n_tokens.data_ptr(), None, packed.max_tokens,
            packed.page_table.data_ptr(), packed.page_table.stride(0), packed.n_pages,
            packed.k_pool.data_ptr(), out.data_ptr(), packed.status.data_ptr(), _stream_ptr(t.device)))
    return out


def unpack_codes(packed: PackedKeys) -> torch.Tensor:
    """uint8 (n_seqs, H, max_tokens, d) codes in coordinate order."""
    t = packed.tables
    out = torch.zeros((packed.n_seqs, t.n_heads, packed.max_tokens, t.d), dtype=torch.uint8, device=t.device)
    if packed.n_seqs and packed.max_tokens:
        _native.check(_native.lib.jqk_unpack_codes(
            t.ref, packed.n_seqs, packed.n_tokens.data_ptr(), packed.max_tokens,
            packed.page_table.data_ptr(), packed.page_table.stride(0), packed.n_pages,
            packed.k_pool.data_ptr(), out.data_ptr(), packed.status.data_ptr(), _stream_ptr(t.device)))
    return out


def score(packed: PackedKeys, q: torch.Tensor, decode_tables: bool = False) -> torch.Tensor:
    """Logits ``q . k_hat / sqrt(d)``: q (n_seqs, Hq, n_queries, d) -> (n_seqs, Hq, n_queries, max_tokens).

    ``decode_tables=False`` sums in fp32 (evaluation metrics); ``True`` scores through the 16-bit
    fixed-point lookup tables exactly as the decode kernel does."""
    t = packed.tables
    if q.dim() != 4 or q.shape[0] != packed.n_seqs or q.shape[3] != t.d:
        raise ValueError(f"q must be ({packed.n_seqs}, Hq, n_queries, {t.d}), got {tuple(q.shape)}")
    if q.shape[1] % t.n_heads:
        raise ValueError(f"Cannot group {q.shape[1]} query heads into {t.n_heads} KV heads evenly.")
    q = q.contiguous()
    if not t.decodable:
        # more wide columns than the score kernel has table memory for: score against the reconstruction
        # (fp32 on the device), which is what the reference's metric does (eval.py:20-21)
        if decode_tables:
            t.require_decodable("scoring through the decode tables")
        k_hat = decompress(packed)                                            # (n_seqs, H, T, d)
        g = q.shape[1] // t.n_heads
        qg = q.float().to(t.device).view(packed.n_seqs, t.n_heads, g, q.shape[2], t.d)
        s = torch.einsum("shgqd,shtd->shgqt", qg, k_hat) / t.d ** 0.5
        s = s.reshape(packed.n_seqs, q.shape[1], q.shape[2], packed.max_tokens)
        pos = torch.arange(packed.max_tokens, device=t.device)
        return s.masked_fill(pos[None, None, None, :] >= packed.n_tokens.view(-1, 1, 1, 1), 0.0)
    out = torch.zeros((packed.n_seqs, q.shape[1], q.shape[2], packed.max_tokens), dtype=torch.float32, device=t.device)
    if out.numel():
        _native.check(_native.lib.jqk_score_paged(
            t.ref, int(decode_tables), q.data_ptr(), _native.torch_dtype_code(q.dtype), packed.n_seqs, q.shape[1], q.shape[2],
            packed.n_tokens.data_ptr(), packed.max_tokens, packed.page_table.data_ptr(),
            packed.page_table.stride(0), packed.n_pages, packed.k_pool.data_ptr(), out.data_ptr(),
            packed.status.data_ptr(), _stream_ptr(t.device)))
    return out


class DecodeWorkspace:
    """Zero-initialised scratch for split-KV decode; reusable across calls on one stream."""

    def __init__(self, n_seqs: int, n_q_heads: int, n_kv_heads: int, max_splits: int, device) -> None:
        nbytes = int(_native.lib.jqk_decode_workspace_bytes(n_seqs, n_q_heads, n_kv_heads, max_splits))
        self.max_splits, self.n_seqs, self.n_q_heads = max_splits, n_seqs, n_q_heads
        self.buf = torch.zeros(max(nbytes, 16), dtype=torch.uint8, device=device)


def default_split(n_seqs: int, n_q_heads: int, n_kv_heads: int, max_seq_len: int) -> int:
    return int(_native.lib.jqk_decode_default_split(n_seqs, n_q_heads, n_kv_heads, max_seq_len))


def split_for_lengths(lengths: list[int], n_q_heads: int, n_kv_heads: int) -> int:
    """Keys per thread block for a batch with these context lengths (fits the block count to waves)."""
    import ctypes

    arr = (ctypes.c_int32 * max(1, len(lengths)))(*[int(n) for n in lengths])
    return int(_native.lib.jqk_decode_split_for_lengths(arr, len(lengths), n_q_heads, n_kv_heads))


def decode_attend(tables: HeadTables, q: torch.Tensor, seq_lens: torch.Tensor, max_seq_len: int,
                  page_table: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                  out: torch.Tensor, workspace: DecodeWorkspace | None, status: torch.Tensor,
                  tokens_per_split: int = 0, v_tables: HeadTables | None = None) -> torch.Tensor:
    """One decode step for one layer.  q bf16 (n_seqs, Hq, d); out fp32 or bf16 (n_seqs, Hq, d).
    With ``v_tables`` the value pool holds packed codes of that compressor (int32 storage)."""
    if q.dtype != torch.bfloat16 or q.dim() != 3 or not q.is_contiguous():
        raise ValueError("q must be a contiguous bf16 (n_seqs, n_q_heads, d) tensor")
    tables.require_decodable("decode attention")
    if v_tables is not None:
        v_tables.require_value_decodable("decode attention over packed values")
        if v_pool.dtype != torch.int32:
            raise ValueError("a packed value pool is int32 storage")
        if out.shape != q.shape or not out.is_contiguous():
            raise ValueError("out must be contiguous with the shape of q")
        ws_ptr, ws_bytes = (None, 0) if workspace is None else (workspace.buf.data_ptr(), workspace.buf.numel())
        _native.check(_native.lib.jqk_decode_attend_packed_values(
            tables.ref, v_tables.ref, q.data_ptr(), q.shape[0], q.shape[1], seq_lens.data_ptr(), int(max_seq_len),
            int(tokens_per_split), page_table.data_ptr(), page_table.stride(0), int(k_pool.shape[0]),
            k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(), _native.torch_dtype_code(out.dtype),
            ws_ptr, ws_bytes, status.data_ptr(), _stream_ptr(tables.device)))
        return out
    if v_pool.dtype != torch.bfloat16:
        raise ValueError("v_pool must be bf16")
    if out.shape != q.shape or not out.is_contiguous():
        raise ValueError("out must be contiguous with the shape of q")
    ws_ptr, ws_bytes = (None, 0) if workspace is None else (workspace.buf.data_ptr(), workspace.buf.numel())
    _native.check(_native.lib.jqk_decode_attend(
        tables.ref, q.data_ptr(), q.shape[0], q.shape[1], seq_lens.data_ptr(), int(max_seq_len),
        int(tokens_per_split), page_table.data_ptr(), page_table.stride(0), int(k_pool.shape[0]),
        k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(), _native.torch_dtype_code(out.dtype),
        ws_ptr, ws_bytes, status.data_ptr(), _stream_ptr(tables.device)))
    return out


def decode_append_attend(tables: HeadTables, q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor,
                         seq_lens: torch.Tensor, max_seq_len: int, page_table: torch.Tensor, k_pool: torch.Tensor,
                         v_pool: torch.Tensor, out: torch.Tensor, workspace: DecodeWorkspace, status: torch.Tensor,
                         tokens_per_split: int = 0, own_key_exact: bool = False,
                         v_tables: HeadTables | None = None) -> torch.Tensor:
    """One generate step in one launch: the rows k_new / v_new (n_seqs, H, 1, d) or (n_seqs, H, d) go
    to position ``seq_lens[s]`` of every sequence (pages already in the table), the step attends
    over ``seq_lens[s] + 1`` keys (``max_seq_len`` covers that) and ``seq_lens`` is advanced on the
    device.  With ``v_tables`` the value row is packed as well.  ``own_key_exact``: the new key is scored from its exact values in
    this step (and from its codes afterwards), the semantics of the reference's Mode B."""
    if q.dtype != torch.bfloat16 or q.dim() != 3 or not q.is_contiguous():
        raise ValueError("q must be a contiguous bf16 (n_seqs, n_q_heads, d) tensor")
    if v_pool.dtype != (torch.bfloat16 if v_tables is None else torch.int32):
        raise ValueError("the value pool is bf16, or int32 storage of packed codes when v_tables is given")
    tables.require_decodable("decode attention")
    if v_tables is not None:
        v_tables.require_value_decodable("decode attention over packed values")
    if out.shape != q.shape or not out.is_contiguous():
        raise ValueError("out must be contiguous with the shape of q")
    if k_new.dim() == 4:
        if k_new.shape[2] != 1 or v_new.shape[2] != 1:
            raise ValueError("one new token per sequence")
        k_new, v_new = k_new[:, :, 0], v_new[:, :, 0]
    n, h, d = k_new.shape
    if (n, h, d) != (q.shape[0], tables.n_heads, tables.d) or v_new.shape != k_new.shape:
        raise ValueError(f"k_new / v_new must be ({q.shape[0]}, {tables.n_heads}, {tables.d}) rows")
    ok = (torch.float32, torch.bfloat16, torch.float16)
    if k_new.dtype not in ok or v_new.dtype not in ok:
        raise ValueError("k_new and v_new must be fp32, bf16 or fp16")
    if k_new.stride(2) != 1 or v_new.stride(2) != 1:
        raise ValueError("rows must be contiguous in their last dimension")
    if seq_lens.dtype != torch.int32:
        raise ValueError("seq_lens must be int32")
    fn = _native.lib.jqk_decode_append_attend if v_tables is None else _native.lib.jqk_decode_append_attend_packed_values
    head = (tables.ref,) if v_tables is None else (tables.ref, v_tables.ref)
    _native.check(fn(
        *head, q.data_ptr(), k_new.data_ptr(), v_new.data_ptr(), _native.torch_dtype_code(k_new.dtype),
        _native.torch_dtype_code(v_new.dtype), k_new.stride(0), k_new.stride(1), v_new.stride(0), v_new.stride(1), n, q.shape[1], seq_lens.data_ptr(),
        int(max_seq_len), int(tokens_per_split), page_table.data_ptr(), page_table.stride(0), int(k_pool.shape[0]),
        k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(), _native.torch_dtype_code(out.dtype),
        1 if own_key_exact else 0, workspace.buf.data_ptr(), workspace.buf.numel(), status.data_ptr(),
        _stream_ptr(tables.device)))
    return out


class PagePool:
    """Physical pages of one layer (packed K and bf16 V side by side, one index space) with a free
    list.  ``take`` hands out pages; when the list runs dry the pool grows: larger tensors are
    allocated, the old contents copied over and the old tensors dropped, so page indices stay valid
    and only the base pointers change (``generation`` counts the moves)."""

    def __init__(self, tables: HeadTables, n_pages: int, growth: float = 1.5, v_tables: HeadTables | None = None) -> None:
        self.tables = tables
        self.v_tables = v_tables          # values as packed codes of this compressor instead of bf16
        self.growth = float(growth)
        n_pages = max(1, int(n_pages))
        self.k_pool = alloc_k_pool(tables, n_pages)
        self.v_pool = self._alloc_v(n_pages)
        self._free = list(range(n_pages - 1, -1, -1))   # pop() hands out ascending indices
        self.generation = 0

    def _alloc_v(self, n_pages: int) -> torch.Tensor:
        return alloc_v_pool(self.tables, n_pages) if self.v_tables is None else alloc_k_pool(self.v_tables, n_pages)

    @property
    def n_pages(self) -> int:
        return int(self.k_pool.shape[0])

    @property
    def n_free(self) -> int:
        return len(self._free)

    def grow(self, n_pages: int) -> None:
        old = self.n_pages
        if n_pages <= old:
            return
        k_new, v_new = alloc_k_pool(self.tables, n_pages), self._alloc_v(n_pages)
        k_new[:old].copy_(self.k_pool)
        v_new[:old].copy_(self.v_pool)
        self.k_pool, self.v_pool = k_new, v_new
        self._free = list(range(n_pages - 1, old - 1, -1)) + self._free
        self.generation += 1

    def take(self, n: int) -> list[int]:
        if n > len(self._free):
            self.grow(max(int(self.n_pages * self.growth) + 1, self.n_pages + n - len(self._free)))
        return [self._free.pop() for _ in range(n)]

    def give_back(self, pages: list[int]) -> None:
        self._free.extend(sorted((int(p) for p in pages), reverse=True))


class PagedKVCache:
    """Packed-K / bf16-V paged cache of one layer for a batch of sequences.

    ``prefill`` (and ``append``, the same call for the newest tokens of a generate loop;
    jointqk_press.py:298-304 compresses only those each step) allocates pages on demand from a
    ``PagePool``, compresses the keys into them and stores the values with one kernel pass each;
    ``decode`` runs the fused attention kernel; ``release`` returns a sequence's pages to the pool.
    ``max_lengths`` reserves pages up front (sequence after sequence, which is all the fixed-size
    workloads need); with ``n_seqs`` alone the cache starts empty and grows, and so does the pool.

    With ``v_tables`` (the head tables of a value-side compressor, centred or not) the values are
    stored as packed codes as well: ``prefill`` compresses them with the same kernel as the keys and
    ``decode`` dequantises them tile by tile inside the attention kernel.
    """

    def __init__(self, tables: HeadTables, max_lengths: list[int] | None = None, *, n_seqs: int | None = None,
                 pool: PagePool | None = None, initial_pages: int = 0, v_tables: HeadTables | None = None) -> None:
        self.tables = tables
        self.v_tables = v_tables if pool is None else pool.v_tables
        dev = tables.device
        if max_lengths is None:
            if n_seqs is None:
                raise ValueError("give max_lengths (reserve) or n_seqs (grow on demand)")
            max_lengths = [0] * int(n_seqs)
        n = len(max_lengths)
        counts = [pages_for(x) for x in max_lengths]
        self.pool = pool if pool is not None else PagePool(tables, max(1, sum(counts), int(initial_pages)), v_tables=v_tables)
        self._pages: list[list[int]] = [self.pool.take(c) for c in counts]
        width = max(1, max(counts) if counts else 1)
        table = torch.zeros((max(1, n), width), dtype=torch.int32)
        for s, pg in enumerate(self._pages):
            table[s, :len(pg)] = torch.tensor(pg, dtype=torch.int32)
        self.page_table = table.to(dev)
        self.lengths = [0] * n
        self.seq_lens = torch.zeros(max(1, n), dtype=torch.int32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self._ws: DecodeWorkspace | None = None
        self._host_step: dict | None = None
        self._host_call: dict | None = None
        self._epoch = 0      # bumped whenever lengths or pages change: cached host-step state compares one integer

    # the pools belong to the PagePool (they move when it grows)
    @property
    def k_pool(self) -> torch.Tensor:
        return self.pool.k_pool

    @property
    def v_pool(self) -> torch.Tensor:
        return self.pool.v_pool

    @property
    def n_pages(self) -> int:
        return self.pool.n_pages

    @property
    def capacity(self) -> list[int]:
        return [len(pg) * PAGE_TOKENS for pg in self._pages]

    def reserve(self, seq: int, n_tokens: int) -> None:
        """Make sure sequence ``seq`` owns pages for ``n_tokens`` tokens in all."""
        need = pages_for(n_tokens) - len(self._pages[seq])
        if need <= 0:
            return
        self._gen_budget = 0
        self._epoch += 1
        have = len(self._pages[seq])
        new = self.pool.take(need)
        self._pages[seq].extend(new)
        if have + need > self.page_table.shape[1]:        # widen the table (amortised doubling)
            width = max(have + need, 2 * self.page_table.shape[1])
            wider = torch.zeros((self.page_table.shape[0], width), dtype=torch.int32, device=self.page_table.device)
            wider[:, : self.page_table.shape[1]] = self.page_table
            self.page_table = wider
            self._host_step = self._host_call = None
        self.page_table[seq, have:have + need] = torch.tensor(new, dtype=torch.int32, device=self.page_table.device)

    def release(self, seq: int) -> None:
        """Forget sequence ``seq`` and return its pages to the pool."""
        self._gen_budget = 0
        self._epoch += 1
        self.pool.give_back(self._pages[seq])
        self._pages[seq] = []
        self.lengths[seq] = 0
        self.seq_lens[seq] = 0

    def prefill(self, keys: torch.Tensor, values: torch.Tensor, lengths: list[int] | None = None) -> None:
        """keys/values (n_seqs, H, S, d).  Appends ``lengths[s]`` tokens to every sequence: one
        compress launch for the keys, one store launch for the values."""
        n_seqs, H, S, d = keys.shape
        lengths = [S] * n_seqs if lengths is None else [int(x) for x in lengths]
        dev = self.tables.device
        for s, n in enumerate(lengths):
            self.reserve(s, self.lengths[s] + n)
        starts = torch.tensor(self.lengths[:n_seqs], dtype=torch.int32, device=dev)
        n_tok = torch.tensor(lengths, dtype=torch.int32, device=dev)
        if max(lengths) > 0:
            compress_into(self.tables, keys, n_tok, max(lengths), self.page_table, self.k_pool, self.status, starts)
            self._store_values(values.to(dev), n_tok, max(lengths), starts)
        for s, n in enumerate(lengths):
            self.lengths[s] += n
        self._epoch += 1
        self.seq_lens[: len(self.lengths)] = torch.tensor(self.lengths, dtype=torch.int32, device=dev)

    def append(self, keys: torch.Tensor, values: torch.Tensor) -> None:
        """One new token for every sequence of the cache: keys/values (n_seqs, H, 1, d).  The step of
        a generate loop: nothing is copied from the host (the current lengths on the device are the
        destinations, and they are advanced on the device), pages are taken from the pool only when a
        sequence crosses a page boundary."""
        n = len(self.lengths)
        if keys.shape[0] != n or keys.shape[2] != 1:
            return self.prefill(keys, values)
        for s in range(n):
            self.reserve(s, self.lengths[s] + 1)
        if getattr(self, "_ones", None) is None or self._ones.numel() != n:
            self._ones = torch.ones(n, dtype=torch.int32, device=self.tables.device)
        compress_into(self.tables, keys, self._ones, 1, self.page_table, self.k_pool, self.status, self.seq_lens)
        self._store_values(values, self._ones, 1, self.seq_lens)
        self.seq_lens[:n] += 1
        for s in range(n):
            self.lengths[s] += 1
        self._epoch += 1

    RESERVE_AHEAD = 64   # tokens of page capacity the fused generate step keeps ahead of the context

    def generate_step(self, k_new: torch.Tensor, v_new: torch.Tensor, q: torch.Tensor,
                      fused_append: bool = True, own_key_exact: bool = False) -> torch.Tensor:
        """One step of a generate loop: append the newest token of every sequence (K compress, V store,
        lengths advanced on the device), then attend.  That is one kernel launch, which reads the rows
        in place (``jqk_decode_append_attend``, or its packed-values form).  ``fused_append=False``:
        the separate compress, store, length and decode launches, replayed as one CUDA graph.  ``own_key_exact`` (fused launch only): the new key attends with
        its exact values in this step, as in the reference's Mode B.

        k_new / v_new (n_seqs, H, 1, d), q bf16 (n_seqs, Hq, d); the result is a device tensor that
        the next call overwrites.  Pages are reserved on the host before the launch, which only
        writes table entries in place.  In the graph form the inputs are first copied into fixed
        staging buffers, so that the captured launches see stable addresses; the graph is captured on
        first use and again whenever something it baked in changes: the page table or the pools moved
        (growth), or the longest context crossed the split boundary the grid was sized for (the split
        set-up rounds the context up to a whole number of splits, so that is every
        ``tokens_per_split`` steps at most)."""
        n = len(self.lengths)
        dev = self.tables.device
        gs = getattr(self, "_gen_step", None)
        # Fast path of the fused step: while no sequence needs a page and the context stays inside
        # what the grid was sized for, a step is one library call and nothing else on the host.
        if (fused_append and gs is not None and gs["fused"] and getattr(self, "_gen_budget", 0) > 0
                and gs["generation"] == self.pool.generation and gs["lengths_after"] == self.lengths
                and gs["shape"] == (tuple(k_new.shape), tuple(q.shape), k_new.dtype, v_new.dtype)
                and gs["strides"] == (k_new.stride(), v_new.stride()) and q.is_contiguous()
                and gs["table_ptr"] == self.page_table.data_ptr() and gs["lens_ptr"] == self.seq_lens.data_ptr()):
            self._gen_budget -= 1
            # the call the slow path below made through decode_append_attend (which checked the
            # arguments), with this step's three pointers, flag and stream put in
            args = gs["args"]
            args[gs["arg0"]], args[gs["arg0"] + 1], args[gs["arg0"] + 2] = q.data_ptr(), k_new.data_ptr(), v_new.data_ptr()
            args[-5] = 1 if own_key_exact else 0
            args[-1] = _stream_ptr(dev)
            _native.check(gs["fn"](*args))
            for s_ in range(n):
                self.lengths[s_] += 1
            self._epoch += 1
            gs["lengths_after"] = list(self.lengths)
            return gs["out"]
        if k_new.shape[0] != n or k_new.shape[2] != 1:
            raise ValueError(f"generate_step takes one token for each of the {n} sequences")
        for s_ in range(n):   # pages a few steps ahead, so that the host touches the table once in a while only
            self.reserve(s_, self.lengths[s_] + (self.RESERVE_AHEAD if fused_append else 1))
        gs = getattr(self, "_gen_step", None)
        new_max = max(self.lengths) + 1
        fused = bool(fused_append)
        if own_key_exact and not fused:
            raise ValueError("own_key_exact needs the fused append launch (fused_append=True)")
        if (gs is None or gs["generation"] != self.pool.generation or gs["table_ptr"] != self.page_table.data_ptr()
                or gs["shape"] != (tuple(k_new.shape), tuple(q.shape), k_new.dtype, v_new.dtype) or new_max > gs["covered"]
                or gs["fused"] != fused):
            n_q_heads = q.shape[1]
            tps = split_for_lengths([x + 1 for x in self.lengths], n_q_heads, self.tables.n_heads)
            covered = -(-new_max // tps) * tps                     # the grid covers contexts up to here
            ws = self._workspace(n, n_q_heads, covered // tps)
            if getattr(self, "_ones", None) is None or self._ones.numel() != n:
                self._ones = torch.ones(n, dtype=torch.int32, device=dev)
            gs = {"generation": self.pool.generation, "table_ptr": self.page_table.data_ptr(), "covered": covered,
                  "shape": (tuple(k_new.shape), tuple(q.shape), k_new.dtype, v_new.dtype), "ws": ws, "tps": tps,
                  "fused": fused, "pools": (self.k_pool, self.v_pool, self.page_table),
                  "out": torch.empty(q.shape, dtype=torch.float32, device=dev)}
            if not fused:
                gs.update({"k": torch.empty_like(k_new, device=dev).contiguous(), "v": torch.empty_like(v_new, device=dev).contiguous(),
                           "q": torch.empty_like(q, device=dev), "stream": torch.cuda.Stream(dev)})

                def enqueue() -> None:
                    compress_into(self.tables, gs["k"], self._ones, 1, self.page_table, self.k_pool, self.status, self.seq_lens)
                    self._store_values(gs["v"], self._ones, 1, self.seq_lens)
                    self.seq_lens[:n] += 1
                    decode_attend(self.tables, gs["q"], self.seq_lens, covered, self.page_table, self.k_pool, self.v_pool,
                                  gs["out"], ws, self.status, tps, v_tables=self.v_tables)

                # the library's one-time set-up (shared-memory attributes) must happen outside a capture:
                # run the step once for real on a scratch copy of the lengths, then restore them
                saved = self.seq_lens.clone()
                gs["k"].copy_(k_new); gs["v"].copy_(v_new); gs["q"].copy_(q)
                with torch.cuda.stream(gs["stream"]):
                    gs["stream"].wait_stream(torch.cuda.current_stream(dev))
                    enqueue()
                    gs["stream"].synchronize()
                    self.seq_lens.copy_(saved)
                    gs["graph"] = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(gs["graph"], stream=gs["stream"]):
                        enqueue()
            self._gen_step = gs
        if fused:
            # one launch on the caller's stream: the kernel reads the rows where they are, appends them,
            # attends and advances the lengths; there is nothing to stage and nothing to capture
            decode_append_attend(self.tables, q if q.is_contiguous() else q.contiguous(), k_new, v_new, self.seq_lens,
                                 gs["covered"], self.page_table, self.k_pool, self.v_pool, gs["out"], gs["ws"],
                                 self.status, gs["tps"], own_key_exact, self.v_tables)
            # the same call's argument list, kept for the steps that change nothing but the rows
            vt = self.v_tables
            head = [self.tables.ref] if vt is None else [self.tables.ref, vt.ref]
            gs["fn"] = _native.lib.jqk_decode_append_attend if vt is None else _native.lib.jqk_decode_append_attend_packed_values
            gs["arg0"] = len(head)
            gs["strides"] = (k_new.stride(), v_new.stride())
            gs["lens_ptr"] = self.seq_lens.data_ptr()
            gs["args"] = head + [
                0, 0, 0, _native.torch_dtype_code(k_new.dtype), _native.torch_dtype_code(v_new.dtype), k_new.stride(0),
                k_new.stride(1), v_new.stride(0), v_new.stride(1), n, q.shape[1], self.seq_lens.data_ptr(), int(gs["covered"]),
                int(gs["tps"]), self.page_table.data_ptr(), self.page_table.stride(0), int(self.k_pool.shape[0]),
                self.k_pool.data_ptr(), self.v_pool.data_ptr(), gs["out"].data_ptr(), _native.torch_dtype_code(gs["out"].dtype),
                0, gs["ws"].buf.data_ptr(), gs["ws"].buf.numel(), self.status.data_ptr(), 0]
        else:
            gs["k"].copy_(k_new, non_blocking=True)
            gs["v"].copy_(v_new, non_blocking=True)
            gs["q"].copy_(q, non_blocking=True)
            gs["graph"].replay()
        for s_ in range(n):
            self.lengths[s_] += 1
        self._epoch += 1
        gs["lengths_after"] = list(self.lengths)
        # steps that need neither a page nor a larger grid
        self._gen_budget = min(min(len(pg) * PAGE_TOKENS - ln for pg, ln in zip(self._pages, self.lengths)),
                               gs["covered"] - max(self.lengths)) if n else 0
        return gs["out"]

    def _store_values(self, values: torch.Tensor, n_tok: torch.Tensor, max_tokens: int, starts: torch.Tensor) -> None:
        if self.v_tables is None:
            store_values_into(values, n_tok, max_tokens, self.page_table, self.v_pool, self.status, starts)
        else:
            if values.dtype not in (torch.float32, torch.bfloat16, torch.float16):
                values = values.float()
            compress_into(self.v_tables, values, n_tok, max_tokens, self.page_table, self.v_pool, self.status, starts)

    def _workspace(self, n_seqs: int, n_q_heads: int, max_splits: int) -> DecodeWorkspace:
        ws = self._ws
        if ws is None or ws.max_splits < max_splits or ws.n_seqs < n_seqs or ws.n_q_heads < n_q_heads:
            ws = self._ws = DecodeWorkspace(n_seqs, n_q_heads, self.tables.n_heads, max_splits, self.tables.device)
        return ws

    def decode(self, q: torch.Tensor, out_dtype: torch.dtype = torch.float32, tokens_per_split: int = 0) -> torch.Tensor:
        n_seqs, n_q_heads, _ = q.shape
        max_len = max(self.lengths) if self.lengths else 0
        tps = tokens_per_split or split_for_lengths(self.lengths[:n_seqs], n_q_heads, self.tables.n_heads)
        ws = self._workspace(n_seqs, n_q_heads, max(1, -(-max_len // tps)))
        out = torch.empty(q.shape, dtype=out_dtype, device=q.device)
        return decode_attend(self.tables, q, self.seq_lens, max_len, self.page_table, self.k_pool, self.v_pool,
                             out, ws, self.status, tps, v_tables=self.v_tables)

    def _host_state_stale(self, hs: dict | None, key: tuple) -> bool:
        return (hs is None or hs["key"] != key or hs["lengths"] != self.lengths
                or hs["generation"] != self.pool.generation or hs["table_ptr"] != self.page_table.data_ptr())

    def decode_host(self, q_host: torch.Tensor, tokens_per_split: int = 0, use_graph: bool = True,
                    zero_copy: bool | str = False) -> torch.Tensor:
        """One decode step from host memory: bf16 query (n_seqs, Hq, d) in, fp32 result out in a
        pinned host tensor that the next call overwrites.

        Default: the query is copied to the device, the step runs on device buffers and the result is
        copied back (three commands).  ``zero_copy=True``: the kernel itself moves the data across the
        bus: the blocks read their query heads from the page-locked staging buffer when they build
        their tables, and the block that finishes a head writes its result straight into the
        page-locked output, so the step is one kernel with no copy commands around it;
        ``zero_copy="out"`` keeps the copy of the query and lets the kernel write the result.  On the
        single-sequence shape the three variants measured within a few percent of one another (44 to
        49 us per step, run-to-run spread included: the step is dominated by the graph launch and the
        wake-up after the wait, not by the two small copies), so the options are for hosts that want
        no copy engine involved, not a speed-up.  Either way the commands are
        captured once as a CUDA graph (per batch shape, context length and split); every call stages
        the query in pinned memory, replays the graph and waits for it, so the host pays one graph
        launch and one synchronisation per step.  The cache must not grow
        between capture and replay: a call after ``prefill`` captures again.  The captured graph keeps
        its own reference to the split workspace it was recorded with, so a later ``decode`` that needs
        a larger workspace does not pull that memory from under it.  ``use_graph=False`` makes one
        call of ``jqk_decode_attend_host`` instead (no capture; three enqueues and a wait)."""
        hs = self._host_step
        # Steady state: the same shape on an unchanged cache.  Two integer comparisons, a copy of the
        # query into the staging buffer, one graph launch, one stream wait.
        if (use_graph and hs is not None and hs["epoch"] == self._epoch and hs["generation"] == self.pool.generation
                and hs["fast_key"] == (q_host.shape, tokens_per_split, zero_copy) and q_host.dtype is torch.bfloat16
                and q_host.device.type == "cpu" and q_host.is_contiguous()):
            if q_host.data_ptr() != hs["q_pin_ptr"]:
                ctypes.memmove(hs["q_pin_ptr"], q_host.data_ptr(), hs["q_bytes"])
            hs["graph"].replay()
            torch.cuda.current_stream(hs["device"]).synchronize()
            return hs["out_pin"]
        if q_host.device.type != "cpu" or q_host.dtype != torch.bfloat16 or q_host.dim() != 3 or not q_host.is_contiguous():
            raise ValueError("q_host must be a contiguous bf16 (n_seqs, n_q_heads, d) tensor in host memory")
        if self.v_tables is not None and not use_graph:
            raise NotImplementedError("with packed values decode_host takes the graph form (jqk_decode_attend_host is wired for bf16 values)")
        if not use_graph:
            return self._decode_host_call(q_host, tokens_per_split, zero_copy)
        dev = self.tables.device
        n_seqs, n_q_heads, d = q_host.shape
        hs = self._host_step
        if zero_copy not in (False, True, "out"):
            raise ValueError("zero_copy is False, True or 'out'")
        key = (n_seqs, n_q_heads, d, int(tokens_per_split), str(zero_copy))
        if self._host_state_stale(hs, key):
            max_len = max(self.lengths) if self.lengths else 0
            tps = tokens_per_split or split_for_lengths(self.lengths[:n_seqs], n_q_heads, self.tables.n_heads)
            hs = {"key": key, "lengths": list(self.lengths), "generation": self.pool.generation,
                  "table_ptr": self.page_table.data_ptr(), "epoch": self._epoch, "device": dev,
                  "fast_key": (q_host.shape, tokens_per_split, zero_copy),
                  "ws": self._workspace(n_seqs, n_q_heads, max(1, -(-max_len // tps))),
                  "pools": (self.k_pool, self.v_pool, self.page_table),
                  "q_pin": torch.empty((n_seqs, n_q_heads, d), dtype=torch.bfloat16).pin_memory(),
                  "out_pin": torch.empty((n_seqs, n_q_heads, d), dtype=torch.float32).pin_memory(),
                  "q_dev": torch.empty((n_seqs, n_q_heads, d), dtype=torch.bfloat16, device=dev),
                  "out_dev": torch.empty((n_seqs, n_q_heads, d), dtype=torch.float32, device=dev),
                  "stream": torch.cuda.Stream(dev)}

            def enqueue() -> None:
                # page-locked host memory is device-addressable: it can stand in for q and / or out
                q_arg = hs["q_pin"] if zero_copy is True else hs["q_dev"]
                out_arg = hs["out_pin"] if zero_copy else hs["out_dev"]
                if q_arg is hs["q_dev"]:
                    hs["q_dev"].copy_(hs["q_pin"], non_blocking=True)
                decode_attend(self.tables, q_arg, self.seq_lens, max_len, hs["pools"][2], hs["pools"][0],
                              hs["pools"][1], out_arg, hs["ws"], self.status, tps, v_tables=self.v_tables)
                if out_arg is hs["out_dev"]:
                    hs["out_pin"].copy_(hs["out_dev"], non_blocking=True)

            hs["q_pin_ptr"], hs["q_bytes"] = hs["q_pin"].data_ptr(), hs["q_pin"].numel() * 2
            hs["q_pin"].copy_(q_host)
            with torch.cuda.stream(hs["stream"]):
                enqueue()                      # first call outside capture: one-time set-up of the library
                hs["stream"].synchronize()
                hs["graph"] = torch.cuda.CUDAGraph()
                with torch.cuda.graph(hs["graph"], stream=hs["stream"]):
                    enqueue()
            self._host_step = hs
        if q_host.data_ptr() != hs["q_pin"].data_ptr():
            hs["q_pin"].copy_(q_host)
        hs["graph"].replay()
        torch.cuda.current_stream(dev).synchronize()   # the graph is launched on the current stream
        return hs["out_pin"]

    def _decode_host_call(self, q_host: torch.Tensor, tokens_per_split: int = 0, zero_copy: bool | str = False) -> torch.Tensor:
        """One decode step from host memory: bf16 query (n_seqs, Hq, d) in, fp32 result out in a
        pinned host tensor that the next call overwrites.

        One call of ``jqk_decode_attend_host``: the query is staged in pinned memory and copied to
        the device, the step runs, the result is copied back and the stream is synchronised, so the
        host pays one foreign-function call per step.  The staging buffers are kept per batch shape,
        together with the workspace and pools whose addresses the cached argument list holds."""
        dev = self.tables.device
        n_seqs, n_q_heads, d = q_host.shape
        hs = self._host_call
        key = (n_seqs, n_q_heads, d, int(tokens_per_split), str(zero_copy))
        if self._host_state_stale(hs, key):
            max_len = max(self.lengths) if self.lengths else 0
            tps = tokens_per_split or split_for_lengths(self.lengths[:n_seqs], n_q_heads, self.tables.n_heads)
            ws = self._workspace(n_seqs, n_q_heads, max(1, -(-max_len // tps)))
            keep = hs if hs is not None and hs["key"] == key else None
            hs = {"key": key, "lengths": list(self.lengths), "max_len": max_len, "tps": tps, "ws": ws,
                  "generation": self.pool.generation, "table_ptr": self.page_table.data_ptr(),
                  "pools": (self.k_pool, self.v_pool, self.page_table),
                  "q_pin": keep["q_pin"] if keep else torch.empty((n_seqs, n_q_heads, d), dtype=torch.bfloat16).pin_memory(),
                  "out_pin": keep["out_pin"] if keep else torch.empty((n_seqs, n_q_heads, d), dtype=torch.float32).pin_memory(),
                  "q_dev": keep["q_dev"] if keep else torch.empty((n_seqs, n_q_heads, d), dtype=torch.bfloat16, device=dev),
                  "out_dev": keep["out_dev"] if keep else torch.empty((n_seqs, n_q_heads, d), dtype=torch.float32, device=dev)}
            hs["args"] = (self.tables.ref, hs["q_pin"].data_ptr(), None if zero_copy is True else hs["q_dev"].data_ptr(), n_seqs, n_q_heads,
                          self.seq_lens.data_ptr(), int(max_len), int(tps), self.page_table.data_ptr(),
                          self.page_table.stride(0), int(self.k_pool.shape[0]), self.k_pool.data_ptr(),
                          self.v_pool.data_ptr(), None if zero_copy else hs["out_dev"].data_ptr(), hs["out_pin"].data_ptr(),
                          _native.DTYPE_F32, ws.buf.data_ptr(), ws.buf.numel(), self.status.data_ptr())
            self._host_call = hs
        a = hs["args"]
        _native.check(_native.lib.jqk_decode_attend_host(a[0], q_host.data_ptr(), *a[1:], _stream_ptr(dev)))
        return hs["out_pin"]
