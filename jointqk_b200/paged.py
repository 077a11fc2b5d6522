"""Paged storage for packed keys and bf16 values, and the calls that fill and read it.

Everything here is plumbing around the C ABI: torch owns the device memory and the stream,
the kernels do the work.  The reference has no counterpart for the storage itself (it keeps
dequantised floats in the HF cache, experiments/stage1/toolkit/jointqk_press.py:306-307).
"""

from __future__ import annotations

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
    """Raise if a kernel flagged a bad page index or an expired wait (synchronises)."""
    v = int(status.item())
    if v & _native.STATUS_BAD_PAGE:
        raise RuntimeError("jointqk_b200: page table holds an index outside the pool")
    if v & _native.STATUS_WAIT_EXPIRED:
        raise RuntimeError("jointqk_b200: a bounded device-side wait expired")


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
            t.ref, packed.n_seqs, packed.n_tokens.data_ptr(), packed.max_tokens,
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
        self.max_splits = max_splits
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
                  tokens_per_split: int = 0) -> torch.Tensor:
    """One decode step for one layer.  q bf16 (n_seqs, Hq, d); out fp32 or bf16 (n_seqs, Hq, d)."""
    if q.dtype != torch.bfloat16 or q.dim() != 3 or not q.is_contiguous():
        raise ValueError("q must be a contiguous bf16 (n_seqs, n_q_heads, d) tensor")
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


class PagedKVCache:
    """Packed-K / bf16-V paged cache of one layer for a batch of sequences.

    ``prefill`` compresses keys into pages and scatters values; ``decode`` runs the fused
    attention kernel.  Pages are assigned sequentially at construction from the maximum
    lengths given, which is all the synthetic workloads need.
    """

    def __init__(self, tables: HeadTables, max_lengths: list[int]) -> None:
        self.tables = tables
        dev = tables.device
        self.page_table, used = sequential_page_table(max_lengths, dev)
        self.n_pages = max(1, used)
        self.k_pool = alloc_k_pool(tables, self.n_pages)
        self.v_pool = alloc_v_pool(tables, self.n_pages)
        self.lengths = [0] * len(max_lengths)
        self.capacity = [pages_for(n) * PAGE_TOKENS for n in max_lengths]
        self.seq_lens = torch.zeros(max(1, len(max_lengths)), dtype=torch.int32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self._ws: DecodeWorkspace | None = None
        self._host_step: dict | None = None
        self._host_call: dict | None = None

    def prefill(self, keys: torch.Tensor, values: torch.Tensor, lengths: list[int] | None = None) -> None:
        """keys/values (n_seqs, H, S, d).  Appends ``lengths[s]`` tokens to every sequence."""
        n_seqs, H, S, d = keys.shape
        lengths = [S] * n_seqs if lengths is None else [int(x) for x in lengths]
        dev = self.tables.device
        for s, n in enumerate(lengths):
            if self.lengths[s] + n > self.capacity[s]:
                raise ValueError(f"sequence {s}: {self.lengths[s]} + {n} tokens exceed its {self.capacity[s]} slots")
        starts = torch.tensor(self.lengths, dtype=torch.int32, device=dev)
        n_tok = torch.tensor(lengths, dtype=torch.int32, device=dev)
        if max(lengths) > 0:
            compress_into(self.tables, keys, n_tok, max(lengths), self.page_table, self.k_pool, self.status, starts)
        for s, n in enumerate(lengths):                      # value scatter: plain torch indexing
            if n == 0:
                continue
            pos = torch.arange(self.lengths[s], self.lengths[s] + n, device=dev)
            pages = self.page_table[s, pos // PAGE_TOKENS].long()
            offs = v_slot_offsets(d, dev)[pos % PAGE_TOKENS]                     # (n, d)
            self.v_pool[pages[:, None], :, offs] = values[s, :, :n, :].to(torch.bfloat16).permute(1, 2, 0)
            self.lengths[s] += n
        self.seq_lens[: len(self.lengths)] = torch.tensor(self.lengths, dtype=torch.int32, device=dev)

    def decode(self, q: torch.Tensor, out_dtype: torch.dtype = torch.float32, tokens_per_split: int = 0) -> torch.Tensor:
        n_seqs, n_q_heads, _ = q.shape
        max_len = max(self.lengths) if self.lengths else 0
        tps = tokens_per_split or split_for_lengths(self.lengths[:n_seqs], n_q_heads, self.tables.n_heads)
        max_splits = max(1, -(-max_len // tps))
        if self._ws is None or self._ws.max_splits < max_splits:
            self._ws = DecodeWorkspace(n_seqs, n_q_heads, self.tables.n_heads, max_splits, self.tables.device)
        out = torch.empty(q.shape, dtype=out_dtype, device=q.device)
        return decode_attend(self.tables, q, self.seq_lens, max_len, self.page_table, self.k_pool, self.v_pool,
                             out, self._ws, self.status, tps)

    def decode_host(self, q_host: torch.Tensor, tokens_per_split: int = 0, use_graph: bool = True) -> torch.Tensor:
        """One decode step from host memory: bf16 query (n_seqs, Hq, d) in, fp32 result out in a
        pinned host tensor that the next call overwrites.

        The copy of the query to the device, the decode launch and the copy of the result back are
        captured once as a CUDA graph (per batch shape, context length and split); every call stages
        the query in pinned memory, replays the graph and waits for it, so the host pays one graph
        launch and one synchronisation per step instead of three enqueues.  The cache must not grow
        between capture and replay: a call after ``prefill`` captures again.  ``use_graph=False`` makes
        one call of ``jqk_decode_attend_host`` instead (no capture; three enqueues and a wait)."""
        if q_host.device.type != "cpu" or q_host.dtype != torch.bfloat16 or q_host.dim() != 3 or not q_host.is_contiguous():
            raise ValueError("q_host must be a contiguous bf16 (n_seqs, n_q_heads, d) tensor in host memory")
        if not use_graph:
            return self._decode_host_call(q_host, tokens_per_split)
        dev = self.tables.device
        n_seqs, n_q_heads, d = q_host.shape
        hs = self._host_step
        key = (n_seqs, n_q_heads, d, int(tokens_per_split))
        if hs is None or hs["key"] != key or hs["lengths"] != self.lengths:
            max_len = max(self.lengths) if self.lengths else 0
            tps = tokens_per_split or split_for_lengths(self.lengths[:n_seqs], n_q_heads, self.tables.n_heads)
            max_splits = max(1, -(-max_len // tps))
            if self._ws is None or self._ws.max_splits < max_splits:
                self._ws = DecodeWorkspace(n_seqs, n_q_heads, self.tables.n_heads, max_splits, dev)
            hs = {"key": key, "lengths": list(self.lengths),
                  "q_pin": torch.empty((n_seqs, n_q_heads, d), dtype=torch.bfloat16).pin_memory(),
                  "out_pin": torch.empty((n_seqs, n_q_heads, d), dtype=torch.float32).pin_memory(),
                  "q_dev": torch.empty((n_seqs, n_q_heads, d), dtype=torch.bfloat16, device=dev),
                  "out_dev": torch.empty((n_seqs, n_q_heads, d), dtype=torch.float32, device=dev),
                  "stream": torch.cuda.Stream(dev)}

            def enqueue() -> None:
                hs["q_dev"].copy_(hs["q_pin"], non_blocking=True)
                decode_attend(self.tables, hs["q_dev"], self.seq_lens, max_len, self.page_table, self.k_pool,
                              self.v_pool, hs["out_dev"], self._ws, self.status, tps)
                hs["out_pin"].copy_(hs["out_dev"], non_blocking=True)

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

    def _decode_host_call(self, q_host: torch.Tensor, tokens_per_split: int = 0) -> torch.Tensor:
        """One decode step from host memory: bf16 query (n_seqs, Hq, d) in, fp32 result out in a
        pinned host tensor that the next call overwrites.

        One call of ``jqk_decode_attend_host``: the query is staged in pinned memory and copied to
        the device, the step runs, the result is copied back and the stream is synchronised, so the
        host pays one foreign-function call per step.  The staging buffers are kept per batch shape."""
        dev = self.tables.device
        n_seqs, n_q_heads, d = q_host.shape
        hs = self._host_call
        key = (n_seqs, n_q_heads, d, int(tokens_per_split))
        if hs is None or hs["key"] != key or hs["lengths"] != self.lengths:
            max_len = max(self.lengths) if self.lengths else 0
            tps = tokens_per_split or split_for_lengths(self.lengths[:n_seqs], n_q_heads, self.tables.n_heads)
            max_splits = max(1, -(-max_len // tps))
            if self._ws is None or self._ws.max_splits < max_splits:
                self._ws = DecodeWorkspace(n_seqs, n_q_heads, self.tables.n_heads, max_splits, dev)
            keep = hs if hs is not None and hs["key"] == key else None
            hs = {"key": key, "lengths": list(self.lengths), "max_len": max_len, "tps": tps,
                  "q_pin": keep["q_pin"] if keep else torch.empty((n_seqs, n_q_heads, d), dtype=torch.bfloat16).pin_memory(),
                  "out_pin": keep["out_pin"] if keep else torch.empty((n_seqs, n_q_heads, d), dtype=torch.float32).pin_memory(),
                  "q_dev": keep["q_dev"] if keep else torch.empty((n_seqs, n_q_heads, d), dtype=torch.bfloat16, device=dev),
                  "out_dev": keep["out_dev"] if keep else torch.empty((n_seqs, n_q_heads, d), dtype=torch.float32, device=dev)}
            hs["args"] = (self.tables.ref, hs["q_pin"].data_ptr(), hs["q_dev"].data_ptr(), n_seqs, n_q_heads,
                          self.seq_lens.data_ptr(), int(max_len), int(tps), self.page_table.data_ptr(),
                          self.page_table.stride(0), int(self.k_pool.shape[0]), self.k_pool.data_ptr(),
                          self.v_pool.data_ptr(), hs["out_dev"].data_ptr(), hs["out_pin"].data_ptr(),
                          _native.DTYPE_F32, self._ws.buf.data_ptr(), self._ws.buf.numel(), self.status.data_ptr())
            self._host_call = hs
        a = hs["args"]
        _native.check(_native.lib.jqk_decode_attend_host(a[0], q_host.data_ptr(), *a[1:], _stream_ptr(dev)))
        return hs["out_pin"]
