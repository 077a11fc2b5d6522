"""A kvpress-shaped press over the paged GPU cache.

Mirrors ``JointQKPress`` (experiments/stage1/toolkit/jointqk_press.py:31-308): the same
constructor fields, ``post_init_from_model`` (:124-233), ``compress`` (:268-273) and
``forward_hook`` (:275-308), so an evaluation harness written against the reference can drive it.
It does not import ``kvpress`` (the hook protocol is duck-typed: a module with ``layer_idx``, a
cache with ``layers[i].keys`` / ``.values``), so it can be exercised with the same stub objects the
reference's parity scripts use.

What differs, on purpose: besides handing reconstructed tensors back to the caller's cache (what
the reference does, so stock attention still works), every compressed layer keeps a
``PagedKVCache`` with the packed keys and the values, filled by the CUDA kernels, and
``decode(layer, q)`` attends over it directly.  Prefill goes through one compress launch and one
value-store launch per layer; in Mode B (``compress_decode=True``) a decode step appends only the
newest token (reference :298-304).
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from . import paged
from .compressor import PerCoordCompressor, build_method_compressor
from .tables import HeadTables
from .v_compressor import CenteredCompressor, build_v_compressor


@dataclass
class JointQKPressB200:
    cca_stats_path: str = ""
    v_stats_path: str = ""
    v_method: str = "v_eigen_waterfill"
    k_method: str = "r_sym_waterfill"
    k_bits: int = 4
    v_bits: int = 2
    rank: int = 64
    layer0_full_precision: bool = True
    quantize_k: bool = True
    quantize_v: bool = True
    compress_decode: bool = False
    eps: float = 1e-6
    compression_ratio: float = 0.0
    # cap on bits per coordinate.  The reference hard-codes 8; the packed format holds that as long as at
    # most 32 coordinates of a head go above 4 bits and the record stays within 512 bits (budgets up to
    # about 3 bits per coordinate on the evaluated spectra).  Beyond that the press still hands back the
    # reference's reconstruction (made without a record) but keeps no paged cache.  4 packs at every budget,
    # with a different allocation than the reference's (a quality cost where outlier channels want more).
    max_bits: int = 8

    _k_compressors: dict = field(default_factory=dict, init=False, repr=False)
    _v_compressors: dict = field(default_factory=dict, init=False, repr=False)
    _n_layers: int = field(default=0, init=False, repr=False)
    _n_kv_heads: int = field(default=0, init=False, repr=False)
    _k_tables: dict = field(default_factory=dict, init=False, repr=False)
    _v_tables: dict = field(default_factory=dict, init=False, repr=False)
    caches: dict = field(default_factory=dict, init=False, repr=False)   # layer -> PagedKVCache

    # ---- construction --------------------------------------------------------------------
    def post_init_from_model(self, model) -> None:
        """Load the calibration artefacts and build one compressor per (layer, kv head).
        Idempotent, like the reference (:124-146)."""
        if (self._k_compressors or not self.quantize_k) and (self._v_compressors or not self.quantize_v):
            return
        if self.quantize_k:
            if not self.cca_stats_path:
                raise ValueError("quantize_k=True requires cca_stats_path")
            cca = torch.load(self.cca_stats_path, map_location="cpu", weights_only=False)
            n_layers, n_kv_heads, d, _ = cca["sigma_q"].shape
            self._n_layers, self._n_kv_heads = n_layers, n_kv_heads
            for L in range(n_layers):
                if L == 0 and self.layer0_full_precision:
                    continue
                for h in range(n_kv_heads):
                    self._k_compressors[(L, h)] = build_method_compressor(
                        method=self.k_method, sigma_q_for_head=cca["sigma_q"][L, h], sigma_k_for_head=cca["sigma_k"][L, h],
                        cca={"P_K": cca["P_K"][L, h], "P_K_inv": cca["P_K_inv"][L, h], "rho": cca["rho"][L, h]},
                        mq_eigvals=cca["mq_eigvals"][L, h] if "mq_eigvals" in cca else None,
                        mq_eigvecs=cca["mq_eigvecs"][L, h] if "mq_eigvecs" in cca else None,
                        b_avg=float(self.k_bits), r=self.rank, seed=42, head_dim=d,
                        V_h=cca["V_h"][L, h] if "V_h" in cca else None,
                        R_sym=cca["R_sym"][L, h] if "R_sym" in cca else None, max_bits=self.max_bits)
        if self.quantize_v:
            if not self.v_stats_path:
                raise ValueError("quantize_v=True requires v_stats_path")
            v_stats = torch.load(self.v_stats_path, map_location="cpu", weights_only=False)
            cov_v = v_stats.get("cov_v", v_stats.get("sigma_v"))
            mu_v = v_stats.get("mu_v")
            n_layers_v, n_kv_heads_v, d_v, _ = cov_v.shape
            if self._n_layers and self._n_layers != n_layers_v:
                raise ValueError(f"V stats n_layers={n_layers_v} != cca_stats n_layers={self._n_layers}")
            self._n_layers, self._n_kv_heads = n_layers_v, n_kv_heads_v
            for L in range(n_layers_v):
                if L == 0 and self.layer0_full_precision:
                    continue
                for h in range(n_kv_heads_v):
                    self._v_compressors[(L, h)] = build_v_compressor(
                        method=self.v_method, cov_v_for_head=cov_v[L, h],
                        mu_v_for_head=(mu_v[L, h] if mu_v is not None else None), head_dim=d_v,
                        bits=int(self.v_bits), seed=42 + L * 1000 + h, max_bits=self.max_bits)

    # ---- device tables per layer ------------------------------------------------------------
    def _layer_tables(self, layer_idx: int, comps: dict, store: dict, device):
        hit = store.get(layer_idx)
        if hit is None or hit.device != torch.device(device):
            heads = [comps[(layer_idx, h)] for h in range(self._n_kv_heads)]
            inner = [c.inner if isinstance(c, CenteredCompressor) else c for c in heads]
            center = None
            if any(isinstance(c, CenteredCompressor) for c in heads):
                center = torch.stack([c.mu.float().cpu() if isinstance(c, CenteredCompressor) else torch.zeros(c.d)
                                      for c in heads])
            if all(c.packable for c in inner):
                hit = HeadTables.from_compressors(inner, device=device, center=center)
            else:
                # an allocation beyond the packed record (the reference's cap of 8 at 4 bits per
                # coordinate, say): the reconstruction is made without one and no cache is kept
                for c in inner:
                    if int(c.bits_int.max()) > 8:
                        c.head_tables(device)      # raises with the explanation
                from .compressor import stack_per_head
                from .dense import DenseTables

                fwd, inv, cb = stack_per_head(inner)
                hit = DenseTables(fwd, inv, cb, device, center=center)
            store[layer_idx] = hit
        return hit

    def _skip(self, layer_idx: int) -> bool:
        return layer_idx == 0 and self.layer0_full_precision

    # ---- the press interface ------------------------------------------------------------------
    @torch.no_grad()
    def compress(self, module, hidden_states, keys: torch.Tensor, values: torch.Tensor, attentions, kwargs):
        """keys / values (B, Hkv, S, d) of one layer -> their reconstructions in the input dtype, and,
        as a side effect, S more tokens in the layer's paged cache.  Layer 0 passes through when
        ``layer0_full_precision`` is set (:259-265)."""
        L = int(module.layer_idx)
        if self._skip(L) or not (self.quantize_k or self.quantize_v):
            return keys, values
        dev = keys.device if keys.is_cuda else torch.device("cuda", torch.cuda.current_device())
        B, H, S, d = keys.shape
        k_dev, v_dev = keys.to(dev), values.to(dev)
        v_out = values
        if self.quantize_v:        # values: compress and reconstruct on the GPU, keep the reconstruction
            vt = self._layer_tables(L, self._v_compressors, self._v_tables, dev)
            v_in = v_dev if v_dev.dtype != torch.float64 else v_dev.float()
            if isinstance(vt, HeadTables):
                v_hat = paged.decompress(paged.compress(vt, v_in))
            else:
                v_hat = torch.stack([vt.roundtrip(v_in[b])[0] for b in range(B)])
            v_dev = v_hat.to(values.dtype)
            v_out = v_dev.to(values.device)
        k_out = keys
        if self.quantize_k:
            kt = self._layer_tables(L, self._k_compressors, self._k_tables, dev)
            if not isinstance(kt, HeadTables):     # no record, so no paged cache: reconstruct and hand back
                k_in = k_dev if k_dev.dtype != torch.float64 else k_dev.float()
                k_hat = torch.stack([kt.roundtrip(k_in[b])[0] for b in range(B)])
                return k_hat.to(keys.dtype).to(keys.device), v_out
            cache = self.caches.get(L)
            if cache is None or len(cache.lengths) != B:
                cache = self.caches[L] = paged.PagedKVCache(kt, n_seqs=B)
            first = list(cache.lengths)
            cache.prefill(k_dev, v_dev)
            # what the caller's dense cache gets: the reconstruction of exactly the rows just stored
            n_tok = torch.full((B,), S, dtype=torch.int32, device=dev)
            starts = torch.tensor(first, dtype=torch.int32, device=dev)
            k_hat = _decompress_range(kt, cache, n_tok, starts, S)
            k_out = k_hat.to(keys.dtype).to(keys.device)
        return k_out, v_out

    @torch.no_grad()
    def forward_hook(self, module, args, kwargs, output):
        """Hook an attention module calls after its forward.  Prefill: compress the layer's whole K/V.
        Decode steps: nothing (Mode A) or the newest token only (Mode B, ``compress_decode``),
        leaving the history untouched (:275-308)."""
        hidden_states = kwargs["hidden_states"]
        cache = kwargs["past_key_values"]
        layer = cache.layers[module.layer_idx]
        q_len = hidden_states.shape[1]
        is_prefill = int(kwargs["cache_position"][-1]) <= q_len
        if not is_prefill and not self.compress_decode:
            return output
        keys, values = layer.keys, layer.values
        if is_prefill:
            self.reset_layer(module.layer_idx)
            keys, values = self.compress(module, hidden_states, keys, values, output[1] if len(output) > 1 else None, kwargs)
        else:
            new_k, new_v = self.compress(module, hidden_states, keys[:, :, -1:, :], values[:, :, -1:, :], None, kwargs)
            keys = torch.cat([keys[:, :, :-1, :], new_k], dim=2)
            values = torch.cat([values[:, :, :-1, :], new_v], dim=2)
        layer.keys, layer.values = keys, values
        return output

    # ---- the paged side -----------------------------------------------------------------------
    def reset_layer(self, layer_idx: int) -> None:
        """Drop the paged cache of a layer (a new prompt starts)."""
        self.caches.pop(int(layer_idx), None)

    @torch.no_grad()
    def decode(self, layer_idx: int, q: torch.Tensor, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
        """softmax(q . k_hat / sqrt(d)) @ V over the layer's paged cache: q bf16 (B, Hq, d)."""
        cache = self.caches.get(int(layer_idx))
        if cache is None:
            raise RuntimeError(
                f"layer {int(layer_idx)} has no paged cache: nothing was compressed yet, or its allocation is beyond the "
                "packed record (more than 32 coordinates above 4 bits or 512 bits per key; see max_bits)")
        return cache.decode(q.to(cache.tables.device), out_dtype=out_dtype)


def _decompress_range(tables: HeadTables, cache: "paged.PagedKVCache", n_tok: torch.Tensor, starts: torch.Tensor,
                      max_tokens: int) -> torch.Tensor:
    """fp32 (B, H, max_tokens, d): reconstruction of tokens [starts, starts + n_tok) of every sequence."""
    from . import _native

    B = len(cache.lengths)
    out = torch.zeros((B, tables.n_heads, max_tokens, tables.d), dtype=torch.float32, device=tables.device)
    _native.check(_native.lib.jqk_decompress_paged(
        tables.ref, B, n_tok.data_ptr(), starts.data_ptr(), int(max_tokens), cache.page_table.data_ptr(),
        cache.page_table.stride(0), cache.n_pages, cache.k_pool.data_ptr(), out.data_ptr(), cache.status.data_ptr(),
        torch.cuda.current_stream(tables.device).cuda_stream))
    return out
