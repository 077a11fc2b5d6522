"""A `transformers` cache layer that keeps keys packed, and the attention function that reads it.

In the reference the press swaps reconstructed keys into the Hugging Face cache after prefill
(experiments/stage1/toolkit/jointqk_press.py:275-308) and stock attention then runs over dense
tensors.  Here a model keeps its keys packed for the whole generation:

* ``PagedCacheLayer`` is a cache layer (``transformers.cache_utils.CacheLayerMixin``).  The prompt's
  keys and values go through one compress launch and one value-store launch into a
  ``PagedKVCache``; prefill attention itself still sees the exact keys, as in the reference, where
  the hook runs after the layer's forward.  A decode step hands its one new key / value row to the
  attention function instead of storing it.
* ``paged_attention_forward`` is registered with ``AttentionInterface`` under ``ATTN_NAME``.  For a
  decode step of a layer with a ``PagedCacheLayer`` it makes one launch
  (``PagedKVCache.generate_step``: append the row, attend over the packed keys, advance the
  lengths; Mode B of the reference, :298-304: every key ends up compressed, the new one attends with
  its exact values in its own step); anything else (prefill, layers kept at full precision) falls
  through to the stock SDPA path.
* ``calibrate`` runs prompts through the model once and accumulates the moments of the post-RoPE
  queries and keys of every layer with the tensor-core moment kernel; ``build_cache`` fits one
  compressor per (layer, kv head) from them and returns a ``Cache`` made of these layers
  (layer 0 at full precision by default, as ``layer0_full_precision`` in the reference's runs).

Limits, checked and raised: one prefill per sequence batch (no chunked prefill: earlier exact keys
are not kept), no beam reordering, no cropping.  Not checked: a decode step attends over every
cached position of its sequence, so the sequences of a batch must be unpadded (prompts of equal
length, or one sequence at a time); a padding mask is honoured by the stock prefill path only.
"""

from __future__ import annotations

import torch

from .compressor import PerCoordCompressor
from .moments import KeyPathMoments
from .paged import PagedKVCache
from .tables import HeadTables
from .v_compressor import build_v_compressor

ATTN_NAME = "jointqk_paged"
# The reference's Mode-B hook compresses a decode key after the attention of the step that produced
# it (jointqk_press.py:298-304), so in that step the key attends with its exact values.  False: the
# new key is scored from its codes like every other key.
OWN_KEY_EXACT = True


def _transformers():
    try:
        import transformers  # noqa: F401
        from transformers import cache_utils, masking_utils, modeling_utils
        from transformers.integrations import sdpa_attention
    except ImportError as e:  # pragma: no cover - the package is an optional extra of this module
        raise ImportError("jointqk_b200.hf needs the `transformers` package") from e
    return cache_utils, masking_utils, modeling_utils, sdpa_attention


def _layer_base():
    return _transformers()[0].CacheLayerMixin


class _Capture:
    """Moment accumulation during ``calibrate``: the attention function feeds it q and k of a layer."""

    def __init__(self, n_layers: int, n_q_heads: int, n_kv_heads: int, d: int, device, with_values: bool) -> None:
        self.moments = KeyPathMoments(n_layers, n_q_heads, n_kv_heads, d, device=device, with_values=with_values)

    def add(self, layer_idx: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> None:
        # (B, H, S, d): one (H, S, d) chunk per sequence, the layout of the moment kernel
        bf = lambda t: t.to(torch.bfloat16).contiguous()
        for b in range(q.shape[0]):
            self.moments.update(layer_idx, bf(q[b]), bf(k[b]), bf(v[b]) if self.moments.with_values else None)


_STATE = {"capture": None, "registered": False, "layer_class": None}


def register() -> None:
    """Register the attention function and its mask builder under ``ATTN_NAME`` (idempotent)."""
    if _STATE["registered"]:
        return
    cache_utils, masking_utils, modeling_utils, _ = _transformers()
    modeling_utils.AttentionInterface.register(ATTN_NAME, paged_attention_forward)
    masking_utils.AttentionMaskInterface.register(ATTN_NAME, masking_utils.sdpa_mask)
    _STATE["registered"] = True


def paged_attention_forward(module, query, key, value, attention_mask, dropout: float = 0.0, scaling=None, **kwargs):
    """Attention of one layer.  query (B, Hq, S, d); returns (B, S, Hq, d) and no weights."""
    _, _, _, sdpa_attention = _transformers()
    cap = _STATE["capture"]
    if cap is not None:
        cap.add(module.layer_idx, query, key[..., -query.shape[2]:, :], value[..., -query.shape[2]:, :])
    layer = getattr(module, "_jqk_layer", None)
    pending = layer.take_pending() if layer is not None else None
    if pending is None:
        return sdpa_attention.sdpa_attention_forward(module, query, key, value, attention_mask, dropout=dropout,
                                                     scaling=scaling, **kwargs)
    d = query.shape[-1]
    if scaling is not None and abs(float(scaling) * d ** 0.5 - 1.0) > 1e-6:
        raise NotImplementedError("the packed decode scores with 1/sqrt(head_dim)")
    k_new, v_new = pending
    q = query[:, :, 0].to(torch.bfloat16).contiguous()
    out = layer.paged.generate_step(k_new, v_new, q, own_key_exact=OWN_KEY_EXACT)   # (B, Hq, d) fp32, one launch
    return out.to(query.dtype).unsqueeze(1), None


def make_paged_layer_class():
    """The cache layer class (built on first use so that importing this module does not import transformers)."""
    if _STATE["layer_class"] is not None:
        return _STATE["layer_class"]
    base = _layer_base()

    class PagedCacheLayer(base):
        is_sliding = False
        is_compileable = False

        def __init__(self, tables: HeadTables, v_tables: HeadTables | None = None) -> None:
            super().__init__()
            self.tables, self.v_tables = tables, v_tables
            self.paged: PagedKVCache | None = None
            self.cumulative_length = 0
            self._pending = None

        def lazy_initialization(self, key_states: torch.Tensor, value_states: torch.Tensor) -> None:
            self.dtype, self.device = key_states.dtype, key_states.device
            self.paged = PagedKVCache(self.tables, n_seqs=key_states.shape[0], v_tables=self.v_tables)
            self.is_initialized = True

        def update(self, key_states: torch.Tensor, value_states: torch.Tensor, *args, **kwargs):
            if not self.is_initialized:
                self.lazy_initialization(key_states, value_states)
            s = key_states.shape[2]
            if self.cumulative_length == 0:
                self.paged.prefill(key_states, value_states)
            elif s == 1:
                self._pending = (key_states, value_states)      # appended by the attention launch itself
            else:
                raise NotImplementedError("a second multi-token pass over a packed cache (chunked prefill) is not supported")
            self.cumulative_length += s
            return key_states, value_states

        def take_pending(self):
            p, self._pending = self._pending, None
            return p

        def get_seq_length(self) -> int:
            return self.cumulative_length

        def get_mask_sizes(self, query_length: int) -> tuple[int, int]:
            # the mask only matters for the stock prefill path, which sees exactly the keys it is given
            return (query_length if self.cumulative_length == 0 else self.cumulative_length + query_length), 0

        def get_max_cache_shape(self) -> int:
            return -1

        def reset(self) -> None:
            self.paged, self.is_initialized, self.cumulative_length, self._pending = None, False, 0, None

        def reorder_cache(self, beam_idx) -> None:
            raise NotImplementedError("beam search over a packed cache is not supported")

        def offload(self) -> None:   # pages stay on the device
            pass

        def prefetch(self) -> None:
            pass

    _STATE["layer_class"] = PagedCacheLayer
    return PagedCacheLayer


def attention_modules(model) -> list:
    """The model's self-attention modules in layer order (anything with ``layer_idx`` and a ``q_proj``)."""
    mods = [m for m in model.modules() if hasattr(m, "layer_idx") and hasattr(m, "q_proj")]
    return sorted(mods, key=lambda m: m.layer_idx)


def set_attention(model) -> None:
    register()
    model.config._attn_implementation = ATTN_NAME


@torch.no_grad()
def calibrate(model, prompts: list[torch.Tensor], with_values: bool = False) -> KeyPathMoments:
    """Second moments of the post-RoPE queries and keys of every layer (and, ``with_values``, first
    and second moments of the values) over ``prompts`` (each a (B, S) tensor of token ids on the
    model's device), through the model's own forward."""
    cfg = model.config
    d = getattr(cfg, "head_dim", None) or cfg.hidden_size // cfg.num_attention_heads
    set_attention(model)
    cap = _Capture(cfg.num_hidden_layers, cfg.num_attention_heads, cfg.num_key_value_heads, d, next(model.parameters()).device,
                   with_values)
    _STATE["capture"] = cap
    try:
        for ids in prompts:
            model(input_ids=ids, use_cache=False)
    finally:
        _STATE["capture"] = None
    return cap.moments


def build_cache(model, moments: KeyPathMoments, k_bits: float, layer0_full_precision: bool = True, eps: float = 1e-4,
                v_bits: int | None = None, max_bits: int = 4):
    """Fit one compressor per (layer, kv head) from the calibration moments (symmetrised Σ_Q Σ_K
    basis, water-fill at ``k_bits`` average, at most ``max_bits`` bits per coordinate: 8 is the
    reference's own cap, storable while at most 32 coordinates of a head go above 4 bits), attach a
    packed cache layer to every attention module and return the ``Cache`` to pass as ``past_key_values``.
    ``v_bits``: values are packed as well (eigenbasis of Cov[V], water-fill, mean-centred: the
    reference's ``v_eigen_waterfill``); the moments must then have been taken ``with_values``.  The
    new token's value is then read from its codes in its own step already (the reference compresses
    it after that step); its key follows ``OWN_KEY_EXACT`` as with bf16 values."""
    cache_utils, _, _, _ = _transformers()
    set_attention(model)
    layer_cls = make_paged_layer_class()
    stats = moments.finalize()
    device = next(model.parameters()).device
    layers, comps_by_layer, v_comps_by_layer = [], {}, {}
    mods = attention_modules(model)
    for m in mods:
        L = m.layer_idx
        if L == 0 and layer0_full_precision:
            layers.append(cache_utils.DynamicLayer())
            m._jqk_layer = None
            continue
        comps = [PerCoordCompressor.fit(stats["sigma_q"][L, h].cpu(), stats["sigma_k"][L, h].cpu(), float(k_bits),
                                        max_bits=int(max_bits), basis="r_sym", eps=eps) for h in range(stats["sigma_k"].shape[1])]
        comps_by_layer[L] = comps
        v_tables = None
        if v_bits is not None:
            if "cov_v" not in stats:
                raise ValueError("v_bits needs moments taken with_values=True")
            d = stats["cov_v"].shape[-1]
            v_comps = [build_v_compressor("v_eigen_waterfill", cov_v_for_head=stats["cov_v"][L, h].cpu(), head_dim=d,
                                          bits=int(v_bits), seed=42, mu_v_for_head=stats["mu_v"][L, h].cpu(), max_bits=int(max_bits))
                       for h in range(stats["cov_v"].shape[1])]
            v_comps_by_layer[L] = v_comps
            v_tables = HeadTables.from_compressors([c.inner for c in v_comps], device=device,
                                                   center=torch.stack([c.mu for c in v_comps]))
        layer = layer_cls(HeadTables.from_compressors(comps, device=device), v_tables)
        layers.append(layer)
        m._jqk_layer = layer
    cache = cache_utils.Cache(layers=layers)
    cache.jqk_compressors = comps_by_layer
    cache.jqk_v_compressors = v_comps_by_layer
    return cache
