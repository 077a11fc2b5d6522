"""CPU restatement of the reference algorithm for the compress-then-attend key path.

TEST INFRASTRUCTURE ONLY.  Nothing in the product imports this module; it is used by
``tests/``, by ``__graft_entry__.smoke()`` as the checker and by ``bench.py`` for the timed
CPU baseline / reference arm.  It is written with the same torch CPU operations as the
reference (fp32 ``@``, ``argmin`` over ``|x - codebook|``, ``einsum``) so that its results and
its running time are those of the reference's own CPU path.

Pinned against the reference itself: ``tests/golden/make_golden.py`` imports a checkout of
the reference (given on ``PYTHONPATH``) and stores reference outputs as fixtures;
``tests/test_oracle_golden.py`` checks every function here against them.

Reference locations (paths inside Amir-zsh/JointQK):
  experiments/stage1/toolkit/per_coord_quantization.py   P = pcq
  experiments/stage1/toolkit/eval.py
  experiments/stage1/toolkit/metric_transform.py
  experiments/stage1/calibration/compute_stats.py
  experiments/stage1/run_cca_vs_waterfill_study.py
"""

from __future__ import annotations

import math

import numpy as np
import torch


# ---- fit-side objects --------------------------------------------------------------------
def codebooks_padded(bits: torch.Tensor, stds: torch.Tensor, unit_tables: dict[int, torch.Tensor]) -> torch.Tensor:
    """(d, K_max) codebook: row j = unit table(b_j) * float(std_j), +inf padded, 0-bit row [0.0]
    (pcq:96-110).  ``unit_tables[b]`` are the unit-variance Lloyd-Max centroids (pcq:25-40)."""
    b = [int(x) for x in bits.tolist()]
    k_max = max([1] + [2 ** x for x in b])
    cb = torch.full((len(b), k_max), float("inf"))
    for j, x in enumerate(b):
        if x == 0:
            cb[j, 0] = 0.0
        else:
            c = unit_tables[x] * float(stds[j])
            cb[j, : c.numel()] = c
    return cb


# ---- compression -------------------------------------------------------------------------
@torch.no_grad()
def transform(states: torch.Tensor, forward_map: torch.Tensor | None) -> torch.Tensor:
    """``states.float() @ forward_map`` on flattened rows (pcq:132-137)."""
    flat = states.reshape(-1, states.shape[-1]).float()
    return flat @ forward_map if forward_map is not None else flat


@torch.no_grad()
def nearest_codes(transformed: torch.Tensor, cb: torch.Tensor, chunk_bytes: int = 1 << 30) -> torch.Tensor:
    """``argmin_l |x_j - cb[j, l]|`` with torch's first-minimum tie rule, chunked along rows the
    way the reference bounds its (N, d, K) temporary (pcq:145-157)."""
    n, d = transformed.shape
    k_max = cb.shape[1]
    chunk = max(1, chunk_bytes // (d * k_max * 4))
    cbu = cb.unsqueeze(0)
    out = torch.empty((n, d), dtype=torch.long)
    for s in range(0, n, chunk):
        e = min(s + chunk, n)
        out[s:e] = (transformed[s:e].unsqueeze(-1) - cbu).abs().argmin(dim=-1)
    return out


@torch.no_grad()
def dequantise(codes: torch.Tensor, cb: torch.Tensor) -> torch.Tensor:
    """Centroid of every code (pcq:158-160)."""
    return torch.gather(cb.unsqueeze(0).expand(codes.shape[0], -1, -1), 2, codes.unsqueeze(-1)).squeeze(-1)


@torch.no_grad()
def roundtrip(states: torch.Tensor, cb: torch.Tensor, forward_map: torch.Tensor | None,
              inverse_map: torch.Tensor | None) -> tuple[torch.Tensor, torch.Tensor]:
    """Full reference ``roundtrip`` (pcq:123-165); also returns the integer codes."""
    x = transform(states, forward_map)
    codes = nearest_codes(x, cb)
    xh = dequantise(codes, cb)
    out = xh @ inverse_map if inverse_map is not None else xh
    return out.reshape(states.shape[:-1] + (states.shape[-1],)), codes.reshape(states.shape)


@torch.no_grad()
def batched_roundtrip(states: torch.Tensor, forward_maps: torch.Tensor, inverse_maps: torch.Tensor,
                      codebooks: torch.Tensor) -> torch.Tensor:
    """All heads with ``bmm`` (pcq:176-216); result in ``states.dtype``."""
    B, H, S, d = states.shape
    flat = states.float().permute(1, 0, 2, 3).reshape(H, B * S, d)
    x = torch.bmm(flat, forward_maps)
    cb = codebooks[:, None, :, :]                                   # (H, 1, d, K)
    idx = (x.unsqueeze(-1) - cb).abs().argmin(-1)
    xh = torch.take_along_dim(cb.expand(H, B * S, d, -1), idx.unsqueeze(-1), dim=-1).squeeze(-1)
    rec = torch.bmm(xh, inverse_maps).reshape(H, B, S, d).permute(1, 0, 2, 3)
    return rec.to(states.dtype)


@torch.no_grad()
def centred_roundtrip(states: torch.Tensor, mu: torch.Tensor, cb: torch.Tensor, forward_map: torch.Tensor,
                      inverse_map: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """The value side's mean-centring wrapper (v_compressor_adapter.py:64-72): subtract ``mu``,
    run the inner ``roundtrip``, add ``mu`` back.  Also returns the codes."""
    centred = states - mu
    recon, codes = roundtrip(centred, cb, forward_map, inverse_map)
    return recon + mu, codes


# ---- scoring / attention -----------------------------------------------------------------
def repeat_kv(keys: torch.Tensor, n_q_heads: int) -> torch.Tensor:
    """GQA expansion: kv head h serves q heads h*g .. h*g+g-1 (metric_transform.py:21-27)."""
    b, h, s, d = keys.shape
    if n_q_heads == h:
        return keys
    g = n_q_heads // h
    return keys[:, :, None].expand(b, h, g, s, d).reshape(b, n_q_heads, s, d)


@torch.no_grad()
def logits(queries: torch.Tensor, keys: torch.Tensor) -> torch.Tensor:
    """``q k^T / sqrt(d)`` in fp32: queries (B, Hq, Tq, d), keys (B, Hkv, S, d) (eval.py:17-21)."""
    k = repeat_kv(keys, queries.shape[1]).float()
    return torch.matmul(queries.float(), k.transpose(-2, -1)) / math.sqrt(keys.shape[-1])


@torch.no_grad()
def attention_metrics(queries: torch.Tensor, reference_keys: torch.Tensor, candidate_keys: torch.Tensor) -> dict:
    """top-1 match, top-5 containment, logit MSE and cosine (eval.py:11-38)."""
    real, approx = logits(queries, reference_keys), logits(queries, candidate_keys)
    rf, af = real.reshape(-1, real.shape[-1]), approx.reshape(-1, approx.shape[-1])
    r1, a1 = rf.argmax(-1), af.argmax(-1)
    topk = af.topk(min(5, rf.shape[-1]), dim=-1).indices
    return {
        "logit_mse": (approx - real).pow(2).mean().item(),
        "logit_cosine": torch.nn.functional.cosine_similarity(rf, af, dim=-1).mean().item(),
        "top1_match": (r1 == a1).float().mean().item(),
        "top5_containment": (topk == r1.unsqueeze(-1)).any(-1).float().mean().item(),
    }


@torch.no_grad()
def decode_attention(q: torch.Tensor, k_hat: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """``softmax(q k_hat^T / sqrt(d)) @ V.float()`` for one decode step.

    q (B, Hq, d), k_hat (B, Hkv, S, d) reconstructed keys, v (B, Hkv, S, d).  The reference has
    no standalone function for the output: it swaps the reconstructed keys into the HF cache
    (jointqk_press.py:306-307) and stock attention runs; the softmax form follows
    scripts/measure_softmax_kl.py:137-152."""
    s = logits(q.unsqueeze(2), k_hat)                               # (B, Hq, 1, S)
    p = torch.softmax(s, dim=-1)
    vv = repeat_kv(v, q.shape[1]).float()
    return torch.matmul(p, vv).squeeze(2)


# ---- calibration moments ------------------------------------------------------------------
@torch.no_grad()
def moment_sums(q: torch.Tensor, k: torch.Tensor) -> dict[str, torch.Tensor]:
    """Sums over tokens for q (L, Hq, T, d), k (L, Hkv, T, d) in fp32 (compute_stats.py:114-123):
    sq = sum_g q_g^T q_g, sk = k^T k, cqk = mean_g(q_g)^T k."""
    L, hq, T, d = q.shape
    hkv = k.shape[1]
    g = hq // hkv
    qf, kf = q.float(), k.float()
    sq = torch.einsum("lhsd,lhse->lhde", qf, qf).view(L, hkv, g, d, d).sum(dim=2)
    sk = torch.einsum("lhsd,lhse->lhde", kf, kf)
    cqk = torch.einsum("lhsd,lhse->lhde", qf.view(L, hkv, g, T, d).mean(dim=2), kf)
    return {"sq_sum": sq, "sk_sum": sk, "cqk_sum": cqk}


def normalise_moments(sums: dict[str, torch.Tensor], group: int, tokens: int) -> dict[str, torch.Tensor]:
    """Sigma_Q = sq/(group*tokens), Sigma_K = sk/tokens, C_QK = cqk/tokens
    (run_cca_vs_waterfill_study.py:257-259)."""
    return {"sigma_q": sums["sq_sum"] / (group * tokens), "sigma_k": sums["sk_sum"] / tokens,
            "cqk": sums["cqk_sum"] / tokens}


# ---- packed record format (numpy; the format itself is new in this build) -------------------
def pack_records(codes: np.ndarray, col_coord: np.ndarray, col_width: np.ndarray, col_bitpos: np.ndarray,
                 n_words: int) -> np.ndarray:
    """codes (N, d) in coordinate order -> (N, n_words) uint32 records."""
    out = np.zeros((codes.shape[0], n_words), dtype=np.uint64)
    for c in range(len(col_coord)):
        w = int(col_width[c])
        if w == 0:
            continue
        bp = int(col_bitpos[c])
        out[:, bp // 32] |= (codes[:, int(col_coord[c])].astype(np.uint64) & ((1 << w) - 1)) << (bp % 32)
    assert out.max(initial=0) < (1 << 32)
    return out.astype(np.uint32)


def unpack_records(records: np.ndarray, col_coord: np.ndarray, col_width: np.ndarray, col_bitpos: np.ndarray,
                   d: int) -> np.ndarray:
    out = np.zeros((records.shape[0], d), dtype=np.uint8)
    for c in range(len(col_coord)):
        w = int(col_width[c])
        if w == 0:
            continue
        bp = int(col_bitpos[c])
        out[:, int(col_coord[c])] = (records[:, bp // 32] >> np.uint32(bp % 32)) & np.uint32((1 << w) - 1)
    return out


def records_to_pages(records: np.ndarray, words_per_record: int) -> np.ndarray:
    """(N, n_words) -> (n_pages, words_per_record, 16) word-major pages of one head."""
    n, nw = records.shape
    n_pages = (n + 15) // 16
    pages = np.zeros((n_pages, words_per_record, 16), dtype=np.uint32)
    for t in range(n):
        pages[t // 16, :nw, t % 16] = records[t]
    return pages
