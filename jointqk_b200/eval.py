"""Attention-retention metrics computed from packed keys.

Same metric definitions as ``compute_attention_metrics`` (experiments/stage1/toolkit/eval.py:11-38)
and ``measure_top1`` (experiments/stage1/scripts/measure_decode_q_top1.py:187-220); the
candidate logits come from the lookup-table score kernel instead of a matmul against
reconstructed keys, the reference logits from a plain fp32 matmul against the original keys.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from . import paged
from .basis import repeat_kv_states


@torch.no_grad()
def packed_logits(packed: paged.PackedKeys, future_queries: torch.Tensor) -> torch.Tensor:
    """(B, Hq, Tq, d) queries against packed keys -> (B, Hq, Tq, S) logits q.k_hat/sqrt(d)."""
    dev = packed.tables.device
    q = future_queries.to(dev)
    if q.dtype not in (torch.float32, torch.bfloat16, torch.float16):
        q = q.float()
    return paged.score(packed, q)


@torch.no_grad()
def compute_attention_metrics(future_queries: torch.Tensor, reference_keys: torch.Tensor,
                              candidate: paged.PackedKeys) -> dict[str, float]:
    """future_queries (B, Hq, Tq, d), reference_keys (B, Hkv, S, d), candidate = packed keys."""
    dim = reference_keys.shape[-1]
    dev = candidate.tables.device
    q = future_queries.to(dev).float()
    ref = repeat_kv_states(reference_keys.to(dev), q.shape[1]).float()
    real = torch.matmul(q, ref.transpose(-2, -1)) / math.sqrt(dim)
    approx = packed_logits(candidate, future_queries)
    diff = approx - real
    real_flat = real.reshape(-1, real.shape[-1])
    approx_flat = approx.reshape(-1, approx.shape[-1])
    k = min(5, real_flat.shape[-1])
    real_top1 = real_flat.argmax(dim=-1)
    approx_top1 = approx_flat.argmax(dim=-1)
    approx_topk = approx_flat.topk(k, dim=-1).indices
    return {
        "logit_mse": diff.pow(2).mean().item(),
        "logit_cosine": F.cosine_similarity(real_flat, approx_flat, dim=-1).mean().item(),
        "top1_match": (real_top1 == approx_top1).float().mean().item(),
        "top5_containment": (approx_topk == real_top1.unsqueeze(-1)).any(dim=-1).float().mean().item(),
    }
