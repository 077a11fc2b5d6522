"""Host-side basis fit for the key compressor.

* ``regularize_batch`` / ``eigvec_desc`` / ``jointqk_basis``
      -- experiments/stage1/calibration/analyze_bases.py:107-128
* ``repeat_kv_states`` (GQA expansion) -- experiments/stage1/toolkit/metric_transform.py:21-27

The eigendecompositions stay on the host in torch (``torch.linalg.eigh``): they run once per
model, and eigenvector signs are implementation-defined, so a device solver would yield
mirrored codes.  Only the moments that feed them are accumulated on the GPU.
"""

from __future__ import annotations

import torch


def _sym(x: torch.Tensor) -> torch.Tensor:
    xf = x.float()
    return 0.5 * (xf + xf.transpose(-1, -2))


def regularize_batch(cov: torch.Tensor, eps: float) -> torch.Tensor:
    """``sym(cov) + eps * max(trace/d, 1e-12) * I`` over leading batch dims."""
    d = cov.shape[-1]
    s = _sym(cov)
    tr = s.diagonal(dim1=-2, dim2=-1).sum(-1)
    eye = torch.eye(d, dtype=s.dtype, device=s.device)
    return s + (eps * (tr / d).clamp_min(1e-12)).unsqueeze(-1).unsqueeze(-1) * eye


def _eigvecs_descending(sym: torch.Tensor) -> torch.Tensor:
    vals, vecs = torch.linalg.eigh(sym)
    order = torch.argsort(vals, dim=-1, descending=True)
    return torch.gather(vecs, -1, order.unsqueeze(-2).expand(*vecs.shape[:-1], -1))


def eigvec_desc(cov: torch.Tensor, eps: float) -> torch.Tensor:
    """Eigenvectors (columns) of the regularised covariance, eigenvalues descending."""
    return _eigvecs_descending(regularize_batch(cov, eps))


def jointqk_basis(sigma_q: torch.Tensor, sigma_k: torch.Tensor, eps: float) -> torch.Tensor:
    """Joint Q-K eigenbasis ``R_sym = eigvec_desc(sym(reg(Sigma_Q) @ reg(Sigma_K)))``."""
    sq = regularize_batch(sigma_q, eps)
    sk = regularize_batch(sigma_k, eps)
    return _eigvecs_descending(_sym(sq @ sk))


def repeat_kv_states(keys: torch.Tensor, num_query_heads: int) -> torch.Tensor:
    """Expand ``(B, Hkv, S, d)`` so that kv head h serves q heads ``h*g .. h*g+g-1``."""
    bsz, n_kv, seq, dim = keys.shape
    if num_query_heads == n_kv:
        return keys
    g = num_query_heads // n_kv
    return keys[:, :, None, :, :].expand(bsz, n_kv, g, seq, dim).reshape(bsz, num_query_heads, seq, dim)
