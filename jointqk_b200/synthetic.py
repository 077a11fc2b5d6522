"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configs.

The reference evaluates on activations captured from Qwen3-8B / Llama-3.1-8B on LongBench
prompts; neither the models nor the data are available offline, so these generators stand in
for them.  Every tensor is a deterministic function of ``(config, layer, head)`` through
``config_seed``.
"""

from __future__ import annotations

import math

import torch

from .codebooks import generate_rotation_matrix

HEAD_DIM = 128


def config_seed(config: int, layer: int = 0, head: int = 0) -> int:
    return 20260504 + 1000 * config + 10 * layer + head


def _randn(shape, seed: int, device) -> torch.Tensor:
    """Standard normal fp32 from a generator on ``device`` (CPU and CUDA streams differ; each is
    reproducible on its own)."""
    dev = torch.device(device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    return torch.randn(shape, generator=gen, device=dev, dtype=torch.float32)


def spectrum_keys(n_tokens: int, seed: int, n_outliers: int = 4, outlier_scale: float = 15.0,
                  device="cpu", dtype=torch.float32, d: int = HEAD_DIM) -> torch.Tensor:
    """Keys ``k = U diag(sqrt(lam)) z`` with ``lam_j = exp(-j/20)``, ``U`` the seeded rotation of
    the reference (quantization.py:53-62), and ``n_outliers`` seeded channels scaled up."""
    U = generate_rotation_matrix(d, seed=seed).to(device)
    lam = torch.exp(-torch.arange(d, dtype=torch.float32, device=device) / 20.0)
    z = _randn((n_tokens, d), seed + 1, device)
    k = (z * lam.sqrt()) @ U.T
    if n_outliers:
        g = torch.Generator(device="cpu")
        g.manual_seed(seed + 2)
        ch = torch.randperm(d, generator=g)[:n_outliers].to(device)
        k[:, ch] *= outlier_scale
    return k.to(dtype)


def second_moment(x: torch.Tensor) -> torch.Tensor:
    """Uncentred second moment x^T x / N in fp64 -> fp32, on the CPU (host-side fit input)."""
    xd = x.double()
    return ((xd.T @ xd) / x.shape[0]).float().cpu()


def fit_sigma_k_heads(keys: torch.Tensor, b_avg: float, max_bits: int = 4, eps: float = 1e-4):
    """keys (H, N, d) -> (compressors, sigma_k (H, d, d)): Sigma_K eigenbasis and water-fill on its
    variances, the fit the parity config prescribes."""
    from .compressor import PerCoordCompressor   # binds the CUDA library; the generators above do not

    sig = torch.stack([second_moment(keys[h].float()) for h in range(keys.shape[0])])
    comps = [PerCoordCompressor.fit(None, sig[h], b_avg, max_bits=max_bits, basis="sigma_k", eps=eps)
             for h in range(keys.shape[0])]
    return comps, sig


def retrieval_queries(keys: torch.Tensor, sigma_k: torch.Tensor, n_queries: int, seed: int):
    """``q = 0.8 k_j + 0.6 n`` with ``n ~ N(0, Sigma_K)`` and ``j`` uniform; returns (q, j)."""
    N, d = keys.shape
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    j = torch.randint(0, N, (n_queries,), generator=g)
    evals, evecs = torch.linalg.eigh(sigma_k.double())
    z = torch.randn(n_queries, d, generator=g, dtype=torch.float64)
    n = (z * evals.clamp_min(0).sqrt()) @ evecs.T
    q = 0.8 * keys[j.to(keys.device)].double().cpu() + 0.6 * n
    return q.float(), j


def correlated_qk(n_tokens: int, n_q_heads: int, n_kv_heads: int, seed: int, device="cpu",
                  dtype=torch.bfloat16, d: int = HEAD_DIM):
    """Calibration inputs: k ~ N(0, I), q_g = k A + 0.5 noise for every q head of the group, with a
    seeded A of spectral norm 1.  Returns q (Hq, T, d), k (Hkv, T, d)."""
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    A = torch.randn(d, d, generator=g)
    A = (A / torch.linalg.matrix_norm(A, ord=2)).to(device)
    group = n_q_heads // n_kv_heads
    k = _randn((n_kv_heads, n_tokens, d), seed + 1, device)
    noise = _randn((n_q_heads, n_tokens, d), seed + 2, device)
    q = (k @ A).repeat_interleave(group, dim=0) + 0.5 * noise
    return q.to(dtype), k.to(dtype)


def uniform_lengths(n_seqs: int, lo: int, hi: int, seed: int) -> list[int]:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return [int(x) for x in torch.randint(lo, hi + 1, (n_seqs,), generator=g)]


def lpt_shards(lengths: list[int], n_shards: int) -> list[list[int]]:
    """Longest-processing-time assignment of sequences to ranks; returns index lists."""
    order = sorted(range(len(lengths)), key=lambda i: -lengths[i])
    load = [0] * n_shards
    out: list[list[int]] = [[] for _ in range(n_shards)]
    for i in order:
        r = min(range(n_shards), key=lambda s: (load[s], s))
        out[r].append(i)
        load[r] += lengths[i]
    return out
