"""Calibration moment accumulators backed by the CUDA contraction kernel.

Interfaces follow the reference:

* ``QueryMomentsAccumulator`` / ``CrossMomentsAccumulator`` / ``compute_query_moments`` /
  ``compute_grouped_query_second_moment`` -- experiments/stage1/toolkit/moments.py:51-132
* ``compute_moments_from_tensors`` -- experiments/stage1/calibration/compute_stats.py:51-154
* ``KeyPathMoments`` is the streaming form of ``_accumulate_calibration_stats``
  (experiments/stage1/run_cca_vs_waterfill_study.py:203-260): sums are kept in fp32, reduced
  across ranks with one all-reduce (the reference adds per-shard sums from files,
  compute_stats.py:224-241), and divided once at the end.

Conventions kept: Sigma_Q is the uncentred second moment pooled over the q heads of a group
(divided by ``group * tokens``), C_QK uses the group-mean query, Sigma_K and C_QK are divided
by ``tokens``.
"""

from __future__ import annotations

import torch

from . import _native


def _dev(t: torch.Tensor) -> torch.device:
    if t.is_cuda:
        return t.device
    if not torch.cuda.is_available():
        raise RuntimeError("jointqk_b200 needs a CUDA device: the moment kernels have no CPU implementation")
    return torch.device("cuda", torch.cuda.current_device())


def _as_kernel_input(x: torch.Tensor, dev: torch.device) -> torch.Tensor:
    """(H, T, d) view with contiguous (T, d) rows on ``dev`` in a dtype the kernel reads."""
    if x.dtype not in (torch.float32, torch.bfloat16, torch.float16):
        x = x.float()
    x = x.to(dev)
    if x.stride(-1) != 1 or x.stride(-2) != x.shape[-1]:
        x = x.contiguous()
    return x


def accumulate_layer(q: torch.Tensor | None, k: torch.Tensor, sq_sum: torch.Tensor | None,
                     sk_sum: torch.Tensor | None, cqk_sum: torch.Tensor | None) -> None:
    """``+=`` the sums of one layer.  q (Hq, T, d) or None, k (Hkv, T, d); outputs fp32 (Hkv, d, d)."""
    dev = k.device
    n_kv, T, d = k.shape
    n_q = q.shape[0] if q is not None else n_kv
    if q is not None and (q.shape[1] != T or q.shape[2] != d or q.dtype != k.dtype):
        raise ValueError("q and k must share tokens, head_dim and dtype")
    if n_q % n_kv != 0:
        raise ValueError(f"GQA mismatch: q_heads={n_q}, kv_heads={n_kv}")
    for o in (sq_sum, sk_sum, cqk_sum):
        if o is not None and (o.dtype != torch.float32 or not o.is_contiguous() or tuple(o.shape) != (n_kv, d, d)):
            raise ValueError(f"moment outputs must be contiguous fp32 ({n_kv}, {d}, {d})")
    _native.check(_native.lib.jqk_moments_accumulate(
        None if q is None else q.data_ptr(), k.data_ptr(), _native.torch_dtype_code(k.dtype), T,
        0 if q is None else q.stride(0), k.stride(0), n_q, n_kv, d,
        None if sq_sum is None else sq_sum.data_ptr(), None if sk_sum is None else sk_sum.data_ptr(),
        None if cqk_sum is None else cqk_sum.data_ptr(), _status_word(dev).data_ptr(), 4,
        torch.cuda.current_stream(dev).cuda_stream))


_STATUS: dict = {}


def _status_word(dev: torch.device) -> torch.Tensor:
    """Per-device status word the moment kernels OR their flags into."""
    key = (dev.type, dev.index)
    if key not in _STATUS:
        _STATUS[key] = torch.zeros(1, dtype=torch.int32, device=dev)
    return _STATUS[key]


def check_status(dev: torch.device | None = None) -> None:
    """Raise if a moment kernel reported an expired bounded wait (synchronises)."""
    for key, word in _STATUS.items():
        if dev is not None and key != (dev.type, dev.index):
            continue
        if int(word.item()) & _native.STATUS_WAIT_EXPIRED:
            raise RuntimeError("jointqk_b200: a bounded device-side wait expired in the moment kernel")


def _second_moment_sum(x: torch.Tensor) -> torch.Tensor:
    """sum_t x x^T per head for x (..., H, T, d) -> fp32 (..., H, d, d) on x's CUDA device."""
    lead = x.shape[:-3]
    H, T, d = x.shape[-3:]
    flat = x.reshape(-1, H, T, d)
    out = torch.zeros((flat.shape[0], H, d, d), dtype=torch.float32, device=x.device)
    for i in range(flat.shape[0]):
        xi = _as_kernel_input(flat[i], x.device)
        accumulate_layer(None, xi, None, out[i], None)
    return out.reshape(lead + (H, d, d))


def compute_query_moments(query_tensor: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(L, H, T, d) -> (mean, cov, second moment) over tokens, fp32, on the input's device."""
    src = query_tensor.device
    q = query_tensor.to(_dev(query_tensor))
    n = q.shape[2]
    mean = q.float().mean(dim=2)
    second = _second_moment_sum(q) / n
    cov = second - torch.einsum("lhd,lhe->lhde", mean, mean)
    return mean.to(src), cov.to(src), second.to(src)


class QueryMomentsAccumulator:
    def __init__(self) -> None:
        self.sum_q: torch.Tensor | None = None
        self.sum_outer: torch.Tensor | None = None
        self.total_count = 0

    def update(self, query_tensor: torch.Tensor) -> None:
        q = query_tensor.to(_dev(query_tensor))
        q_sum = q.float().sum(dim=2)
        q_outer = _second_moment_sum(q)
        if self.sum_q is None:
            self.sum_q, self.sum_outer = q_sum, q_outer
        else:
            self.sum_q += q_sum
            self.sum_outer += q_outer
        self.total_count += q.shape[2]

    def finalize(self) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        if self.sum_q is None or self.sum_outer is None or self.total_count == 0:
            raise RuntimeError("No query statistics were accumulated.")
        mean = self.sum_q / self.total_count
        second = self.sum_outer / self.total_count
        cov = second - torch.einsum("lhd,lhe->lhde", mean, mean)
        return mean, cov, second


class CrossMomentsAccumulator:
    """Streaming C_QK = (1/N) sum_t mean_g(q_g,t) k_t^T per kv head (moments.py:86-120)."""

    def __init__(self) -> None:
        self.sum_qk: torch.Tensor | None = None
        self.total_count = 0

    def update(self, queries: torch.Tensor, keys: torch.Tensor, num_kv_heads: int) -> None:
        bsz, n_q, seq_len, dim = queries.shape
        if n_q % num_kv_heads != 0:
            raise ValueError(f"Cannot group {n_q} query heads into {num_kv_heads} KV heads evenly.")
        dev = _dev(keys)
        if self.sum_qk is None:
            self.sum_qk = torch.zeros((num_kv_heads, dim, dim), dtype=torch.float32, device=dev)
        dt = keys.dtype if keys.dtype == queries.dtype else torch.float32
        for b in range(bsz):
            accumulate_layer(_as_kernel_input(queries[b].to(dt), dev), _as_kernel_input(keys[b].to(dt), dev),
                             None, None, self.sum_qk)
        self.total_count += bsz * seq_len

    def finalize(self) -> torch.Tensor:
        if self.sum_qk is None or self.total_count == 0:
            raise RuntimeError("No cross-moment statistics were accumulated.")
        return self.sum_qk / self.total_count


def compute_grouped_query_second_moment(future_queries: torch.Tensor, num_kv_heads: int) -> torch.Tensor:
    """(B, Hq, T, d) -> (Hkv, d, d): every q head of a group counted as a sample (moments.py:123-132)."""
    bsz, n_q, T, dim = future_queries.shape
    if n_q % num_kv_heads != 0:
        raise ValueError(f"Cannot group {n_q} query heads into {num_kv_heads} KV heads evenly.")
    dev = _dev(future_queries)
    sq = torch.zeros((num_kv_heads, dim, dim), dtype=torch.float32, device=dev)
    for b in range(bsz):
        qb = _as_kernel_input(future_queries[b], dev)
        kb = qb[:: n_q // num_kv_heads]                      # any (Hkv, T, d) tensor; only sq is requested
        accumulate_layer(qb, kb if kb.stride(-2) == dim else kb.contiguous(), sq, None, None)
    return (sq / (bsz * (n_q // num_kv_heads) * T)).to(future_queries.device)


@torch.no_grad()
def compute_moments_from_tensors(q_post: torch.Tensor, k_post: torch.Tensor, v: torch.Tensor | None,
                                 prompt_length: int, device: torch.device | str | None = None, *,
                                 gpu_budget_bytes: int = 8 << 30) -> dict:
    """Per-(layer, kv_head) sums over the first ``prompt_length`` tokens.

    q_post (L, Hq, T_full, d); k_post, v (L, Hkv, T_full, d).  Returns CPU fp32 tensors under
    the reference's keys (``sq_sum``, ``sk_sum``, ``cqk_sum``, ``sv_sum``, ``sum_q``, ``sum_k``,
    ``sum_v``) plus shape metadata.  ``gpu_budget_bytes`` is accepted for signature
    compatibility; the kernel reads the 16-bit inputs directly, so nothing is promoted."""
    n_layers, n_kv, _, d = (int(x) for x in k_post.shape)
    n_q = int(q_post.shape[1])
    tokens = int(prompt_length)
    if n_q % n_kv != 0:
        raise ValueError(f"GQA mismatch: q_heads={n_q}, kv_heads={n_kv}")
    group = n_q // n_kv
    dev = torch.device(device) if device is not None else _dev(k_post)
    if dev.type != "cuda":
        dev = _dev(k_post)
    shape = (n_layers, n_kv, d, d)
    sq = torch.zeros(shape, dtype=torch.float32, device=dev)
    sk = torch.zeros(shape, dtype=torch.float32, device=dev)
    cqk = torch.zeros(shape, dtype=torch.float32, device=dev)
    sv = torch.zeros(shape, dtype=torch.float32, device=dev)
    sum_q = torch.zeros((n_layers, n_kv, d), dtype=torch.float32, device=dev)
    sum_k = torch.zeros((n_layers, n_kv, d), dtype=torch.float32, device=dev)
    sum_v = torch.zeros((n_layers, n_kv, d), dtype=torch.float32, device=dev)
    for l in range(n_layers):
        ql = _as_kernel_input(q_post[l, :, :tokens, :], dev)
        kl = _as_kernel_input(k_post[l, :, :tokens, :], dev)
        if ql.dtype != kl.dtype:
            ql, kl = ql.float(), kl.float()
        accumulate_layer(ql, kl, sq[l], sk[l], cqk[l])
        sum_q[l] = ql.float().view(n_kv, group, tokens, d).sum(dim=(1, 2))
        sum_k[l] = kl.float().sum(dim=1)
        if v is not None:
            vl = _as_kernel_input(v[l, :, :tokens, :], dev)
            accumulate_layer(None, vl, None, sv[l], None)
            sum_v[l] = vl.float().sum(dim=1)
    return {
        "tokens": tokens, "n_layers": n_layers, "n_kv_heads": n_kv, "n_q_heads": n_q, "group": group,
        "head_dim": d, "sq_sum": sq.cpu(), "sk_sum": sk.cpu(), "cqk_sum": cqk.cpu(), "sv_sum": sv.cpu(),
        "sum_q": sum_q.cpu(), "sum_k": sum_k.cpu(), "sum_v": sum_v.cpu(),
    }


class KeyPathMoments:
    """Streaming Sigma_Q / Sigma_K / C_QK sums for all layers, sharded over ranks by tokens."""

    def __init__(self, n_layers: int, n_q_heads: int, n_kv_heads: int, head_dim: int, device) -> None:
        if n_q_heads % n_kv_heads != 0:
            raise ValueError(f"GQA mismatch: q_heads={n_q_heads}, kv_heads={n_kv_heads}")
        self.n_layers, self.n_q_heads, self.n_kv_heads, self.d = n_layers, n_q_heads, n_kv_heads, head_dim
        self.group = n_q_heads // n_kv_heads
        # one block so that a single all-reduce covers everything: [L][3][Hkv][d][d]
        self.sums = torch.zeros((n_layers, 3, n_kv_heads, head_dim, head_dim), dtype=torch.float32, device=device)
        self.tokens = torch.zeros(n_layers, dtype=torch.float64, device=device)

    def update(self, layer: int, q: torch.Tensor, k: torch.Tensor) -> None:
        """q (Hq, T, d), k (Hkv, T, d) of one layer's chunk of tokens."""
        accumulate_layer(q, k, self.sums[layer, 0], self.sums[layer, 1], self.sums[layer, 2])
        self.tokens[layer] += k.shape[1]

    def all_reduce(self, group=None) -> None:
        """Sum the partial sums and token counts over the ranks of ``group``."""
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(self.sums, op=dist.ReduceOp.SUM, group=group)
            dist.all_reduce(self.tokens, op=dist.ReduceOp.SUM, group=group)

    def finalize(self) -> dict[str, torch.Tensor]:
        tok = self.tokens.clamp_min(1).float().view(-1, 1, 1, 1)
        if float(self.tokens.min()) <= 0:
            raise RuntimeError("no calibration tokens accumulated")
        return {
            "sigma_q": self.sums[:, 0] / (self.group * tok),
            "sigma_k": self.sums[:, 1] / tok,
            "cqk": self.sums[:, 2] / tok,
            "total_tokens": self.tokens.clone(),
        }
