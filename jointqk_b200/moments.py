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
                     sk_sum: torch.Tensor | None, cqk_sum: torch.Tensor | None,
                     q_sum: torch.Tensor | None = None, k_sum: torch.Tensor | None = None,
                     max_chain_tokens: int = 0) -> None:
    """``+=`` the sums of one layer in one pass over the inputs.  q (Hq, T, d) or None, k (Hkv, T, d);
    second moments fp32 (Hkv, d, d); first moments ``q_sum`` (pooled over the group) and ``k_sum``
    fp32 (Hkv, d).  ``max_chain_tokens`` bounds the length of an fp32 running sum inside the tensor
    core (0 = library default); shorter is more accurate and slower."""
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
    for o in (q_sum, k_sum):
        if o is not None and (o.dtype != torch.float32 or not o.is_contiguous() or tuple(o.shape) != (n_kv, d)):
            raise ValueError(f"first-moment outputs must be contiguous fp32 ({n_kv}, {d})")
    p = lambda t: None if t is None else t.data_ptr()
    _native.check(_native.lib.jqk_moments_accumulate(
        p(q), k.data_ptr(), _native.torch_dtype_code(k.dtype), T,
        0 if q is None else q.stride(0), k.stride(0), n_q, n_kv, d,
        p(sq_sum), p(sk_sum), p(cqk_sum), p(q_sum), p(k_sum), int(max_chain_tokens),
        _status_word(dev).data_ptr(), 4, torch.cuda.current_stream(dev).cuda_stream))


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


def _moment_sums(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """(sum_t x x^T, sum_t x) per head for x (..., H, T, d) -> fp32 (..., H, d, d), (..., H, d) on
    x's CUDA device, both from one pass of the kernel."""
    lead = x.shape[:-3]
    H, T, d = x.shape[-3:]
    flat = x.reshape(-1, H, T, d)
    out = torch.zeros((flat.shape[0], H, d, d), dtype=torch.float32, device=x.device)
    first = torch.zeros((flat.shape[0], H, d), dtype=torch.float32, device=x.device)
    for i in range(flat.shape[0]):
        xi = _as_kernel_input(flat[i], x.device)
        accumulate_layer(None, xi, None, out[i], None, None, first[i])
    return out.reshape(lead + (H, d, d)), first.reshape(lead + (H, d))


def compute_query_moments(query_tensor: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(L, H, T, d) -> (mean, cov, second moment) over tokens, fp32, on the input's device."""
    src = query_tensor.device
    q = query_tensor.to(_dev(query_tensor))
    n = q.shape[2]
    outer, first = _moment_sums(q)
    check_status(q.device)
    mean, second = first / n, outer / n
    cov = second - torch.einsum("lhd,lhe->lhde", mean, mean)
    return mean.to(src), cov.to(src), second.to(src)


class QueryMomentsAccumulator:
    def __init__(self) -> None:
        self.sum_q: torch.Tensor | None = None
        self.sum_outer: torch.Tensor | None = None
        self.total_count = 0

    def update(self, query_tensor: torch.Tensor) -> None:
        q = query_tensor.to(_dev(query_tensor))
        q_outer, q_sum = _moment_sums(q)
        if self.sum_q is None:
            self.sum_q, self.sum_outer = q_sum, q_outer
        else:
            self.sum_q += q_sum
            self.sum_outer += q_outer
        self.total_count += q.shape[2]

    def finalize(self) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        if self.sum_q is None or self.sum_outer is None or self.total_count == 0:
            raise RuntimeError("No query statistics were accumulated.")
        check_status(self.sum_q.device)
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
        check_status(self.sum_qk.device)
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
    check_status(dev)
    return (sq / (bsz * (n_q // num_kv_heads) * T)).to(future_queries.device)


@torch.no_grad()
def compute_moments_from_tensors(q_post: torch.Tensor, k_post: torch.Tensor, v: torch.Tensor | None,
                                 prompt_length: int, device: torch.device | str | None = None, *,
                                 gpu_budget_bytes: int = 8 << 30) -> dict:
    """Per-(layer, kv_head) sums over the first ``prompt_length`` tokens.

    q_post (L, Hq, T_full, d); k_post, v (L, Hkv, T_full, d).  Returns CPU fp32 tensors under
    the reference's keys (``sq_sum``, ``sk_sum``, ``cqk_sum``, ``sv_sum``, ``sum_q``, ``sum_k``,
    ``sum_v``) plus shape metadata.  Second and first moments of a layer come from one pass of the
    kernel over q and k (and one over v).  ``gpu_budget_bytes`` is accepted for signature
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
        accumulate_layer(ql, kl, sq[l], sk[l], cqk[l], sum_q[l], sum_k[l])
        if v is not None:
            vl = _as_kernel_input(v[l, :, :tokens, :], dev)
            accumulate_layer(None, vl, None, sv[l], None, None, sum_v[l])
    check_status(dev)
    return {
        "tokens": tokens, "n_layers": n_layers, "n_kv_heads": n_kv, "n_q_heads": n_q, "group": group,
        "head_dim": d, "sq_sum": sq.cpu(), "sk_sum": sk.cpu(), "cqk_sum": cqk.cpu(), "sv_sum": sv.cpu(),
        "sum_q": sum_q.cpu(), "sum_k": sum_k.cpu(), "sum_v": sum_v.cpu(),
    }


class KeyPathMoments:
    """Streaming sums for all layers, sharded over ranks by tokens: Sigma_Q / Sigma_K / C_QK and the
    first moments of q and k; with ``with_values=True`` also the second and first moments of V
    (compute_stats.py:124,127), which the V-side compressor is fitted from.

    ``sums`` is one fp32 block ``[L][3 or 4][Hkv][d][d]`` (sq, sk, cqk, then sv) and ``firsts`` one
    block ``[L][2 or 3][Hkv][d]`` (sum_q pooled over the group, sum_k, then sum_v), so that one
    all-reduce per block covers a rank's whole contribution."""

    def __init__(self, n_layers: int, n_q_heads: int, n_kv_heads: int, head_dim: int, device,
                 with_values: bool = False, max_chain_tokens: int = 0, first_moments: bool = True) -> None:
        if n_q_heads % n_kv_heads != 0:
            raise ValueError(f"GQA mismatch: q_heads={n_q_heads}, kv_heads={n_kv_heads}")
        self.n_layers, self.n_q_heads, self.n_kv_heads, self.d = n_layers, n_q_heads, n_kv_heads, head_dim
        self.group = n_q_heads // n_kv_heads
        self.with_values = bool(with_values)
        # first moments ride on the same pass but are not free: their products re-read the operand tiles
        # from shared memory (about 15 % of the kernel time on the calibration shape); a caller that only
        # wants Sigma_Q / Sigma_K / C_QK switches them off
        self.first_moments = bool(first_moments)
        self.max_chain_tokens = int(max_chain_tokens)
        n_mat = 4 if with_values else 3
        self.sums = torch.zeros((n_layers, n_mat, n_kv_heads, head_dim, head_dim), dtype=torch.float32, device=device)
        self.firsts = torch.zeros((n_layers, n_mat - 1, n_kv_heads, head_dim), dtype=torch.float32, device=device)
        self._tokens = torch.zeros(n_layers, dtype=torch.float64, device=device)
        self._pending = [0] * n_layers       # token counts not yet added on the device (no launch per update)

    @property
    def tokens(self) -> torch.Tensor:
        """Tokens seen per layer, fp64 on the accumulator's device."""
        if any(self._pending):
            self._tokens += torch.tensor(self._pending, dtype=torch.float64).to(self._tokens.device)
            self._pending = [0] * self.n_layers
        return self._tokens

    def update(self, layer: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor | None = None) -> None:
        """q (Hq, T, d), k (Hkv, T, d) and, when values are tracked, v (Hkv, T, d) of one layer's
        chunk of tokens."""
        if self.sums.device.type != "cuda":
            raise RuntimeError("jointqk_b200: the moment kernels have no CPU implementation")
        fm = self.first_moments
        accumulate_layer(q, k, self.sums[layer, 0], self.sums[layer, 1], self.sums[layer, 2],
                         self.firsts[layer, 0] if fm else None, self.firsts[layer, 1] if fm else None,
                         self.max_chain_tokens)
        if self.with_values:
            if v is None:
                raise ValueError("this accumulator tracks values: pass v")
            accumulate_layer(None, v, None, self.sums[layer, 3], None, None, self.firsts[layer, 2] if fm else None,
                             self.max_chain_tokens)
        self._pending[layer] += int(k.shape[1])

    def all_reduce(self, group=None) -> None:
        """Sum the partial sums and token counts over the ranks of ``group``."""
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(self.sums, op=dist.ReduceOp.SUM, group=group)
            dist.all_reduce(self.firsts, op=dist.ReduceOp.SUM, group=group)
            dist.all_reduce(self.tokens, op=dist.ReduceOp.SUM, group=group)

    def finalize(self) -> dict[str, torch.Tensor]:
        """Divide once (compute_stats.py:235-244 / analyze_bases.py:264-279): second moments, means
        and covariances per (layer, kv head)."""
        if self.sums.device.type == "cuda":
            check_status(self.sums.device)
        if float(self.tokens.min()) <= 0:
            raise RuntimeError("no calibration tokens accumulated")
        tok = self.tokens.clamp_min(1).float()
        t4, t3 = tok.view(-1, 1, 1, 1), tok.view(-1, 1, 1)
        outer = lambda m: torch.einsum("lhd,lhe->lhde", m, m)
        out = {
            "sigma_q": self.sums[:, 0] / (self.group * t4),
            "sigma_k": self.sums[:, 1] / t4,
            "cqk": self.sums[:, 2] / t4,
            "total_tokens": self.tokens.clone(),
        }
        if self.with_values:
            out["sigma_v"] = self.sums[:, 3] / t4
        if self.first_moments:
            out["mu_q"] = self.firsts[:, 0] / (self.group * t3)
            out["mu_k"] = self.firsts[:, 1] / t3
            out["cov_q"] = out["sigma_q"] - outer(out["mu_q"])
            out["cov_k"] = out["sigma_k"] - outer(out["mu_k"])
            if self.with_values:
                out["mu_v"] = self.firsts[:, 2] / t3
                out["cov_v"] = out["sigma_v"] - outer(out["mu_v"])
        return out

    def calibration_artifacts(self, eps: float = 1e-4, source: str = "jointqk_b200") -> tuple[dict, dict | None]:
        """The two dictionaries the reference writes with ``torch.save`` as ``cca_stats_*.pt`` and
        ``v_stats_*.pt`` (scripts/build_calibration_artifacts_from_pool.py:108-127,148-163), on the
        CPU, so that its press (jointqk_press.py:124-233) can load a calibration made here.  The
        CCA-only fields the press constructor touches but ``r_sym_waterfill`` never reads are the
        same placeholders the reference writes.  The second dictionary is None when values were not
        tracked."""
        import time

        from .basis import jointqk_basis

        if not self.first_moments:
            raise RuntimeError("the artefacts need means and covariances: accumulate with first_moments=True")
        fin = {k: v.float().cpu() for k, v in self.finalize().items()}
        L, H, d = self.n_layers, self.n_kv_heads, self.d
        if len({int(t) for t in self.tokens.tolist()}) != 1:
            raise RuntimeError("layers saw different token counts")
        total = int(self.tokens[0].item())
        eye = torch.eye(d, dtype=torch.float32).expand(L, H, d, d).contiguous()
        zeros_diag = torch.zeros(L, H, d, dtype=torch.float32)
        cca = {
            "sigma_q": fin["sigma_q"], "sigma_k": fin["sigma_k"],
            "R_sym": jointqk_basis(fin["sigma_q"], fin["sigma_k"], eps=float(eps)).float(),
            "cqk": torch.zeros_like(fin["sigma_q"]), "rho": zeros_diag, "P_K": eye, "P_K_inv": eye, "P_Q": eye,
            "mq_eigvals": zeros_diag, "mq_eigvecs": eye, "V_h": eye,
            "n_layers": L, "n_kv_heads": H, "head_dim": d, "total_prefill_tokens": total,
            "calibration_source": source, "calibration_date": time.strftime("%Y-%m-%d"),
        }
        v_art = None
        if self.with_values:
            v_art = {"cov_v": fin["cov_v"], "mu_v": fin["mu_v"], "sigma_v": fin["sigma_v"],
                     "metadata": {"n_layers": L, "n_kv_heads": H, "head_dim": d, "n_examples": None,
                                  "total_token_count": total, "prefill_only": True, "bundle": source, "version": 2}}
        return cca, v_art
