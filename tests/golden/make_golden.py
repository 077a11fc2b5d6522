"""Generate the golden fixtures in this directory from the reference implementation.

Run where a checkout of the reference is available, from the root of this repository:

    PYTHONPATH=<reference checkout>:. python tests/golden/make_golden.py

Every array saved under a name starting with ``ref_`` is an output of the reference's own
functions (Amir-zsh/JointQK, experiments/stage1/...); the other arrays are the seeded inputs
they were computed from.  The fixtures travel with the repository; the reference does not.
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parents[1]))

from experiments.stage1.calibration.analyze_bases import (  # noqa: E402
    allocate_bits as ref_allocate_bits, eigvec_desc as ref_eigvec_desc, jointqk_basis as ref_jointqk_basis,
    regularize_batch as ref_regularize_batch)
from experiments.stage1.calibration.compute_stats import compute_moments_from_tensors as ref_moments  # noqa: E402
from experiments.stage1.toolkit.eval import compute_attention_metrics as ref_metrics  # noqa: E402
from experiments.stage1.toolkit.metric_transform import repeat_kv_states as ref_repeat, water_fill as ref_water_fill  # noqa: E402
from experiments.stage1.toolkit.moments import (  # noqa: E402
    CrossMomentsAccumulator as RefCross, QueryMomentsAccumulator as RefQuery,
    compute_grouped_query_second_moment as ref_grouped, compute_query_moments as ref_query_moments)
from experiments.stage1.toolkit.per_coord_quantization import (  # noqa: E402
    PerCoordCompressor as RefCompressor, batched_roundtrip as ref_batched, build_method_compressor as ref_build,
    round_bits_to_integer as ref_round, stack_per_head as ref_stack, unit_gaussian_centroids as ref_unit)
from experiments.stage1.toolkit.quantization import generate_rotation_matrix as ref_rot, solve_lloyd_max as ref_lloyd  # noqa: E402

from jointqk_b200.synthetic import config_seed, retrieval_queries, second_moment, spectrum_keys  # noqa: E402


def _import_v_adapter():
    """The reference's V-side module imports TurboQuant's value compressor at module level
    (experiments/stage1/toolkit/v_compressor_adapter.py:43), a third-party package that is not part
    of the reference checkout.  The methods used here (v_eigen_uniform, v_eigen_waterfill, v_random
    and the mean-centring wrapper) never touch it, so a placeholder module satisfies the import."""
    import types

    if "turboquant_pytorch.compressors_v3" not in sys.modules:
        pkg, mod = types.ModuleType("turboquant_pytorch"), types.ModuleType("turboquant_pytorch.compressors_v3")

        class MSECompressor:  # never constructed by the methods exercised here
            def __init__(self, *a, **k):
                raise RuntimeError("TurboQuant is not available")

        mod.MSECompressor = MSECompressor
        pkg.compressors_v3 = mod
        sys.modules["turboquant_pytorch"], sys.modules["turboquant_pytorch.compressors_v3"] = pkg, mod
    from experiments.stage1.toolkit import v_compressor_adapter

    return v_compressor_adapter


def save(name: str, **arrays) -> None:
    out = {k: (v.detach().cpu().numpy() if isinstance(v, torch.Tensor) else np.asarray(v)) for k, v in arrays.items()}
    np.savez_compressed(HERE / f"{name}.npz", **out)
    print(name, {k: v.shape for k, v in out.items()})


def ref_codes(comp: RefCompressor, keys: torch.Tensor) -> torch.Tensor:
    """Integer codes through the public API only: with inverse_map = I the roundtrip returns the
    chosen centroid of every coordinate, whose position in the codebook row is the code."""
    probe = RefCompressor(comp.bits_int, comp.stds, forward_map=comp.forward_map, inverse_map=torch.eye(comp.d))
    cents = probe.roundtrip(keys)                                           # (N, d)
    eq = cents.unsqueeze(-1) == probe.codebooks_padded.unsqueeze(0)          # (N, d, K)
    assert bool(eq.any(-1).all())
    return eq.float().argmax(-1).to(torch.uint8)


def main() -> None:
    torch.manual_seed(0)
    # 1. Lloyd-Max tables
    save("centroids",
         **{f"ref_unit_{b}": ref_unit(b) for b in range(1, 9)},
         **{f"ref_lloyd128_{b}": ref_lloyd(128, b)[0] for b in range(1, 5)},
         ref_rotation_16_seed7=ref_rot(16, 7))

    # 2. water-fill and integer allocations on the config spectra
    keys = spectrum_keys(4096, config_seed(0, 0, 0))
    sig_k = second_moment(keys)
    R = ref_eigvec_desc(sig_k, 1e-4)
    var = (R.T @ sig_k @ R).diagonal().clamp_min(1e-30)
    g = torch.Generator().manual_seed(11)
    w = torch.rand(128, generator=g) + 0.1
    alloc = {"variances": var, "weights": w}
    for tag, v in (("var", var), ("wvar", var * w)):
        for b in (2, 3, 4):
            alloc[f"ref_waterfill_{tag}_{b}"] = ref_water_fill(v.unsqueeze(0), total_bits=float(b * 128)).squeeze(0)
            alloc[f"ref_alloc_{tag}_{b}_cap4"] = ref_allocate_bits(v.unsqueeze(0), b, max_coord_bits=4).squeeze(0)
            alloc[f"ref_alloc_{tag}_{b}_cap8"] = ref_allocate_bits(v.unsqueeze(0), b, max_coord_bits=8).squeeze(0)
        cont = ref_water_fill(v.unsqueeze(0), total_bits=2.5 * 128)
        alloc[f"ref_waterfill_{tag}_2p5"] = cont.squeeze(0)
        alloc[f"ref_round_{tag}_2p5"] = ref_round(cont, total_bits=int(2.5 * 128)).squeeze(0)
        alloc[f"ref_waterfill_{tag}_2_max4"] = ref_water_fill(v.unsqueeze(0), total_bits=256.0, max_bits=4.0).squeeze(0)
    small = torch.tensor([[4.0, 1.0, 0.25, 0.01]])
    alloc["small_variances"] = small
    alloc["ref_small_waterfill_8"] = ref_water_fill(small, total_bits=8.0)
    alloc["ref_small_alloc_2"] = ref_allocate_bits(small, 2, max_coord_bits=8)
    save("allocation", **alloc)

    # 3. bases
    g = torch.Generator().manual_seed(5)
    a = torch.randn(2, 16, 16, generator=g)
    b_ = torch.randn(2, 16, 16, generator=g)
    sq16, sk16 = a @ a.transpose(-1, -2) / 16, b_ @ b_.transpose(-1, -2) / 16
    save("basis", sigma_q=sq16, sigma_k=sk16, ref_regularized=ref_regularize_batch(sk16, 1e-4),
         ref_eigvec_desc=ref_eigvec_desc(sk16, 1e-4), ref_jointqk_basis=ref_jointqk_basis(sq16, sk16, 1e-4))

    # 4. compressor: fit through the reference's build_method_compressor, then roundtrip
    k256 = keys[:256].clone()
    g = torch.Generator().manual_seed(3)
    qs = torch.randn(1024, 128, generator=g) @ ref_rot(128, 99) * torch.linspace(2.0, 0.2, 128)
    sig_q = second_moment(qs)
    R_sym = ref_jointqk_basis(sig_q, sig_k, 1e-4)
    comp8 = ref_build("r_sym_waterfill", sig_q, sig_k, None, None, None, 2.0, None, 0, 128, R_sym=R_sym)
    bits4 = ref_allocate_bits(((R_sym.T @ sig_q @ R_sym).diagonal().clamp_min(1e-30)
                               * (R_sym.T @ sig_k @ R_sym).diagonal().clamp_min(1e-30)).unsqueeze(0), 2,
                              max_coord_bits=4).squeeze(0)
    comp4 = RefCompressor(bits4, comp8.stds, forward_map=R_sym, inverse_map=R_sym.T)
    comp4b = RefCompressor(ref_allocate_bits(var.unsqueeze(0), 3, max_coord_bits=4).squeeze(0),
                           torch.sqrt(var), forward_map=R, inverse_map=R.T)
    fwd, inv, cbs = ref_stack([comp4, comp4b])
    kb = torch.stack([k256, k256.flip(0)], 0).unsqueeze(0)               # (1, 2, 256, 128)
    save("compressor", keys=k256, sigma_q=sig_q, sigma_k=sig_k, R_sym=R_sym,
         ref_bits_cap8=comp8.bits_int, ref_stds=comp8.stds, ref_codebooks_cap8=comp8.codebooks_padded,
         ref_roundtrip_cap8=comp8.roundtrip(k256),
         bits_cap4=bits4, ref_codebooks_cap4=comp4.codebooks_padded, ref_roundtrip_cap4=comp4.roundtrip(k256),
         ref_codes_cap4=ref_codes(comp4, k256), ref_roundtrip_cap4_bf16=comp4.roundtrip(k256.to(torch.bfloat16)),
         ref_codes_cap4_bf16=ref_codes(comp4, k256.to(torch.bfloat16)),
         basis_b=R, bits_b=comp4b.bits_int, stds_b=comp4b.stds, ref_codebooks_b=comp4b.codebooks_padded,
         ref_codes_b=ref_codes(comp4b, k256), ref_roundtrip_b=comp4b.roundtrip(k256),
         ref_batched_roundtrip=ref_batched(kb, fwd, inv, cbs))

    # 5. attention metrics on the retrieval queries of the parity config
    q, j = retrieval_queries(keys, sig_k, 64, config_seed(0, 0, 0) + 7)
    k_ref = keys[:1024].view(1, 1, 1024, 128)
    k_hat = comp4b.roundtrip(keys[:1024]).view(1, 1, 1024, 128)
    qq = q.view(1, 1, 64, 128)
    m = ref_metrics(qq, k_ref, k_hat)
    rep = ref_repeat(torch.arange(2 * 3 * 4 * 2, dtype=torch.float32).view(2, 3, 4, 2), 6)
    save("attention", queries=qq, ref_keys=k_ref, cand_keys=k_hat,
         ref_metric_values=np.array([m["logit_mse"], m["logit_cosine"], m["top1_match"], m["top5_containment"]]),
         ref_repeat_kv=rep)

    # 6. moments
    g = torch.Generator().manual_seed(9)
    qm = torch.randn(2, 4, 96, 32, generator=g).to(torch.bfloat16)
    km = torch.randn(2, 2, 96, 32, generator=g).to(torch.bfloat16)
    vm = torch.randn(2, 2, 96, 32, generator=g).to(torch.bfloat16)
    mom = ref_moments(qm, km, vm, 80, torch.device("cpu"))
    cross = RefCross()
    cross.update(qm[:1].float(), km[:1].float(), 2)
    cross.update(qm[1:].float(), km[1:].float(), 2)
    qacc = RefQuery()
    qacc.update(qm[:, :, :40].float())
    qacc.update(qm[:, :, 40:].float())
    mean, cov, second = qacc.finalize()
    m2 = ref_query_moments(qm.float())
    save("moments", q=qm.float(), k=km.float(), v=vm.float(),
         **{f"ref_{k_}": v_ for k_, v_ in mom.items() if isinstance(v_, torch.Tensor)},
         ref_cross=cross.finalize(), ref_qacc_mean=mean, ref_qacc_cov=cov, ref_qacc_second=second,
         ref_qm_mean=m2[0], ref_qm_cov=m2[1], ref_qm_second=m2[2],
         ref_grouped_second=ref_grouped(qm.float(), 2))

    # 7. V-side compressors: eigenbasis of the centred covariance, uniform / water-fill bits, mean centring
    va = _import_v_adapter()
    g = torch.Generator().manual_seed(11)
    U = ref_rot(128, seed=config_seed(5, 0, 0))
    lam = torch.exp(-torch.arange(128, dtype=torch.float32) / 40.0)
    mu_v = 0.3 * torch.randn(128, generator=g)
    vals = (torch.randn(4096, 128, generator=g) * lam.sqrt()) @ U.T + mu_v
    sigma_v = second_moment(vals)
    mean_v = vals.double().mean(0).float()
    cov_v = sigma_v - torch.outer(mean_v, mean_v)
    v256, v256_bf16 = vals[:256], vals[:256].to(torch.bfloat16)
    out = {"values": v256, "cov_v": cov_v, "mu_v": mean_v}
    for method, bits in (("v_eigen_uniform", 3), ("v_eigen_waterfill", 3), ("v_eigen_waterfill", 2), ("v_random", 2)):
        comp = va.build_v_compressor(method, cov_v_for_head=cov_v, head_dim=128, bits=bits, seed=42, mu_v_for_head=mean_v)
        tag = f"{method}_{bits}"
        out[f"ref_bits_{tag}"] = comp.inner.bits_int
        out[f"ref_stds_{tag}"] = comp.inner.stds
        out[f"ref_forward_{tag}"] = comp.inner.forward_map
        out[f"ref_codebooks_{tag}"] = comp.inner.codebooks_padded
        out[f"ref_roundtrip_{tag}"] = comp.roundtrip(v256)
        out[f"ref_roundtrip_bf16_{tag}"] = comp.roundtrip(v256_bf16)
    plain = va.build_v_compressor("v_eigen_uniform", cov_v_for_head=cov_v, head_dim=128, bits=3, seed=42)
    out["ref_roundtrip_uncentred_v_eigen_uniform_3"] = plain.roundtrip(v256)
    save("v_compressor", **out)


if __name__ == "__main__":
    main()
