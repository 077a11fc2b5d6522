"""GPU parity of the calibration moment kernels and accumulators against the oracle and the
reference fixtures.  Both sides are fp32 sums in different orders, so each is compared with an
fp64 sum.  The GPU's relative Frobenius error must be <= 1e-4 everywhere.  The CUDA-core kernel
(short inputs, other dtypes) must also stay within 2x the oracle's own error (+2e-6).  The
tensor-core kernel cannot: tcgen05 accumulates in fp32 with truncation, which biases long
running sums (measured 1e-5 .. 2.5e-5 for 2048-token blocks against 4e-7 .. 8e-7 for the blocked
CPU sum); its bound is 6e-5, and the measured values are printed."""

import numpy as np
import pytest
import torch

import jointqk_b200 as jq
from jointqk_b200.moments import KeyPathMoments, accumulate_layer
from jointqk_b200.synthetic import correlated_qk
from oracle import reference_port as orc

pytestmark = pytest.mark.gpu


def _t(a):
    return torch.from_numpy(np.asarray(a))


def _fro(a, b):
    return float((a.double() - b.double()).norm() / b.double().norm())


def test_reference_fixture_sums(golden):
    g = golden("moments")
    q, k, v = (_t(g[n]).to(torch.bfloat16) for n in ("q", "k", "v"))
    out = jq.compute_moments_from_tensors(q, k, v, 80, torch.device("cuda"))
    for name in ("sq_sum", "sk_sum", "cqk_sum", "sv_sum", "sum_q", "sum_k", "sum_v"):
        assert out[name].device.type == "cpu"
        torch.testing.assert_close(out[name], _t(g[f"ref_{name}"]), rtol=2e-5, atol=2e-4)
    assert out["tokens"] == 80 and out["group"] == 2 and out["head_dim"] == 32


def test_reference_fixture_accumulators(golden):
    g = golden("moments")
    q, k = _t(g["q"]).cuda(), _t(g["k"]).cuda()
    cross = jq.CrossMomentsAccumulator()
    cross.update(q[:1], k[:1], 2)
    cross.update(q[1:], k[1:], 2)
    torch.testing.assert_close(cross.finalize().cpu(), _t(g["ref_cross"]), rtol=2e-5, atol=2e-5)
    acc = jq.QueryMomentsAccumulator()
    acc.update(q[:, :, :40])
    acc.update(q[:, :, 40:])
    mean, cov, second = (x.cpu() for x in acc.finalize())
    torch.testing.assert_close(mean, _t(g["ref_qacc_mean"]), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(second, _t(g["ref_qacc_second"]), rtol=2e-5, atol=2e-5)
    torch.testing.assert_close(cov, _t(g["ref_qacc_cov"]), rtol=2e-5, atol=2e-5)
    m2 = jq.compute_query_moments(q)
    torch.testing.assert_close(m2[2].cpu(), _t(g["ref_qm_second"]), rtol=2e-5, atol=2e-5)
    grouped = jq.compute_grouped_query_second_moment(q, 2)
    torch.testing.assert_close(grouped.cpu(), _t(g["ref_grouped_second"]), rtol=2e-5, atol=2e-5)
    with pytest.raises(RuntimeError):
        jq.CrossMomentsAccumulator().finalize()
    with pytest.raises(ValueError, match="Cannot group"):
        jq.CrossMomentsAccumulator().update(q[:1, :3], k[:1], 2)


@pytest.mark.parametrize("tokens", [1, 100, 4096 + 33, 262144])
def test_calibration_shape_against_fp64(tokens):
    q, k = correlated_qk(tokens, 32, 8, seed=31, device="cuda")
    acc = KeyPathMoments(1, 32, 8, 128, device="cuda")
    acc.update(0, q, k)
    gpu = {"sq_sum": acc.sums[0, 0].cpu(), "sk_sum": acc.sums[0, 1].cpu(), "cqk_sum": acc.sums[0, 2].cpu()}
    ora = orc.moment_sums(q[None].cpu(), k[None].cpu())
    qd, kd = q.double(), k.double()
    exact = {
        "sq_sum": torch.einsum("hsd,hse->hde", qd, qd).view(8, 4, 128, 128).sum(1).cpu(),
        "sk_sum": torch.einsum("hsd,hse->hde", kd, kd).cpu(),
        "cqk_sum": torch.einsum("hsd,hse->hde", qd.view(8, 4, tokens, 128).mean(1), kd).cpu(),
    }
    for name in gpu:
        e_gpu, e_ora = _fro(gpu[name], exact[name]), _fro(ora[name][0], exact[name])
        print(f"{name} tokens={tokens}: gpu {e_gpu:.2e} oracle {e_ora:.2e}")
        assert e_gpu <= 1e-4
        if tokens < 64:                 # CUDA-core kernel
            assert e_gpu <= 2 * e_ora + 2e-6
        else:                           # tensor-core kernel
            assert e_gpu <= 6e-5


def test_linearity_and_finalize():
    q, k = correlated_qk(3000, 8, 2, seed=5, device="cuda")
    whole = KeyPathMoments(2, 8, 2, 128, device="cuda")
    whole.update(1, q, k)
    parts = KeyPathMoments(2, 8, 2, 128, device="cuda")
    parts.update(1, q[:, :1234].contiguous(), k[:, :1234].contiguous())
    parts.update(1, q[:, 1234:], k[:, 1234:])                       # strided heads, contiguous rows
    scale = float(whole.sums[1].abs().max())
    assert float((parts.sums[1] - whole.sums[1]).abs().max()) <= 1e-4 * scale
    with pytest.raises(RuntimeError):
        whole.finalize()                                            # layer 0 never saw a token
    whole.update(0, q, k)
    fin = whole.finalize()
    n = orc.normalise_moments(orc.moment_sums(q[None].cpu(), k[None].cpu()), group=4, tokens=3000)
    for name in ("sigma_q", "sigma_k", "cqk"):
        ref = n[name][0]
        assert float((fin[name][0].cpu() - ref).norm() / ref.norm()) <= 1e-4
    # fit from GPU moments agrees with a fit from oracle moments up to column sign
    Rg = jq.jointqk_basis(fin["sigma_q"][0, 0].cpu(), fin["sigma_k"][0, 0].cpu(), 1e-4)
    Ro = jq.jointqk_basis(n["sigma_q"][0, 0], n["sigma_k"][0, 0], 1e-4)
    assert float((Rg * Ro).sum(0).abs().min()) > 0.99


def test_partial_outputs_and_errors():
    q, k = correlated_qk(64, 4, 2, seed=6, device="cuda")
    sk = torch.zeros(2, 128, 128, device="cuda")
    accumulate_layer(None, k, None, sk, None)
    torch.testing.assert_close(sk.cpu(), orc.moment_sums(q[None].cpu(), k[None].cpu())["sk_sum"][0], rtol=1e-5, atol=1e-4)
    with pytest.raises(ValueError, match="GQA mismatch"):
        accumulate_layer(q[:3], k, torch.zeros(2, 128, 128, device="cuda"), None, None)
