"""Value-side compressors against fixtures made by the reference's own ``build_v_compressor`` /
``CenteredCompressor`` (tests/golden/make_golden.py, section 7).  The host-side fit and the oracle's
centring run on the CPU; the CUDA roundtrip is compared with the reference outputs under ``-m gpu``."""

import numpy as np
import pytest
import torch

import jointqk_b200 as jq
from oracle import reference_port as orc

CASES = (("v_eigen_uniform", 3), ("v_eigen_waterfill", 3), ("v_eigen_waterfill", 2), ("v_random", 2))


def _t(a):
    return torch.from_numpy(np.asarray(a))


def _build(g, method, bits, centred=True):
    return jq.build_v_compressor(method, cov_v_for_head=_t(g["cov_v"]), head_dim=128, bits=bits, seed=42,
                                 mu_v_for_head=_t(g["mu_v"]) if centred else None)


def _from_fixture(g, method, bits, centred=True):
    """The compressor the reference built, from its stored bits / stds / basis: an eigendecomposition
    redone on another host may differ in the last bits, which moves codes that sit on a decision
    boundary, so the GPU comparison must not depend on refitting."""
    tag = f"{method}_{bits}"
    fwd = _t(g[f"ref_forward_{tag}"])
    inner = jq.PerCoordCompressor(_t(g[f"ref_bits_{tag}"]), _t(g[f"ref_stds_{tag}"]), forward_map=fwd,
                                  inverse_map=fwd.transpose(-1, -2))
    assert torch.equal(inner.codebooks_padded, _t(g[f"ref_codebooks_{tag}"]))
    return jq.CenteredCompressor(inner, _t(g["mu_v"])) if centred else inner


@pytest.mark.parametrize("method,bits", CASES)
def test_fit_equals_reference_and_oracle_centring_is_pinned(golden, method, bits):
    g = golden("v_compressor")
    tag = f"{method}_{bits}"
    comp = _build(g, method, bits)
    assert torch.equal(comp.inner.bits_int, _t(g[f"ref_bits_{tag}"]))
    torch.testing.assert_close(comp.inner.stds, _t(g[f"ref_stds_{tag}"]), rtol=1e-4, atol=1e-7)
    fwd = _t(g[f"ref_forward_{tag}"])
    assert float((comp.inner.forward_map * fwd).sum(0).abs().min()) > 0.999       # same basis up to column sign
    assert int(comp.inner.bits_int.sum()) == bits * 128
    comp = _from_fixture(g, method, bits)
    for dtype, name in ((torch.float32, "ref_roundtrip_"), (torch.bfloat16, "ref_roundtrip_bf16_")):
        out, _ = orc.centred_roundtrip(_t(g["values"]).to(dtype), comp.mu, comp.inner.codebooks_padded,
                                       comp.inner.forward_map, comp.inner.inverse_map)
        assert torch.equal(out, _t(g[name + tag]))


def test_builder_errors_follow_the_reference():
    with pytest.raises(ValueError, match="requires cov_v_for_head"):
        jq.build_v_compressor("v_eigen_uniform", head_dim=128, bits=2)
    with pytest.raises(ValueError, match="Unknown V method"):
        jq.build_v_compressor("v_nope", cov_v_for_head=torch.eye(16), head_dim=16, bits=2)
    with pytest.raises(ValueError, match="third-party"):
        jq.build_v_compressor("v_turboquant", head_dim=128, bits=2)
    legacy = jq.build_v_compressor("v_eigen_uniform", sigma_v_for_head=torch.eye(16), head_dim=16, bits=2)
    assert legacy.d == 16 and jq.V_METHOD_NAMES[2] == "v_eigen_waterfill"


@pytest.mark.gpu
@pytest.mark.parametrize("method,bits", CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_cuda_roundtrip_matches_the_reference(golden, method, bits, dtype):
    g = golden("v_compressor")
    tag = f"{method}_{bits}"
    comp = _from_fixture(g, method, bits)
    vals = _t(g["values"]).to(dtype)
    ref = _t(g[("ref_roundtrip_" if dtype == torch.float32 else "ref_roundtrip_bf16_") + tag])
    _, ref_codes = orc.centred_roundtrip(vals, comp.mu, comp.inner.codebooks_padded, comp.inner.forward_map,
                                         comp.inner.inverse_map)
    packed = comp.compress(vals.cuda())
    from jointqk_b200 import paged

    codes = paged.unpack_codes(packed)[0, 0].cpu()
    bad = int((codes.long() != ref_codes).sum())
    out = comp.roundtrip(vals.cuda()).cpu()
    rows_ok = (codes.long() == ref_codes).all(-1)
    scale = float(ref.abs().max())
    err = float((out[rows_ok] - ref[rows_ok]).abs().max())
    print(f"{tag} {dtype}: {bad} code mismatches of {codes.numel()}, max abs err on agreeing rows {err:.2e}")
    assert bad <= 1 and err < 1e-5 * scale
    assert out.shape == vals.shape and out.dtype == torch.float32


@pytest.mark.gpu
def test_uncentred_value_compressor_and_mean_handling(golden):
    g = golden("v_compressor")
    plain = _from_fixture(g, "v_eigen_uniform", 3, centred=False)
    out = plain.roundtrip(_t(g["values"]).cuda()).cpu()
    ref = _t(g["ref_roundtrip_uncentred_v_eigen_uniform_3"])
    close = (out - ref).abs().amax(-1) < 1e-5 * float(ref.abs().max())
    assert float(close.float().mean()) > 0.99           # a row with a boundary flip differs by one level
    centred = _build(g, "v_eigen_uniform", 3)
    assert centred.to("cpu") is centred and centred.mu.device.type == "cpu"
    with pytest.raises(ValueError, match="last-dim"):
        centred.roundtrip(torch.zeros(4, 64, device="cuda"))
