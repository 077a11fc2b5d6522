"""Host-side fit objects of the product against reference outputs (tests/golden/)."""

import numpy as np
import pytest
import torch

import jointqk_b200 as jq
from jointqk_b200.allocation import cap_and_redistribute


def _t(a):
    return torch.from_numpy(np.asarray(a))


def test_lloyd_max_tables_bit_equal(golden):
    g = golden("centroids")
    for b in range(1, 9):
        assert torch.equal(jq.unit_gaussian_centroids(b), _t(g[f"ref_unit_{b}"])), b
    for b in range(1, 5):
        assert torch.equal(jq.solve_lloyd_max(128, b)[0], _t(g[f"ref_lloyd128_{b}"])), b
    assert torch.equal(jq.unit_gaussian_centroids(0), torch.zeros(1))
    assert torch.equal(jq.generate_rotation_matrix(16, 7), _t(g["ref_rotation_16_seed7"]))


def test_lloyd_max_known_answers():
    # classical Gaussian Lloyd-Max constants
    c1, c2, c3 = (jq.unit_gaussian_centroids(b) for b in (1, 2, 3))
    assert c1.tolist() == pytest.approx([-0.79788458, 0.79788458], abs=1e-7)
    assert c2.tolist() == pytest.approx([-1.51041758, -0.45278004, 0.45278004, 1.51041758], abs=1e-7)
    assert c3[4:].tolist() == pytest.approx([0.24509418, 0.75600529, 1.34390926, 2.15194559], abs=1e-7)
    assert float(jq.unit_gaussian_centroids(4)[-1]) == pytest.approx(2.73307800, abs=1e-6)


def test_water_fill_and_allocations(golden):
    g = golden("allocation")
    for tag, v in (("var", _t(g["variances"])), ("wvar", _t(g["variances"]) * _t(g["weights"]))):
        for b in (2, 3, 4):
            assert torch.equal(jq.water_fill(v.unsqueeze(0), float(b * 128)).squeeze(0), _t(g[f"ref_waterfill_{tag}_{b}"]))
            for cap in (4, 8):
                got = jq.allocate_bits(v.unsqueeze(0), b, max_coord_bits=cap).squeeze(0)
                assert torch.equal(got, _t(g[f"ref_alloc_{tag}_{b}_cap{cap}"])), (tag, b, cap)
                assert int(got.sum()) == b * 128
        cont = jq.water_fill(v.unsqueeze(0), 2.5 * 128)
        assert torch.equal(cont.squeeze(0), _t(g[f"ref_waterfill_{tag}_2p5"]))
        rounded = jq.round_bits_to_integer(cont, total_bits=int(2.5 * 128)).squeeze(0)
        assert torch.equal(rounded, _t(g[f"ref_round_{tag}_2p5"]))
        capped = jq.allocate_bits_for_budget(v.unsqueeze(0), 2.5 * 128, 4).squeeze(0)
        assert torch.equal(capped, cap_and_redistribute(rounded, 4))
        assert int(capped.sum()) == 320 and int(capped.max()) <= 4
        assert torch.equal(jq.water_fill(v.unsqueeze(0), 256.0, max_bits=4.0).squeeze(0), _t(g[f"ref_waterfill_{tag}_2_max4"]))
    small = _t(g["small_variances"])
    assert torch.equal(jq.water_fill(small, 8.0), _t(g["ref_small_waterfill_8"]))
    assert torch.equal(jq.allocate_bits(small, 2, 8), _t(g["ref_small_alloc_2"]))


def test_water_fill_properties():
    g = torch.Generator().manual_seed(1)
    v = torch.rand(3, 64, generator=g) * 10 + 1e-3
    b = jq.water_fill(v, 128.0)
    assert torch.allclose(b.sum(-1), torch.full((3,), 128.0), atol=1e-3)
    assert (b >= 0).all()
    order = torch.argsort(v[0])
    assert (torch.diff(b[0][order]) >= -1e-5).all()       # more variance, never fewer bits
    capped = jq.water_fill(v, 128.0, max_bits=3.0)
    assert float(capped.max()) <= 3.0 + 1e-6 and torch.allclose(capped.sum(-1), torch.full((3,), 128.0), atol=1e-3)
    assert jq.water_fill(v[0], 128.0).shape == (64,)


def test_bases_match_reference_up_to_sign(golden):
    g = golden("basis")
    sq, sk = _t(g["sigma_q"]), _t(g["sigma_k"])
    assert torch.equal(jq.regularize_batch(sk, 1e-4), _t(g["ref_regularized"]))
    for mine, ref in ((jq.eigvec_desc(sk, 1e-4), _t(g["ref_eigvec_desc"])),
                      (jq.jointqk_basis(sq, sk, 1e-4), _t(g["ref_jointqk_basis"]))):
        dots = (mine * ref).sum(-2).abs()
        assert float(dots.min()) > 0.99999


def test_compressor_object_matches_reference(golden):
    g = golden("compressor")
    R = _t(g["R_sym"])
    comp = jq.build_method_compressor("r_sym_waterfill", _t(g["sigma_q"]), _t(g["sigma_k"]), None, None, None,
                                      2.0, None, 0, 128, R_sym=R)
    assert torch.equal(comp.bits_int, _t(g["ref_bits_cap8"]))
    assert torch.equal(comp.stds, _t(g["ref_stds"]))
    assert torch.equal(comp.codebooks_padded, _t(g["ref_codebooks_cap8"]))
    comp4 = jq.build_method_compressor("r_sym_waterfill", _t(g["sigma_q"]), _t(g["sigma_k"]), None, None, None,
                                       2.0, None, 0, 128, R_sym=R, max_bits=4)
    assert torch.equal(comp4.bits_int, _t(g["bits_cap4"]))
    assert torch.equal(comp4.codebooks_padded, _t(g["ref_codebooks_cap4"]))
    assert comp4.codebook_lengths.tolist() == (2 ** comp4.bits_int).tolist()
    fwd, inv, cb = jq.stack_per_head([comp4, comp4])
    assert fwd.shape == (2, 128, 128) and cb.shape == (2, 128, 16) and torch.equal(inv[0], R.T)
    assert jq.build_method_compressor("v3", None, None) is None
    with pytest.raises(ValueError):
        jq.build_method_compressor("cca_waterfill", _t(g["sigma_q"]), _t(g["sigma_k"]), R_sym=R)


def test_compressor_constructor_errors():
    with pytest.raises(ValueError, match="1D"):
        jq.PerCoordCompressor(torch.zeros(2, 2), torch.zeros(2, 2))
    with pytest.raises(ValueError, match="shape mismatch"):
        jq.PerCoordCompressor(torch.zeros(4), torch.zeros(5))
    with pytest.raises(ValueError, match="forward_map"):
        jq.PerCoordCompressor(torch.zeros(4), torch.ones(4), forward_map=torch.eye(3))
    c = jq.PerCoordCompressor(torch.tensor([0, 1, 2, 0]), torch.ones(4), forward_map=torch.eye(4))
    assert torch.equal(c.inverse_map, torch.eye(4))
    assert c.codebooks_padded.shape == (4, 4) and float(c.codebooks_padded[0, 0]) == 0.0
    with pytest.raises(ValueError, match="last-dim"):
        c.roundtrip(torch.zeros(3, 5))


def test_fit_sigma_k_histogram():
    from jointqk_b200.synthetic import config_seed, fit_sigma_k_heads, spectrum_keys

    keys = spectrum_keys(4096, config_seed(0, 0, 0))
    comps, sig = fit_sigma_k_heads(keys[None], 2.0)
    c = comps[0]
    assert int(c.bits_int.sum()) == 256 and int(c.bits_int.max()) <= 4
    assert torch.allclose(c.forward_map @ c.inverse_map, torch.eye(128), atol=1e-4)
    var = (c.forward_map.T @ sig[0] @ c.forward_map).diagonal()
    assert torch.allclose(c.stds, var.clamp_min(1e-30).sqrt(), rtol=1e-5)
