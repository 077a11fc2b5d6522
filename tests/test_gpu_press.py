"""The kvpress-shaped press driven by stub objects, the way the reference's own parity scripts drive
``JointQKPress`` (experiments/stage1/tests/test_press_roundtrip_parity.py:25-94 builds the press
from artefact files, calls ``post_init_from_model(FakeModel())`` and compares the press's
compressors with offline ``build_method_compressor`` / ``build_v_compressor`` to max-abs 1e-5).
Here the artefacts come from this library's own calibration pass, and the hook protocol is
exercised with a fake attention module and a fake cache."""

from types import SimpleNamespace

import pytest
import torch

import jointqk_b200 as jq
from jointqk_b200.moments import KeyPathMoments
from jointqk_b200.synthetic import config_seed, spectrum_keys
from oracle import reference_port as orc

pytestmark = pytest.mark.gpu
L, HQ, HKV, D, T = 2, 8, 2, 128, 4096


class FakeModel:
    pass


def _calibration(tmp_path):
    g = torch.Generator().manual_seed(21)
    acc = KeyPathMoments(L, HQ, HKV, D, device="cuda", with_values=True)
    data = {}
    for layer in range(L):
        k = torch.stack([spectrum_keys(T, config_seed(6, layer, h), n_outliers=0) for h in range(HKV)])
        q = (0.7 * k.repeat_interleave(HQ // HKV, 0) + 0.5 * torch.randn(HQ, T, D, generator=g))
        v = torch.stack([spectrum_keys(T, config_seed(7, layer, h), n_outliers=0) for h in range(HKV)]) + 0.2
        data[layer] = (q, k, v)
        acc.update(layer, q.to(torch.bfloat16).cuda(), k.to(torch.bfloat16).cuda(), v.to(torch.bfloat16).cuda())
    cca, vst = acc.calibration_artifacts(eps=1e-4, source="test")
    torch.save(cca, tmp_path / "cca_stats.pt")
    torch.save(vst, tmp_path / "v_stats.pt")
    return cca, vst, data


@pytest.mark.parametrize("cap", [4, 8])
def test_press_compressors_equal_offline_builders_and_the_oracle(tmp_path, cap):
    """``cap`` 8 is what the reference's builders hard-code (per_coord_quantization.py:367)."""
    cca, vst, data = _calibration(tmp_path)
    press = jq.JointQKPressB200(cca_stats_path=str(tmp_path / "cca_stats.pt"), v_stats_path=str(tmp_path / "v_stats.pt"),
                                v_method="v_eigen_waterfill", k_method="r_sym_waterfill", k_bits=2, v_bits=3, rank=64, max_bits=cap)
    press.post_init_from_model(FakeModel())
    press.post_init_from_model(FakeModel())                      # idempotent
    assert (0, 0) not in press._k_compressors and (1, 1) in press._k_compressors   # layer 0 stays full precision
    LAYER, HEAD = 1, 1
    k, v = data[LAYER][1][HEAD, :512], data[LAYER][2][HEAD, :512]
    off_k = jq.build_method_compressor("r_sym_waterfill", cca["sigma_q"][LAYER, HEAD], cca["sigma_k"][LAYER, HEAD],
                                       cca={"P_K": None, "P_K_inv": None, "rho": None}, b_avg=2.0, r=64, seed=42, head_dim=D,
                                       R_sym=cca["R_sym"][LAYER, HEAD], max_bits=cap)
    off_v = jq.build_v_compressor("v_eigen_waterfill", cov_v_for_head=vst["cov_v"][LAYER, HEAD],
                                  mu_v_for_head=vst["mu_v"][LAYER, HEAD], head_dim=D, bits=3,
                                  seed=42 + LAYER * 1000 + HEAD, max_bits=cap)
    pk, pv = press._k_compressors[(LAYER, HEAD)], press._v_compressors[(LAYER, HEAD)]
    assert (int(pk.bits_int.max()) > 4) == (cap == 8)
    k_diff = (off_k.roundtrip(k) - pk.roundtrip(k)).abs().max().item()
    v_diff = (off_v.roundtrip(v) - pv.roundtrip(v)).abs().max().item()
    print(f"K parity max-abs-diff: {k_diff:.2e}   V parity max-abs-diff: {v_diff:.2e}")
    assert k_diff < 1e-5 and v_diff < 1e-5
    # and both against the CPU restatement of the reference
    ref_k, codes_k = orc.roundtrip(k, pk.codebooks_padded, pk.forward_map, pk.inverse_map)
    got_k = pk.roundtrip(k)
    same = (pk.codes(k).long() == codes_k).all(-1)
    assert float(same.float().mean()) > 0.99 and (got_k[same] - ref_k[same]).abs().max().item() < 1e-5 * float(ref_k.abs().max())
    ref_v, codes_v = orc.centred_roundtrip(v, pv.mu, pv.inner.codebooks_padded, pv.inner.forward_map, pv.inner.inverse_map)
    assert ((pv.roundtrip(v) - ref_v).abs().amax(-1) < 1e-5 * float(ref_v.abs().max())).float().mean().item() > 0.99


def test_forward_hook_prefill_then_mode_b_decode_steps(tmp_path):
    cca, vst, data = _calibration(tmp_path)
    press = jq.JointQKPressB200(cca_stats_path=str(tmp_path / "cca_stats.pt"), v_stats_path=str(tmp_path / "v_stats.pt"),
                                k_bits=2, v_bits=3, layer0_full_precision=False, compress_decode=True)
    press.post_init_from_model(FakeModel())
    S0, steps, B = 300, 5, 2
    module = SimpleNamespace(layer_idx=1)
    q_all, k_all, v_all = data[1]
    keys = torch.stack([k_all[:, :S0 + steps], k_all.flip(1)[:, :S0 + steps]]).to(torch.bfloat16).cuda()     # (B, Hkv, S, d)
    vals = torch.stack([v_all[:, :S0 + steps], v_all.flip(1)[:, :S0 + steps]]).to(torch.bfloat16).cuda()
    layer = SimpleNamespace(keys=keys[:, :, :S0].clone(), values=vals[:, :, :S0].clone())
    cache = SimpleNamespace(layers={1: layer})
    hidden = torch.zeros(B, S0, 16)
    out = press.forward_hook(module, (), {"hidden_states": hidden, "past_key_values": cache,
                                          "cache_position": torch.arange(S0)}, ("attn_out", None))
    assert out == ("attn_out", None) and press.caches[1].lengths == [S0, S0]
    assert layer.keys.dtype == torch.bfloat16 and layer.keys.shape == (B, HKV, S0, D)
    # the dense cache now holds the reference's reconstruction of the prefill keys
    for h in range(HKV):
        comp = press._k_compressors[(1, h)]
        ref, _ = orc.roundtrip(keys[0, h, :S0].cpu(), comp.codebooks_padded, comp.forward_map, comp.inverse_map)
        close = (layer.keys[0, h].float().cpu() - ref.to(torch.bfloat16).float()).abs().amax(-1) <= 2e-2 * float(ref.abs().max())
        assert float(close.float().mean()) > 0.99
    history = layer.keys.clone()
    for t in range(S0, S0 + steps):                                # decode steps: the model appended one raw token
        layer.keys = torch.cat([layer.keys, keys[:, :, t:t + 1]], dim=2)
        layer.values = torch.cat([layer.values, vals[:, :, t:t + 1]], dim=2)
        press.forward_hook(module, (), {"hidden_states": hidden[:, :1], "past_key_values": cache,
                                        "cache_position": torch.tensor([t])}, ("attn_out", None))
    assert press.caches[1].lengths == [S0 + steps] * 2 and layer.keys.shape[2] == S0 + steps
    assert torch.equal(layer.keys[:, :, :S0], history)            # history untouched
    assert not torch.equal(layer.keys[:, :, S0:], keys[:, :, S0:S0 + steps])   # the new tokens were quantised
    # attention over the paged cache equals dense attention over what the hook left in the dense cache
    q = q_all[:, 77].to(torch.bfloat16).unsqueeze(0).expand(B, HQ, D).contiguous()
    got = press.decode(1, q.cuda()).cpu()
    want = orc.decode_attention(q, layer.keys.float().cpu(), layer.values.cpu())
    err = ((got - want).abs() / want.abs().amax(-1, keepdim=True)).max().item()
    print(f"paged decode vs dense attention over the hook's cache: rel err {err:.2e}")
    assert err < 1e-2          # the dense cache holds bf16-rounded reconstructions, the paged one exact codes
    # Mode A: decode steps are left alone
    press_a = jq.JointQKPressB200(cca_stats_path=str(tmp_path / "cca_stats.pt"), v_stats_path=str(tmp_path / "v_stats.pt"),
                                  k_bits=2, v_bits=3, layer0_full_precision=True)
    press_a.post_init_from_model(FakeModel())
    raw = SimpleNamespace(keys=keys.clone(), values=vals.clone())
    press_a.forward_hook(SimpleNamespace(layer_idx=1), (), {"hidden_states": hidden[:, :1], "past_key_values": SimpleNamespace(layers={1: raw}),
                                                            "cache_position": torch.tensor([S0 + steps])}, ("o", None))
    assert torch.equal(raw.keys, keys)
    k0, v0 = press_a.compress(SimpleNamespace(layer_idx=0), None, keys, vals, None, {})
    assert k0 is keys and v0 is vals                               # layer 0 passes through


def test_press_with_the_reference_constructor_defaults_beyond_the_record(tmp_path):
    """k_bits = 4 at the reference's cap of 8 (its constructor default and its hard-coded cap) puts
    more coordinates above 4 bits than a record holds: the hook still swaps in the reference's
    reconstruction, made on the GPU without a record; there is no paged cache to decode over."""
    cca, vst, data = _calibration(tmp_path)
    press = jq.JointQKPressB200(cca_stats_path=str(tmp_path / "cca_stats.pt"), v_stats_path=str(tmp_path / "v_stats.pt"),
                                k_bits=4, v_bits=2, layer0_full_precision=False, max_bits=8)
    press.post_init_from_model(FakeModel())
    assert not press._k_compressors[(1, 0)].packable
    S0, B = 200, 2
    q_all, k_all, v_all = data[1]
    keys = torch.stack([k_all[:, :S0], k_all.flip(1)[:, :S0]]).cuda()
    vals = torch.stack([v_all[:, :S0], v_all.flip(1)[:, :S0]]).cuda()
    layer = SimpleNamespace(keys=keys.clone(), values=vals.clone())
    press.forward_hook(SimpleNamespace(layer_idx=1), (), {"hidden_states": torch.zeros(B, S0, 16),
                                                          "past_key_values": SimpleNamespace(layers={1: layer}),
                                                          "cache_position": torch.arange(S0)}, ("o", None))
    for h in range(HKV):
        kc, vc = press._k_compressors[(1, h)], press._v_compressors[(1, h)]
        ref_k, _ = orc.roundtrip(keys[1, h].cpu(), kc.codebooks_padded, kc.forward_map, kc.inverse_map)
        ref_v, _ = orc.centred_roundtrip(vals[1, h].cpu(), vc.mu, vc.inner.codebooks_padded, vc.inner.forward_map, vc.inner.inverse_map)
        for got, ref in ((layer.keys[1, h].cpu(), ref_k), (layer.values[1, h].cpu(), ref_v)):
            close = ((got - ref).abs().amax(-1) < 1e-4 * float(ref.abs().max())).float().mean().item()
            assert close > 0.99
    assert 1 not in press.caches
    with pytest.raises(RuntimeError, match="no paged cache"):
        press.decode(1, torch.zeros(B, HQ, D, dtype=torch.bfloat16))
