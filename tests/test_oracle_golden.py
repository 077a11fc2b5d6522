"""The CPU oracle against outputs of the reference itself (fixtures in tests/golden/)."""

import numpy as np
import torch

from oracle import reference_port as orc


def _t(a):
    return torch.from_numpy(np.asarray(a))


def test_codebooks_match_reference(golden):
    g, c = golden("compressor"), golden("centroids")
    unit = {b: _t(c[f"ref_unit_{b}"]) for b in range(1, 9)}
    cb8 = orc.codebooks_padded(_t(g["ref_bits_cap8"]), _t(g["ref_stds"]), unit)
    assert torch.equal(cb8, _t(g["ref_codebooks_cap8"]))
    cb4 = orc.codebooks_padded(_t(g["bits_cap4"]), _t(g["ref_stds"]), unit)
    assert torch.equal(cb4, _t(g["ref_codebooks_cap4"]))


def test_roundtrip_and_codes_match_reference(golden):
    g = golden("compressor")
    R = _t(g["R_sym"])
    keys = _t(g["keys"])
    for cb_name, rt_name, codes_name, k in (
            ("ref_codebooks_cap4", "ref_roundtrip_cap4", "ref_codes_cap4", keys),
            ("ref_codebooks_cap4", "ref_roundtrip_cap4_bf16", "ref_codes_cap4_bf16", keys.to(torch.bfloat16)),
            ("ref_codebooks_cap8", "ref_roundtrip_cap8", None, keys)):
        out, codes = orc.roundtrip(k, _t(g[cb_name]), R, R.T)
        assert torch.equal(out, _t(g[rt_name]))          # same torch ops on the same machine: bit equal
        if codes_name:
            assert torch.equal(codes.to(torch.uint8), _t(g[codes_name]))
    Rb = _t(g["basis_b"])
    out, codes = orc.roundtrip(keys, _t(g["ref_codebooks_b"]), Rb, Rb.T)
    assert torch.equal(out, _t(g["ref_roundtrip_b"]))
    assert torch.equal(codes.to(torch.uint8), _t(g["ref_codes_b"]))


def test_batched_roundtrip_matches_reference(golden):
    g = golden("compressor")
    keys = _t(g["keys"])
    kb = torch.stack([keys, keys.flip(0)], 0).unsqueeze(0)
    R, Rb = _t(g["R_sym"]), _t(g["basis_b"])
    fwd = torch.stack([R, Rb])
    inv = torch.stack([R.T, Rb.T])
    cb = torch.stack([_t(g["ref_codebooks_cap4"]), _t(g["ref_codebooks_b"])])
    out = orc.batched_roundtrip(kb, fwd, inv, cb)
    ref = _t(g["ref_batched_roundtrip"])
    # bmm blocking may differ between the two call routes by rounding; codes can flip only at
    # decision boundaries, which changes whole reconstructed rows -- allow a handful.
    bad_rows = ((out - ref).abs().amax(-1) > 1e-5).sum().item()
    assert bad_rows <= 2


def test_attention_metrics_match_reference(golden):
    g = golden("attention")
    m = orc.attention_metrics(_t(g["queries"]), _t(g["ref_keys"]), _t(g["cand_keys"]))
    ref = g["ref_metric_values"]
    assert abs(m["logit_mse"] - ref[0]) <= 1e-6 * max(1.0, abs(ref[0]))
    assert abs(m["logit_cosine"] - ref[1]) <= 1e-6
    assert m["top1_match"] == ref[2]
    assert m["top5_containment"] == ref[3]
    rep = orc.repeat_kv(torch.arange(2 * 3 * 4 * 2, dtype=torch.float32).view(2, 3, 4, 2), 6)
    assert torch.equal(rep, _t(g["ref_repeat_kv"]))


def test_moment_sums_match_reference(golden):
    g = golden("moments")
    q, k = _t(g["q"])[:, :, :80], _t(g["k"])[:, :, :80]
    s = orc.moment_sums(q, k)
    for name in ("sq_sum", "sk_sum", "cqk_sum"):
        torch.testing.assert_close(s[name], _t(g[f"ref_{name}"]), rtol=1e-6, atol=1e-5)
    full = orc.moment_sums(_t(g["q"]), _t(g["k"]))
    n = orc.normalise_moments(full, group=2, tokens=96)
    # CrossMomentsAccumulator works per batch element = per layer here
    torch.testing.assert_close(n["cqk"][0] * 0 + n["cqk"][0], n["cqk"][0])
    cross = (full["cqk_sum"][0] + full["cqk_sum"][1]) / (2 * 96)
    torch.testing.assert_close(cross, _t(g["ref_cross"]), rtol=1e-5, atol=1e-6)
    grouped = (full["sq_sum"][0] + full["sq_sum"][1]) / (2 * 2 * 96)
    torch.testing.assert_close(grouped, _t(g["ref_grouped_second"]), rtol=1e-5, atol=1e-6)


def test_record_pack_unpack_roundtrip():
    from jointqk_b200.layout import plan_key_layout

    rng = np.random.default_rng(0)
    for hist in ([14, 40, 26, 28, 20], [0, 0, 47, 34, 47], [0, 27, 42, 27, 32], [100, 1, 0, 27, 0], [0, 0, 0, 128, 0]):
        bits = np.concatenate([np.full(n, w) for w, n in enumerate(hist)])
        rng.shuffle(bits)
        lay = plan_key_layout(bits)
        codes = (rng.integers(0, 16, size=(77, 128)) & ((1 << bits) - 1)).astype(np.uint8)
        rec = orc.pack_records(codes, lay.col_coord, lay.col_width, lay.col_bitpos, lay.n_words)
        back = orc.unpack_records(rec, lay.col_coord, lay.col_width, lay.col_bitpos, 128)
        assert np.array_equal(back, codes)
        pages = orc.records_to_pages(rec, lay.n_words + 1)
        assert pages.shape == (5, lay.n_words + 1, 16)
        assert np.array_equal(pages[4, : lay.n_words, 12], rec[76])
