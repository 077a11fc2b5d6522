"""Record layout, decision thresholds and device tables, checked on the CPU through a NumPy
model of the kernels' index arithmetic (tests/kernel_model.py) against the oracle."""

import numpy as np
import pytest
import torch

from jointqk_b200.layout import decision_thresholds, plan_key_layout
from jointqk_b200.tables import HeadTables, split_bf16_limbs
from oracle import reference_port as orc

import kernel_model as km

HISTS = [[14, 40, 26, 28, 20], [0, 0, 47, 34, 47], [0, 27, 42, 27, 32], [23, 27, 28, 27, 23],
         [0, 15, 28, 27, 58], [0, 0, 0, 128, 0], [0, 0, 0, 0, 128], [128, 0, 0, 0, 0], [100, 1, 0, 27, 0],
         [0, 128, 0, 0, 0], [3, 2, 1, 121, 1]]


def _bits(hist, seed=0):
    b = np.concatenate([np.full(n, w) for w, n in enumerate(hist)])
    np.random.default_rng(seed).shuffle(b)
    return b


@pytest.mark.parametrize("hist", HISTS)
def test_layout_invariants(hist):
    bits = _bits(hist)
    lay = plan_key_layout(bits)
    n = lay.n_active
    assert n == int((bits > 0).sum()) and lay.n_cols % 16 == 0 and lay.n_cols >= max(n, 16)
    assert sorted(lay.col_coord[:n].tolist()) == np.nonzero(bits > 0)[0].tolist()
    assert np.array_equal(lay.col_width[:n], bits[lay.col_coord[:n]])
    # fields never overlap and never straddle a 32-bit word
    used = np.zeros(32 * lay.n_words, bool)
    for c in range(n):
        p, w = int(lay.col_bitpos[c]), int(lay.col_width[c])
        assert p // 32 == (p + w - 1) // 32
        assert not used[p:p + w].any()
        used[p:p + w] = True
    assert used.sum() == lay.payload_bits
    assert lay.n_words <= 16 and lay.n_tables <= 208
    # every column is referenced by exactly one table field
    refs = [int(f) & 255 for f in lay.table_fields.reshape(-1) if f >= 0]
    assert sorted(refs) == list(range(n))


def test_layout_packs_named_configs_without_waste():
    for hist, nbytes in (([14, 40, 26, 28, 20], 32), ([0, 27, 42, 27, 32], 40), ([0, 0, 47, 34, 47], 48)):
        lay = plan_key_layout(_bits(hist))
        assert lay.record_bytes == nbytes and lay.waste_bits == 0


def test_layout_rejects_unsupported():
    with pytest.raises(ValueError):
        plan_key_layout(np.full(128, 5))
    with pytest.raises(ValueError):
        plan_key_layout(np.full(100, 2))


def test_decision_thresholds_reproduce_argmin():
    from jointqk_b200.codebooks import unit_gaussian_centroids

    rng = np.random.default_rng(1)
    widths = np.array([1, 2, 3, 4, 4, 2])
    stds = np.array([1.0, 0.37, 15.2, 1e-3, 3.3, 0.011], np.float32)
    cb = np.zeros((6, 16), np.float32)
    for i, w in enumerate(widths):
        cb[i, : 2 ** w] = unit_gaussian_centroids(int(w)).numpy() * np.float32(stds[i])
    thr = decision_thresholds(cb, widths)
    for i, w in enumerate(widths):
        lv = cb[i, : 2 ** w]
        xs = [rng.normal(size=50000).astype(np.float32) * stds[i] * 1.5]
        for t in thr[i, : 2 ** w - 1]:
            xs.append(np.array([np.nextafter(t, -np.inf), t, np.nextafter(t, np.inf)], np.float32))
        # |x| stays below 2^20 level gaps: beyond ~2^24 gaps the fp32 distances to several levels
        # round to the same value and torch's first-index tie rule takes over (documented limit)
        xs.append(np.array([0.0, -0.0, -1e30, 1e4 * stds[i], -1e4 * stds[i], lv[0], lv[-1]], np.float32))
        x = np.concatenate(xs)
        ref = np.abs(x[:, None] - lv[None, :]).argmin(-1)
        mine = (x[:, None] >= thr[i][None, :]).sum(-1)
        assert np.array_equal(ref, mine)


def test_bf16_limbs_reconstruct_fp32():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(64, 64, generator=g)
    limbs = split_bf16_limbs(x, 3)
    err = (limbs.float().sum(0) - x).abs().max().item()
    assert err <= 2.0 ** -22 * x.abs().max().item()


def _tables_from_golden(g):
    R, Rb = torch.from_numpy(g["R_sym"]), torch.from_numpy(g["basis_b"])
    fwd, inv = torch.stack([R, Rb]), torch.stack([R.T, Rb.T])
    cb = torch.stack([torch.from_numpy(g["ref_codebooks_cap4"]), torch.from_numpy(g["ref_codebooks_b"])])
    return HeadTables(fwd, inv, cb, device="cpu")


def test_kernel_model_codes_match_reference(golden):
    g = golden("compressor")
    tab = _tables_from_golden(g)
    keys = g["keys"]
    for h, name in ((0, "ref_codes_cap4"), (1, "ref_codes_b")):
        rec = km.compress_model(tab, h, keys)
        codes = km.unpack_model(tab, h, rec)
        mism = int((codes != g[name]).sum())
        assert mism <= 1, mism              # summation order may flip a code on a decision boundary
        lay = tab.layouts[h]
        ref_rec = orc.pack_records(g[name], lay.col_coord, lay.col_width, lay.col_bitpos, lay.n_words)
        assert (rec != ref_rec).sum() <= 1


def test_kernel_model_scores_match_reference(golden):
    g = golden("compressor")
    tab = _tables_from_golden(g)
    rng = np.random.default_rng(3)
    for h, codes_name, rt_name in ((0, "ref_codes_cap4", "ref_roundtrip_cap4"), (1, "ref_codes_b", "ref_roundtrip_b")):
        lay = tab.layouts[h]
        rec = orc.pack_records(g[codes_name], lay.col_coord, lay.col_width, lay.col_bitpos, lay.n_words)
        q = rng.normal(size=(4, 128)).astype(np.float32)
        s = km.score_model(tab, h, rec, q)
        ref = (q @ g[rt_name].T) / np.sqrt(128.0)
        rms = np.sqrt((ref ** 2).mean(-1, keepdims=True))
        rel = np.abs(s - ref) / np.maximum(np.abs(ref), rms)
        assert rel.max() < 2e-3, rel.max()
        assert rel.max() < 1e-3           # the fixed-point tables stay well inside the bar
        assert np.array_equal(s.argmax(-1), ref.argmax(-1))


def test_head_tables_reject_codebooks_beyond_8_bits():
    cb = torch.arange(512.0).expand(1, 16, 512).clone()
    with pytest.raises(ValueError, match="8 bits"):
        HeadTables(None, None, cb, device="cpu")


def test_layout_with_wide_columns():
    """Coordinates of 5..8 bits take a byte each in whole words between the nibble region and the byte
    region; packing and unpacking such records round-trips, and more than 32 wide coordinates are refused."""
    from oracle import reference_port as orc

    rng = np.random.default_rng(3)
    for _ in range(20):
        bits = rng.integers(0, 5, 128)
        wide = rng.choice(128, size=rng.integers(1, 33), replace=False)
        bits[wide] = rng.integers(5, 9, len(wide))
        if bits.sum() > 400:
            continue
        lay = plan_key_layout(bits)
        n = lay.n_active
        assert lay.n_wide == len(wide) and n == int((bits > 0).sum())
        wc = slice(lay.wide_first, lay.wide_first + lay.n_wide)
        assert np.all(lay.col_width[wc] > 4) and np.all(lay.col_bitpos[wc] % 8 == 0)
        assert np.all(np.delete(lay.col_width[:n], np.arange(lay.wide_first, lay.wide_first + lay.n_wide)) <= 4)
        assert np.all(np.diff(lay.col_bitpos[:n]) >= lay.col_width[:n - 1])            # fields do not overlap
        assert np.all(lay.col_bitpos[:n] // 32 == (lay.col_bitpos[:n] + lay.col_width[:n] - 1) // 32)   # nor straddle words
        codes = np.stack([rng.integers(0, 1 << max(int(b), 0) if b else 1, 50) for b in bits], 1)      # (50, 128) coordinate order
        rec = orc.pack_records(codes, lay.col_coord[:n], lay.col_width[:n], lay.col_bitpos[:n], lay.n_words)
        back = orc.unpack_records(rec, lay.col_coord[:n], lay.col_width[:n], lay.col_bitpos[:n], 128)
        assert np.array_equal(back, codes)
    too_many = np.zeros(128, dtype=np.int64)
    too_many[:33] = 5
    with pytest.raises(ValueError, match="at most 32"):
        plan_key_layout(too_many)


def test_unit_quantiser_tables_are_exact():
    """The shared coarse-to-exact quantiser of the tensor-core kernel (one FMA -> cell of a common grid
    -> index of the one threshold left to compare) must reproduce the full threshold count of every
    width for every input, whether the device fuses the multiply-add or not."""
    from jointqk_b200.codebooks import unit_gaussian_centroids
    from jointqk_b200.layout import BUCKETS, unit_quantiser_tables

    rng = np.random.default_rng(0)
    unit = {b: unit_gaussian_centroids(b).numpy() for b in range(1, 5)}
    thr, pre, aff = unit_quantiser_tables(unit)
    flat = thr.reshape(-1)
    for b in range(1, 5):
        n = 2 ** b - 1
        assert np.all(np.isfinite(thr[b - 1, :n])) and np.all(np.isinf(thr[b - 1, n:]))
        assert pre[b - 1].min() >= 16 * (b - 1) and pre[b - 1].max() <= 16 * (b - 1) + max(n - 1, 0)
        xs = [rng.normal(size=200000).astype(np.float32) * 1.7]
        for t in thr[b - 1, :n]:
            xs.append(np.array([np.nextafter(t, -np.inf), t, np.nextafter(t, np.inf)], np.float32))
        xs.append(np.array([0, -0.0, 1e30, -1e30, np.nan], np.float32))
        x = np.concatenate(xs)
        ref = (x[:, None] >= thr[b - 1, :n][None, :]).sum(-1)
        for fused in (True, False):
            with np.errstate(invalid="ignore", over="ignore"):
                if fused:
                    y = np.float32(x.astype(np.float64) * float(aff[0]) + float(aff[1]))
                else:
                    y = np.float32(np.float32(x * aff[0]) + aff[1])
            y = np.fmin(np.fmax(y, np.float32(2 ** 23)), np.float32(2 ** 23 + BUCKETS - 1))
            cell = y.view(np.uint32) & (BUCKETS - 1)
            j = pre[b - 1][cell].astype(np.int64)
            assert np.array_equal((j & 15) + (x >= flat[j]), ref)


def test_scaled_limbs_quantise_like_the_reference_rule():
    """Columns scaled by 1 / sigma and compared with the unit thresholds give the codes of the
    per-column thresholds except within rounding of a boundary (rate far below 1e-5)."""
    from jointqk_b200.codebooks import unit_gaussian_centroids
    from jointqk_b200.layout import unit_quantiser_tables

    rng = np.random.default_rng(1)
    unit = {b: unit_gaussian_centroids(b).numpy() for b in range(1, 5)}
    uthr, _, _ = unit_quantiser_tables(unit)
    bad = tot = 0
    for b in range(1, 5):
        for sigma in (1e-3, 0.37, 1.0, 21.5):
            cb = np.zeros((1, 16), np.float32)
            cb[0, : 2 ** b] = unit[b] * np.float32(sigma)
            thr = decision_thresholds(cb, np.array([b]))[0, : 2 ** b - 1]
            scale = np.float32(float(unit[b][-1]) / float(cb[0, 2 ** b - 1]))
            x = (rng.normal(size=400000) * sigma).astype(np.float32)
            want = (x[:, None] >= thr[None, :]).sum(-1)
            got = ((x * scale)[:, None] >= uthr[b - 1, : 2 ** b - 1][None, :]).sum(-1)
            bad += int((want != got).sum())
            tot += x.size
    assert bad / tot < 2e-6


def test_wide_decision_thresholds_reproduce_the_argmin():
    """Thresholds of 5..8-bit codebooks (256-entry rows): counting them gives the reference's
    first-minimum argmin over |x - level| in fp32, also for inputs right at the thresholds."""
    from jointqk_b200.codebooks import unit_gaussian_centroids

    rng = np.random.default_rng(11)
    for bits, sigma in ((5, 3.7), (6, 0.21), (7, 41.0), (8, 1.3)):
        levels = (unit_gaussian_centroids(bits) * float(np.float32(sigma))).numpy().astype(np.float32)
        rows = np.zeros((1, 256), np.float32)
        rows[0, :len(levels)] = levels
        thr = decision_thresholds(rows, np.array([bits]), max_levels=256)[0]
        n_thr = (1 << bits) - 1
        assert np.all(np.isfinite(thr[:n_thr])) and np.all(np.isinf(thr[n_thr:])) and np.all(np.diff(thr[:n_thr]) >= 0)
        x = np.concatenate([rng.normal(0, sigma, 20000).astype(np.float32), thr[:n_thr],
                            np.nextafter(thr[:n_thr], np.float32(-np.inf)), np.nextafter(thr[:n_thr], np.float32(np.inf))])
        want = np.abs(x[:, None] - levels[None, :]).argmin(1)                    # fp32, first minimum
        got = (x[:, None] >= thr[None, :n_thr]).sum(1)
        assert np.array_equal(got, want), bits


def test_packable_follows_the_record_limits():
    """A compressor knows whether the packed record holds its allocation: at most 32 coordinates above
    4 bits and 512 bits per key; beyond that ``roundtrip`` takes the record-free path (GPU tests)."""
    import jointqk_b200 as jq
    from jointqk_b200.compressor import _codebooks_packable

    stds = torch.ones(128)
    eye = torch.eye(128)
    fits = jq.PerCoordCompressor(torch.tensor([8] * 4 + [2] * 100 + [0] * 24), stds, eye, eye)
    too_many_wide = jq.PerCoordCompressor(torch.tensor([5] * 33 + [1] * 95), stds, eye, eye)
    too_long = jq.PerCoordCompressor(torch.tensor([8] * 32 + [4] * 96), stds, eye, eye)        # 256 + 384 bits
    assert fits.packable and fits.decodable
    assert not too_many_wide.packable and not too_many_wide.decodable
    assert not too_long.packable
    _, _, cb = jq.stack_per_head([fits, fits])
    assert _codebooks_packable(cb)
    _, _, cb = jq.stack_per_head([fits, too_long])
    assert not _codebooks_packable(cb)
