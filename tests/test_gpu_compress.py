"""GPU parity of prefill compression / reconstruction against the oracle and the reference
fixtures.  Codes: bit-exact except on coordinates within rounding of a decision boundary
(mismatch rate <= 1e-5).  Reconstruction: max-abs < 1e-5 * scale on rows whose codes agree."""

import numpy as np
import pytest
import torch

import jointqk_b200 as jq
from jointqk_b200 import paged
from jointqk_b200.synthetic import config_seed, fit_sigma_k_heads, spectrum_keys
from gpu_util import code_mismatch, oracle_codes_and_recon
from oracle import reference_port as orc

pytestmark = pytest.mark.gpu
MAX_RATE = 1e-5


def _t(a):
    return torch.from_numpy(np.asarray(a))


def _golden_comp(g, which):
    if which == "a":
        R = _t(g["R_sym"])
        return jq.PerCoordCompressor(_t(g["bits_cap4"]), _t(g["ref_stds"]), R, R.T)
    R = _t(g["basis_b"])
    return jq.PerCoordCompressor(_t(g["bits_b"]), _t(g["stds_b"]), R, R.T)


@pytest.mark.parametrize("which,codes_name,rt_name,dtype", [
    ("a", "ref_codes_cap4", "ref_roundtrip_cap4", torch.float32),
    ("a", "ref_codes_cap4_bf16", "ref_roundtrip_cap4_bf16", torch.bfloat16),
    ("b", "ref_codes_b", "ref_roundtrip_b", torch.float32)])
def test_codes_and_roundtrip_against_reference_fixture(golden, which, codes_name, rt_name, dtype):
    g = golden("compressor")
    comp = _golden_comp(g, which)
    keys = _t(g["keys"]).to(dtype).cuda()
    codes = comp.codes(keys)
    bad, _ = code_mismatch(codes, _t(g[codes_name]))
    assert bad <= 1, f"{bad} code mismatches on 32768 coordinates"
    out = comp.roundtrip(keys)
    assert out.dtype == torch.float32 and out.shape == keys.shape and out.is_cuda
    ref = _t(g[rt_name])
    row_ok = (codes.cpu() == _t(g[codes_name])).all(-1)
    err = (out.cpu() - ref)[row_ok].abs().max().item()
    assert err < 1e-5 * max(1.0, ref.abs().max().item()), err


def test_reference_default_cap8_roundtrip_against_reference_fixture(golden):
    """The reference's own recipe, cap of 8 bits per coordinate untouched
    (build_method_compressor defaults, per_coord_quantization.py:365-379): outlier coordinates take a
    byte each in the record.  Bits, stds and codebooks equal the fixture bit for bit; the GPU
    roundtrip equals the reference's roundtrip except on rows where a code sits on a decision
    threshold; the codes equal the oracle's."""
    g = golden("compressor")
    R = _t(g["R_sym"])
    comp = jq.build_method_compressor("r_sym_waterfill", _t(g["sigma_q"]), _t(g["sigma_k"]), None, None, None, 2.0, None, 0,
                                      128, R_sym=R)
    assert torch.equal(comp.bits_int, _t(g["ref_bits_cap8"]).long()) and torch.equal(comp.codebooks_padded, _t(g["ref_codebooks_cap8"]))
    assert int(comp.bits_int.max()) > 4 and comp.packable and comp.decodable
    keys = _t(g["keys"])
    out = comp.roundtrip(keys.cuda()).cpu()
    ref = _t(g["ref_roundtrip_cap8"])
    bad_rows = ((out - ref).abs().amax(-1) > 1e-5 * max(1.0, ref.abs().max().item())).sum().item()
    assert bad_rows <= 1, bad_rows
    want = orc.nearest_codes(orc.transform(keys, comp.forward_map), comp.codebooks_padded)
    bad, _ = code_mismatch(comp.codes(keys.cuda()), want.to(torch.uint8))
    assert bad <= 1, bad
    # the same through the token kernel (one key at a time) and the batched call
    one = torch.cat([comp.roundtrip(keys[i:i + 1].cuda()).cpu() for i in range(8)])
    assert ((one - ref[:8]).abs().amax(-1) > 1e-5 * max(1.0, ref.abs().max().item())).sum().item() == 0


def test_roundtrip_accepts_cpu_tensors_and_leading_dims(golden):
    g = golden("compressor")
    comp = _golden_comp(g, "b")
    keys = _t(g["keys"]).view(2, 4, 32, 128)
    out = comp.roundtrip(keys)
    assert out.device.type == "cpu" and out.shape == keys.shape
    ref = _t(g["ref_roundtrip_b"]).view(2, 4, 32, 128)
    assert ((out - ref).abs().amax(-1) > 1e-4).sum() <= 1


def test_batched_roundtrip_against_reference_fixture(golden):
    g = golden("compressor")
    ca, cb = _golden_comp(g, "a"), _golden_comp(g, "b")
    fwd, inv, cbs = jq.stack_per_head([ca, cb])
    keys = _t(g["keys"])
    kb = torch.stack([keys, keys.flip(0)], 0).unsqueeze(0).cuda()
    out = jq.batched_roundtrip(kb, fwd, inv, cbs)
    assert out.shape == kb.shape and out.dtype == kb.dtype
    ref = _t(g["ref_batched_roundtrip"])
    assert ((out.cpu() - ref).abs().amax(-1) > 1e-4).sum() <= 2
    out16 = jq.batched_roundtrip(kb.to(torch.bfloat16), fwd, inv, cbs)
    assert out16.dtype == torch.bfloat16


@pytest.mark.parametrize("b_avg,dtype,n_out,scale", [(2.0, torch.float32, 4, 15.0), (3.0, torch.float32, 4, 15.0),
                                                      (2.5, torch.bfloat16, 8, 20.0), (1.0, torch.bfloat16, 4, 15.0),
                                                      (4.0, torch.bfloat16, 4, 15.0), (4.0, torch.float32, 4, 15.0)])
def test_parity_config_codes(b_avg, dtype, n_out, scale):
    """8 heads x 4096 keys of the parity config: codes vs the oracle, mismatch rate reported."""
    H, N = 8, 4096
    keys = torch.stack([spectrum_keys(N, config_seed(0, 0, h), n_out, scale) for h in range(H)]).to(dtype)
    comps, _ = fit_sigma_k_heads(keys.float(), b_avg)
    tables = jq.HeadTables.from_compressors(comps, device="cuda")
    assert tables.record_bytes == int(b_avg * 16)
    packed = paged.compress(tables, keys.cuda().unsqueeze(0))
    codes = paged.unpack_codes(packed)[0].cpu()
    recon = paged.decompress(packed)[0].cpu()
    paged.check_status(packed.status)
    total_bad = 0
    for h in range(H):
        ref_codes, ref_out = oracle_codes_and_recon(comps[h], keys[h])
        bad, _ = code_mismatch(codes[h], ref_codes)
        total_bad += bad
        ok = (codes[h].long() == ref_codes).all(-1)
        err = (recon[h] - ref_out)[ok].abs().max().item()
        assert err < 1e-5 * max(1.0, ref_out.abs().max().item())
        assert int(codes[h].max()) <= 15 and (codes[h][:, comps[h].bits_int == 0] == 0).all()
    rate = total_bad / (H * N * 128)
    print(f"code mismatch rate b_avg={b_avg} {dtype}: {total_bad}/{H * N * 128} = {rate:.2e}")
    assert rate <= MAX_RATE


def test_ragged_empty_and_append_equivalence():
    H, d = 2, 128
    keys = torch.stack([spectrum_keys(300, config_seed(0, 1, h)) for h in range(H)])
    comps, _ = fit_sigma_k_heads(keys, 3.0)
    tables = jq.HeadTables.from_compressors(comps, device="cuda")
    kb = torch.stack([keys, keys.flip(1), keys * 0.5]).cuda()                 # 3 sequences
    lens = [300, 37, 0]
    packed = paged.compress(tables, kb, lens)
    codes = paged.unpack_codes(packed).cpu()
    one = paged.unpack_codes(paged.compress(tables, kb[:1])).cpu()
    assert torch.equal(codes[0], one[0])
    two = paged.unpack_codes(paged.compress(tables, kb[1:2, :, :37])).cpu()
    assert torch.equal(codes[1, :, :37], two[0])
    assert int(codes[1, :, 37:].abs().sum()) == 0 and int(codes[2].abs().sum()) == 0
    # empty batch and empty sequences do not launch and do not fail
    empty = paged.compress(tables, kb[:1, :, :0])
    assert paged.decompress(empty).shape == (1, H, 0, d)
    # appending 23 then 277 keys (mid-page boundary) equals one shot of 300
    cache = paged.PagedKVCache(tables, [300])
    v = torch.zeros(1, H, 300, d, device="cuda", dtype=torch.bfloat16)
    cache.prefill(kb[:1, :, :23], v[:, :, :23])
    cache.prefill(kb[:1, :, 23:], v[:, :, 23:])
    n_pages_used = packed.page_table[0, : paged.pages_for(300)]
    assert torch.equal(cache.k_pool[: paged.pages_for(300)], packed.k_pool[n_pages_used.long()])
    paged.check_status(cache.status)


def test_bad_page_index_sets_status_and_is_skipped():
    keys = spectrum_keys(64, config_seed(0, 2, 0))[None]
    comps, _ = fit_sigma_k_heads(keys, 2.0)
    tables = jq.HeadTables.from_compressors(comps, device="cuda")
    packed = paged.compress(tables, keys.cuda().unsqueeze(0))
    packed.page_table[0, 1] = 10_000                       # outside the pool
    paged.decompress(packed)
    with pytest.raises(RuntimeError, match="outside the pool"):
        paged.check_status(packed.status)


def test_small_head_dim_and_identity_map():
    d = 64
    g = torch.Generator().manual_seed(4)
    x = torch.randn(100, d, generator=g) * torch.linspace(3, 0.1, d)
    bits = torch.tensor([4] * 8 + [3] * 12 + [2] * 20 + [1] * 12 + [0] * 12)
    comp = jq.PerCoordCompressor(bits, torch.linspace(3, 0.1, d))          # no maps: identity
    from oracle import reference_port as orc
    ref, ref_codes = orc.roundtrip(x, comp.codebooks_padded, None, None)
    assert torch.equal(comp.codes(x).long(), ref_codes)
    assert torch.allclose(comp.roundtrip(x), ref, atol=1e-6)


def test_idempotence_at_scale():
    """Full-size property: re-compressing the reconstruction reproduces the codes."""
    H, N = 8, 32768
    keys = torch.stack([spectrum_keys(N, config_seed(4, 0, h), 8, 20.0, device="cuda") for h in range(H)])
    comps, _ = fit_sigma_k_heads(keys[:, :4096].cpu(), 2.5)
    tables = jq.HeadTables.from_compressors(comps, device="cuda")
    p1 = paged.compress(tables, keys.to(torch.bfloat16).unsqueeze(0))
    c1 = paged.unpack_codes(p1)
    p2 = paged.compress(tables, paged.decompress(p1))
    c2 = paged.unpack_codes(p2)
    rate = float((c1 != c2).float().mean())
    assert rate <= MAX_RATE, rate


def test_tensor_core_path_ragged_bf16_and_append():
    """bf16 keys take the tcgen05 kernel: ragged batch, tile tails, a mid-page append offset and
    a strided (non-contiguous) key tensor, all against the oracle's codes."""
    H = 3
    base = torch.stack([spectrum_keys(700, config_seed(4, 1, h), 8, 20.0) for h in range(H)])
    comps, _ = fit_sigma_k_heads(base, 2.5)
    tables = jq.HeadTables.from_compressors(comps, device="cuda")
    keys = torch.stack([base, base.flip(1), base * 0.7, base.roll(5, 1)]).to(torch.bfloat16)      # (4, H, 700, d)
    lens = [700, 129, 0, 512]
    # a view with a larger token stride (e.g. keys living inside a fused qkv buffer)
    wide = torch.zeros(4, H, 700, 256, dtype=torch.bfloat16, device="cuda")
    wide[..., :128] = keys.cuda()
    packed = paged.compress(tables, wide[..., :128], lens)
    paged.check_status(packed.status)
    codes = paged.unpack_codes(packed).cpu()
    bad = 0
    for s, n in enumerate(lens):
        for h in range(H):
            ref_codes, _ = oracle_codes_and_recon(comps[h], keys[s, h, :n])
            bad += int((codes[s, h, :n].long() != ref_codes).sum())
        assert int(codes[s, :, n:].abs().sum()) == 0
    assert bad <= 2, bad
    # append at a mid-page offset: 23 keys through the fp32 kernel, then 677 through the tensor cores
    cache = paged.PagedKVCache(tables, [700])
    v = torch.zeros(1, H, 700, 128, device="cuda", dtype=torch.bfloat16)
    cache.prefill(keys[:1, :, :23].cuda(), v[:, :, :23])
    cache.prefill(keys[:1, :, 23:].cuda(), v[:, :, 23:])
    paged.check_status(cache.status)
    pk = paged.PackedKeys(tables, cache.k_pool, cache.page_table, cache.seq_lens, [700], cache.status)
    again = paged.unpack_codes(pk).cpu()
    assert int((again[0] != codes[0]).sum()) <= 2


@pytest.mark.parametrize("hist", [
    (0, 128, 0, 0, 0),       # every column 1-bit: four words of 32 columns
    (0, 0, 128, 0, 0),       # every column 2-bit
    (0, 64, 0, 64, 0),       # (3,1) pairs only
    (0, 0, 0, 0, 128),       # every column 4-bit: sixteen words
    (10, 33, 21, 30, 34),    # odd counts: slots and bytes of every kind, words shared by two regions
    (100, 9, 7, 7, 5),       # few active columns, a record of two words
    (0, 2, 43, 42, 41),      # (3,3,2) bytes
    (60, 20, 20, 12, 12, 1, 1, 1, 1),     # the reference's cap of 8: one word of byte-wide codes, every width 5..8
    (0, 36, 36, 18, 18, 5, 5, 5, 5),      # twenty byte-wide columns: five words, units of two and of one
    (32, 0, 0, 0, 64, 0, 0, 0, 32),       # the most a record holds: thirty-two 8-bit columns beside regular 4-bit words
    (90, 10, 10, 10, 5, 0, 2, 0, 1),      # three byte-wide columns: a word with a free byte
])
def test_tensor_core_path_allocations(hist):
    """Allocations that reach each way the tensor-core kernel quantises a 16-column read (general
    lookups, plain comparisons for 1- and 2-bit columns, regular 4-bit and (3,1) words, units of one
    and two words): bf16 keys, two ragged sequences, codes against the oracle."""
    H, N, d = 2, 1500, 128
    gen = torch.Generator().manual_seed(1234 + sum(i * c for i, c in enumerate(hist)))
    comps, keys = [], []
    for h in range(H):
        bits = torch.cat([torch.full((c,), b, dtype=torch.long) for b, c in enumerate(hist)])
        bits = bits[torch.randperm(d, generator=gen)]
        R = jq.generate_rotation_matrix(d, seed=77 + h)
        stds = torch.exp(torch.randn(d, generator=gen))
        x = torch.randn(N, d, generator=gen) * stds
        keys.append((x @ R.T).to(torch.bfloat16))
        comps.append(jq.PerCoordCompressor(bits, stds, R, R.T))
    tables = jq.HeadTables.from_compressors(comps, device="cuda")
    assert tables.fwd_limbs is not None and (tables.n_wide > 0) == (len(hist) > 5)   # the tensor-core kernel serves them all
    kb = torch.stack([torch.stack(keys), torch.stack(keys).flip(1)])              # (2, H, N, d)
    lens = [N, 700]
    packed = paged.compress(tables, kb.cuda(), lens)
    paged.check_status(packed.status)
    codes = paged.unpack_codes(packed).cpu()
    bad = total = step = 0
    for s, n in enumerate(lens):
        for h in range(H):
            ref_codes, _ = oracle_codes_and_recon(comps[h], kb[s, h, :n])
            diff = (codes[s, h, :n].long() - ref_codes).abs()
            bad += int((diff != 0).sum())
            step = max(step, int(diff.max()))
            total += n * d
    print(f"code mismatch rate hist={hist}: {bad}/{total}")
    # a value within an fp32 rounding of a decision threshold may fall either side; an 8-bit coordinate
    # has 255 thresholds for that to happen at, a 4-bit one 15
    n_wide_coords = total * sum(hist[5:]) // d
    assert step <= 1 and bad <= max(2, int(MAX_RATE * total + 1e-4 * n_wide_coords)), (bad, step)


def test_tensor_core_path_centred_rows_at_the_reference_cap():
    """Value-side tables as the reference builds them by default (eigenbasis water-fill, cap 8,
    mean-centred): outlier coordinates carry byte-wide codes, the rows go through the tensor-core
    kernel raw and the mean leaves in column space; codes and reconstruction against the oracle."""
    from jointqk_b200.synthetic import config_seed, second_moment, spectrum_keys

    H, N = 2, 3000
    g = torch.Generator().manual_seed(11)
    vals = torch.stack([spectrum_keys(N, config_seed(0, 60, h)) for h in range(H)]) + 0.3 * torch.randn(H, 1, 128, generator=g)
    v_comps = []
    for h in range(H):
        mu = vals[h].double().mean(0).float()
        v_comps.append(jq.build_v_compressor("v_eigen_waterfill", cov_v_for_head=second_moment(vals[h]) - torch.outer(mu, mu),
                                             head_dim=128, bits=3, seed=42 + h, mu_v_for_head=mu))      # max_bits: the default 8
    assert max(int(c.inner.bits_int.max()) for c in v_comps) > 4
    tables = jq.HeadTables.from_compressors([c.inner for c in v_comps], device="cuda", center=torch.stack([c.mu for c in v_comps]))
    assert tables.n_wide > 0 and tables.fwd_limbs is not None and tables.center_cols is not None
    vb = vals.to(torch.bfloat16).unsqueeze(0)
    packed = paged.compress(tables, vb.cuda())
    paged.check_status(packed.status)
    codes = paged.unpack_codes(packed).cpu()
    out = paged.decompress(packed).cpu()
    bad = 0
    for h in range(H):
        c = v_comps[h]
        want, want_codes = orc.centred_roundtrip(vb[0, h], c.mu, c.inner.codebooks_padded, c.inner.forward_map, c.inner.inverse_map)
        bad += int((codes[0, h].long() != want_codes).sum())
        same = (codes[0, h].long() == want_codes).all(-1)
        assert (out[0, h][same] - want[same]).abs().max().item() < 1e-5 * max(1.0, want.abs().max().item())
    print(f"centred cap-8 rows: {bad} code mismatches of {H * N * 128}")
    assert bad <= max(2, int(MAX_RATE * H * N * 128)), bad


def test_allocations_beyond_the_record_roundtrip_without_one(golden):
    """The reference's default cap of 8 at 4.0 bits per coordinate puts 40-odd coordinates above 4
    bits and 600-odd bits in a key: more than the packed record holds.  ``roundtrip``, ``codes``,
    ``batched_roundtrip`` and the centred wrapper then run through jqk_roundtrip_dense; codes and
    reconstruction against the oracle, and the same codes as the packed path where both apply."""
    H, N = 2, 3000
    keys = torch.stack([spectrum_keys(N, config_seed(0, 0, h)) for h in range(H)])
    comps, _ = fit_sigma_k_heads(keys, 4.0, max_bits=8)
    assert not comps[0].packable and int((comps[0].bits_int > 4).sum()) > 32
    with pytest.raises(ValueError, match="512 bits per key"):
        comps[0].compress(keys[0].cuda())
    bad = 0
    for h in range(H):
        c = comps[h]
        want, want_codes = orc.roundtrip(keys[h], c.codebooks_padded, c.forward_map, c.inverse_map)
        codes = c.codes(keys[h].cuda()).cpu()
        out = c.roundtrip(keys[h].cuda()).cpu()
        bad += int((codes.long() != want_codes).sum())
        same = (codes.long() == want_codes).all(-1)
        assert (out[same] - want[same]).abs().max().item() < 1e-5 * max(1.0, want.abs().max().item())
        assert c.roundtrip(keys[h].to(torch.bfloat16)).device.type == "cpu"        # host rows in, host rows out
    print(f"record-free roundtrip at 4.0 bits, cap 8: {bad} code mismatches of {H * N * 128}")
    assert bad <= 1e-4 * H * N * 128
    fwd, inv, cb = jq.stack_per_head(comps)
    got = jq.batched_roundtrip(keys.unsqueeze(0).cuda(), fwd, inv, cb).cpu()[0]
    for h in range(H):
        assert torch.equal(got[h], comps[h].roundtrip(keys[h].cuda()).cpu())
    # centred rows (the value side's wrapper)
    mu = keys[0].mean(0) + 0.5
    cc = jq.CenteredCompressor(comps[0], mu)
    want, _ = orc.centred_roundtrip(keys[0] + 0.5, mu, comps[0].codebooks_padded, comps[0].forward_map, comps[0].inverse_map)
    got = cc.roundtrip((keys[0] + 0.5).cuda()).cpu()
    close = ((got - want).abs().amax(-1) < 1e-4 * float(want.abs().max())).float().mean().item()
    assert close > 0.99
    # where the record applies too, both paths assign the same codes (fp32 rows: the CUDA-core kernels)
    from jointqk_b200.dense import DenseTables

    small, _ = fit_sigma_k_heads(keys, 2.0, max_bits=8)
    dense = DenseTables(small[0].forward_map.unsqueeze(0), small[0].inverse_map.unsqueeze(0),
                        small[0].codebooks_padded.unsqueeze(0), torch.device("cuda", 0))
    out_d, codes_d = dense.roundtrip(keys[:1].cuda(), want_codes=True)
    assert small[0].packable and torch.equal(codes_d[0], small[0].codes(keys[0].cuda()))
    assert torch.allclose(out_d[0], small[0].roundtrip(keys[0].cuda()), atol=1e-5 * float(keys.abs().max()))
