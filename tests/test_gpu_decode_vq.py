"""Decode attention over packed values (keys and values both stored as per-coordinate codes).

The oracle attends over the reference's reconstructions: keys from the K codes, values from the V
codes through ``CenteredCompressor`` semantics (dequantise, inverse map, add the mean;
experiments/stage1/toolkit/v_compressor_adapter.py:64-72).  The kernel multiplies bf16 centroids on
the tensor cores, so the comparison is made twice: against the oracle with the value centroids
rounded to bf16 like the kernel's (the arithmetic being checked) and against the exact fp32
reconstruction (which adds the rounding itself; the reference keeps reconstructed values in the
model's bf16 cache, which rounds as much).  Both within 2e-3 of the row maximum, as for bf16 values;
measured 1e-5 .. 8e-5 and 1e-4 .. 1.3e-3."""

import pytest
import torch

import jointqk_b200 as jq
from jointqk_b200 import paged
from jointqk_b200.synthetic import config_seed, fit_sigma_k_heads, second_moment, spectrum_keys
from gpu_util import recon_from_codes
from oracle import reference_port as orc

pytestmark = pytest.mark.gpu


def _setup(H, N, k_bits, v_bits, v_method="v_eigen_waterfill", layer=11, cap=4):
    keys = torch.stack([spectrum_keys(N, config_seed(0, layer, h)) for h in range(H)])
    comps, _ = fit_sigma_k_heads(keys[:, :4096], k_bits, max_bits=cap)
    tables = jq.HeadTables.from_compressors(comps, device="cuda")
    g = torch.Generator().manual_seed(layer)
    # (at the reference's cap of 8 the values get two outlier channels, so that codes of every width up to 8 occur)
    vals = torch.stack([spectrum_keys(N, config_seed(0, layer + 50, h), n_outliers=0 if cap == 4 else 2) for h in range(H)]) \
        + 0.3 * torch.randn(H, 1, 128, generator=g)
    v_comps = []
    for h in range(H):
        sig = second_moment(vals[h, :4096])
        mu = vals[h, :4096].double().mean(0).float()
        v_comps.append(jq.build_v_compressor(v_method, cov_v_for_head=sig - torch.outer(mu, mu), head_dim=128, bits=v_bits,
                                             seed=42 + h, mu_v_for_head=mu, max_bits=cap))
    v_tables = jq.HeadTables.from_compressors([c.inner for c in v_comps], device="cuda",
                                              center=torch.stack([c.mu for c in v_comps]))
    return keys, vals, comps, v_comps, tables, v_tables


def _case(lens, hq, hkv, k_bits, v_bits, tps=0, v_method="v_eigen_waterfill", cap=4):
    N = max(max(lens), 1)
    keys, vals, comps, v_comps, tables, v_tables = _setup(hkv, max(N, 4096), k_bits, v_bits, v_method, cap=cap)
    if cap > 4:
        assert tables.n_wide > 0 and v_tables.n_wide > 0
    S = len(lens)
    g = torch.Generator().manual_seed(99 + S)
    q = torch.randn(S, hq, 128, generator=g).to(torch.bfloat16)
    kb = torch.stack([keys.roll(7 * s, 1)[:, :N] for s in range(S)]).cuda()
    vb = torch.stack([vals.roll(5 * s, 1)[:, :N] for s in range(S)]).to(torch.bfloat16)
    cache = paged.PagedKVCache(tables, [max(n, 1) for n in lens], v_tables=v_tables)
    cache.prefill(kb, vb.cuda(), lens)
    out = cache.decode(q.cuda(), tokens_per_split=tps).cpu()
    paged.check_status(cache.status)
    pk = paged.PackedKeys(tables, cache.k_pool, cache.page_table, cache.seq_lens, list(lens), cache.status)
    pv = paged.PackedKeys(v_tables, cache.v_pool, cache.page_table, cache.seq_lens, list(lens), cache.status)
    k_codes, v_codes = paged.unpack_codes(pk).cpu(), paged.unpack_codes(pv).cpu()
    v_dec = paged.decompress(pv).cpu()
    ref = torch.zeros(S, hq, 128)
    ref16 = torch.zeros(S, hq, 128)
    bad = tot = 0
    for s, n in enumerate(lens):
        if n == 0:
            continue
        k_hat = torch.stack([recon_from_codes(comps[h], k_codes[s, h, :n]) for h in range(hkv)]).unsqueeze(0)
        v_hat, v_hat16 = [], []
        for h in range(hkv):
            c = v_comps[h]
            want, want_codes = orc.centred_roundtrip(vb[s, h, :n], c.mu, c.inner.codebooks_padded, c.inner.forward_map,
                                                     c.inner.inverse_map)
            bad += int((v_codes[s, h, :n].long() != want_codes).sum())
            tot += want_codes.numel()
            xh = orc.dequantise(v_codes[s, h, :n].long(), c.inner.codebooks_padded)
            v_hat.append(xh @ c.inner.inverse_map + c.mu)
            v_hat16.append(xh.to(torch.bfloat16).float() @ c.inner.inverse_map + c.mu)
            same = (v_codes[s, h, :n].long() == want_codes).all(-1)
            assert (v_dec[s, h, :n][same] - want[same]).abs().max().item() < 1e-5 * float(want.abs().max())
        ref[s] = orc.decode_attention(q[s:s + 1], k_hat, torch.stack(v_hat).unsqueeze(0))[0]
        ref16[s] = orc.decode_attention(q[s:s + 1], k_hat, torch.stack(v_hat16).unsqueeze(0))[0]
    scale = ref.abs().amax(-1, keepdim=True).clamp_min(1e-6)
    return out, ref, ref16, scale, bad / max(tot, 1)


@pytest.mark.parametrize("lens,hq,hkv,kb,vbits,tps,method", [
    ([1000, 37, 1, 16], 8, 2, 2.0, 3, 0, "v_eigen_waterfill"),
    ([4096], 32, 8, 2.0, 3, 0, "v_eigen_waterfill"),
    ([513, 0, 2048], 8, 2, 3.0, 2, 256, "v_eigen_waterfill"),
    ([700, 300], 16, 2, 3.0, 3, 128, "v_eigen_uniform"),
    ([1500, 900], 8, 2, 2.0, 4, 0, "v_random"),
    ([6000, 5000], 32, 8, 2.0, 3, 128, "v_eigen_waterfill")])        # 696 blocks: several waves
def test_packed_value_decode_matches_oracle(lens, hq, hkv, kb, vbits, tps, method):
    out, ref, ref16, scale, v_rate = _case(lens, hq, hkv, kb, vbits, tps, method)
    err16 = ((out - ref16).abs() / scale).max().item()
    err = ((out - ref).abs() / scale).max().item()
    print(f"packed V decode lens={lens} K {kb} bits V {vbits} bits ({method}) tps={tps}: rel err vs bf16-centroid oracle "
          f"{err16:.2e}, vs exact reconstruction {err:.2e}, V code mismatch rate {v_rate:.2e}")
    assert err16 < 2e-3 and err < 2e-3 and v_rate <= 1e-5
    for s, n in enumerate(lens):
        if n == 0:
            assert float(out[s].abs().max()) == 0.0


@pytest.mark.parametrize("lens,hq,hkv,kb,vbits,tps", [
    ([1000, 37, 1, 16], 8, 2, 2.0, 3, 0),
    ([3000, 2500], 32, 8, 2.5, 3, 128),          # several waves
    ([513, 0, 2048], 16, 2, 3.0, 2, 256)])
def test_packed_value_decode_at_the_reference_caps(lens, hq, hkv, kb, vbits, tps):
    """Keys and values both at the reference's default cap of 8 bits per coordinate
    (per_coord_quantization.py:367, v_compressor_adapter.py:165-226): byte-wide codes on both sides."""
    out, ref, ref16, scale, v_rate = _case(lens, hq, hkv, kb, vbits, tps, cap=8)
    err16 = ((out - ref16).abs() / scale).max().item()
    err = ((out - ref).abs() / scale).max().item()
    print(f"packed V decode at cap 8, lens={lens} K {kb} bits V {vbits} bits tps={tps}: rel err vs bf16-centroid oracle "
          f"{err16:.2e}, vs exact reconstruction {err:.2e}, V code mismatch rate {v_rate:.2e}")
    # the outlier channels' centroids are large, and their bf16 rounding (2^-9 relative, as in the bf16
    # cache the reference keeps its reconstructed values in) shows against the exact reconstruction
    assert err16 < 2e-3 and err < 1e-2 and v_rate <= 2e-5


def test_packed_values_append_and_bytes():
    """A generate loop over packed values: append one token at a time, then the same result as one
    prefill; and the cache holds what the bit budgets say."""
    keys, vals, comps, v_comps, tables, v_tables = _setup(2, 4096, 2.0, 3)
    n0, steps = 200, 20
    kb = keys[:, : n0 + steps].unsqueeze(0).cuda()
    vb = vals[:, : n0 + steps].unsqueeze(0).to(torch.bfloat16).cuda()
    a = paged.PagedKVCache(tables, n_seqs=1, v_tables=v_tables)
    a.prefill(kb[:, :, :n0], vb[:, :, :n0])
    for t in range(n0, n0 + steps):
        a.append(kb[:, :, t:t + 1], vb[:, :, t:t + 1])
    b = paged.PagedKVCache(tables, [n0 + steps], v_tables=v_tables)
    b.prefill(kb, vb)
    q = torch.randn(1, 8, 128, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16).cuda()
    assert torch.equal(a.decode(q), b.decode(q))
    assert a.v_pool.dtype == torch.int32 and a.v_pool.shape[2] == v_tables.words_per_record
    assert v_tables.payload_bytes_per_key == 48.0 and tables.payload_bytes_per_key == 32.0
    paged.check_status(a.status)


def test_decode_from_host_buffers_with_packed_values():
    """decode_host (replayed graph of H2D copy, decode over packed keys and values, D2H copy) returns
    what decode() returns."""
    keys, vals, comps, v_comps, tables, v_tables = _setup(2, 4096, 2.0, 3)
    cache = paged.PagedKVCache(tables, [3000], v_tables=v_tables)
    cache.prefill(keys[:, :3000].unsqueeze(0).cuda(), vals[:, :3000].to(torch.bfloat16).unsqueeze(0).cuda())
    g = torch.Generator().manual_seed(4)
    for _ in range(2):
        q = torch.randn(1, 8, 128, generator=g).to(torch.bfloat16)
        want = cache.decode(q.cuda()).cpu()
        assert torch.equal(cache.decode_host(q).clone(), want)
        assert torch.equal(cache.decode_host(q, zero_copy="out").clone(), want)
    with pytest.raises(NotImplementedError):
        cache.decode_host(q, use_graph=False)
    paged.check_status(cache.status)


@pytest.mark.parametrize("dtype,cap", [(torch.bfloat16, 4), (torch.float32, 4), (torch.bfloat16, 8)])
def test_fused_append_with_packed_values_equals_the_separate_launches(dtype, cap):
    """jqk_decode_append_attend_packed_values against the graph of compress (K), compress (V, centred),
    length and decode launches: same outputs, same key and value codes in the pages, same lengths,
    over ragged sequences that cross page and split boundaries.  (cap 8: byte-wide codes on both sides.)"""
    keys, vals, comps, v_comps, tables, v_tables = _setup(2, 4096, 2.0, 3, cap=cap)
    n0, steps = [370, 29, 1], 50
    total = max(n0) + steps
    g = torch.Generator().manual_seed(11)
    kk = torch.stack([keys[:, :total].roll(5 * s, 1) for s in range(3)]).cuda()
    vv = torch.stack([vals[:, :total].roll(9 * s, 1) for s in range(3)]).to(torch.bfloat16).cuda()
    qs = torch.randn(steps, 3, 8, 128, generator=g).to(torch.bfloat16).cuda()
    caches = [paged.PagedKVCache(tables, [n + steps for n in n0], v_tables=v_tables) for _ in range(2)]
    for c in caches:
        c.prefill(kk[:, :, :max(n0)], vv[:, :, :max(n0)], lengths=n0)
    for i in range(steps):
        kn = torch.stack([kk[s, :, n0[s] + i] for s in range(3)]).to(dtype).unsqueeze(2)
        vn = torch.stack([vv[s, :, n0[s] + i] for s in range(3)]).to(dtype).unsqueeze(2)
        got = caches[0].generate_step(kn, vn, qs[i]).clone()
        want = caches[1].generate_step(kn, vn, qs[i], fused_append=False)
        assert torch.equal(got, want), f"step {i}: {(got - want).abs().max().item()}"
    a, b = caches
    assert a._gen_step["fused"] and not b._gen_step["fused"]
    assert a.seq_lens.tolist() == b.seq_lens.tolist() == a.lengths == [n + steps for n in n0]
    for s in range(3):
        for t, pool in ((tables, "k_pool"), (v_tables, "v_pool")):
            pk = [paged.PackedKeys(t, getattr(c, pool), c.page_table[s:s + 1], c.seq_lens[s:s + 1], [c.lengths[s]], c.status)
                  for c in caches]
            assert torch.equal(paged.unpack_codes(pk[0]), paged.unpack_codes(pk[1])), (s, pool)
    for c in caches:
        paged.check_status(c.status)


def test_value_tables_whose_wide_levels_outgrow_the_kernel_are_refused_by_decode_only():
    """Twenty-five 8-bit value columns carry 6400 levels, more than the decode kernel holds (6144):
    the rows are still packed and reconstructed, decode over them raises."""
    H, N = 2, 600
    g = torch.Generator().manual_seed(5)
    bits = torch.tensor([8] * 25 + [2] * 60 + [0] * 43)
    R = jq.generate_rotation_matrix(128, seed=3)
    stds = torch.exp(0.3 * torch.randn(128, generator=g))
    v_comps = [jq.PerCoordCompressor(bits, stds, R, R.T) for _ in range(H)]
    v_tables = jq.HeadTables.from_compressors(v_comps, device="cuda", center=torch.zeros(H, 128))
    assert v_tables.n_wide == 25 and not v_tables.value_decodable
    keys = torch.stack([spectrum_keys(N, config_seed(0, 0, h)) for h in range(H)])
    comps, _ = fit_sigma_k_heads(keys, 2.0)
    tables = jq.HeadTables.from_compressors(comps, device="cuda")
    vals = ((torch.randn(H, N, 128, generator=g) * stds) @ R.T).to(torch.bfloat16)
    cache = paged.PagedKVCache(tables, [N], v_tables=v_tables)
    cache.prefill(keys.unsqueeze(0).cuda(), vals.unsqueeze(0).cuda())
    pv = paged.PackedKeys(v_tables, cache.v_pool, cache.page_table, cache.seq_lens, [N], cache.status)
    want = torch.stack([orc.roundtrip(vals[h], v_comps[h].codebooks_padded, v_comps[h].forward_map, v_comps[h].inverse_map)[0]
                        for h in range(H)])
    got = paged.decompress(pv).cpu()[0]
    ok = ((got - want).abs().amax(-1) < 1e-4 * float(want.abs().max())).float().mean().item()
    assert ok > 0.99                      # (rows with a code on a threshold may differ)
    with pytest.raises(ValueError, match="exceed the 6144"):
        cache.decode(torch.zeros(1, 8, 128, dtype=torch.bfloat16, device="cuda"))
    paged.check_status(cache.status)
