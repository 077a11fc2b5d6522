"""GPU parity of lookup-table scoring and paged decode attention against the oracle.

Scores are compared against the oracle's logits on the reconstruction of the *same codes*
(so a boundary flip in compression is not counted twice), within 2e-3 by the metric
max_i |s_i - ref_i| / max(|ref_i|, rms_row(ref)).  Top-1 retention on the parity config's
queries must equal the oracle's."""

import math

import pytest
import torch

import jointqk_b200 as jq
from jointqk_b200 import paged
from jointqk_b200.synthetic import config_seed, fit_sigma_k_heads, retrieval_queries, spectrum_keys
from gpu_util import recon_from_codes, score_rel_error
from oracle import reference_port as orc

pytestmark = pytest.mark.gpu
SCORE_TOL = 2e-3
OUT_TOL = 2e-3      # attention output, relative to max |out| of the row


def _setup(H, N, b_avg, cfg_layer=0, dtype=torch.float32):
    keys = torch.stack([spectrum_keys(N, config_seed(0, cfg_layer, h)) for h in range(H)]).to(dtype)
    comps, sig = fit_sigma_k_heads(keys.float(), b_avg)
    tables = jq.HeadTables.from_compressors(comps, device="cuda")
    return keys, comps, sig, tables


def _k_hat_from_packed(packed, comps):
    codes = paged.unpack_codes(packed).cpu()                      # (S, H, T, d)
    return torch.stack([torch.stack([recon_from_codes(comps[h], codes[s, h]) for h in range(len(comps))])
                        for s in range(codes.shape[0])])


@pytest.mark.parametrize("b_avg", [2.0, 3.0])
def test_parity_config_scores_and_top1(b_avg):
    H, N, NQ = 8, 4096, 256
    keys, comps, sig, tables = _setup(H, N, b_avg)
    packed = paged.compress(tables, keys.cuda().unsqueeze(0))
    q = torch.stack([retrieval_queries(keys[h], sig[h], NQ, config_seed(0, 0, h) + 7)[0] for h in range(H)])
    qq = q.unsqueeze(0)                                            # (1, H, NQ, d): one q head per kv head
    s = paged.score(packed, qq.cuda()).cpu()                        # fp32 sums
    s_tab = paged.score(packed, qq.cuda(), decode_tables=True).cpu()  # what the decode kernel scores with
    k_hat = _k_hat_from_packed(packed, comps)
    ref = orc.logits(qq, k_hat)
    err, err_tab = score_rel_error(s, ref), score_rel_error(s_tab, ref)
    print(f"score rel error b_avg={b_avg}: fp32 {err:.2e}, decode tables {err_tab:.2e}")
    assert err < 1e-5 and err_tab < SCORE_TOL
    # retention: argmax over compressed scores vs argmax over exact scores, GPU vs oracle
    real = orc.logits(qq, keys.unsqueeze(0))
    ret_gpu = (s.argmax(-1) == real.argmax(-1)).float().mean().item()
    ret_ref = orc.attention_metrics(qq, keys.unsqueeze(0), k_hat)["top1_match"]
    print(f"top-1 retention b_avg={b_avg}: gpu {ret_gpu:.4f} oracle {ret_ref:.4f}")
    assert torch.equal(s.argmax(-1), ref.argmax(-1))
    assert ret_gpu == ret_ref
    m = jq.compute_attention_metrics(qq, keys.unsqueeze(0), packed)
    assert m["top1_match"] == ret_ref


@pytest.mark.parametrize("hq,hkv,dtype", [(8, 2, torch.bfloat16), (2, 2, torch.float32), (16, 2, torch.bfloat16)])
def test_scores_gqa_groups(hq, hkv, dtype):
    keys, comps, _, tables = _setup(hkv, 777, 2.0, cfg_layer=3)
    kb = torch.stack([keys, keys.flip(1)]).cuda()
    packed = paged.compress(tables, kb, [777, 130])
    g = torch.Generator().manual_seed(hq)
    q = torch.randn(2, hq, 3, 128, generator=g).to(dtype)
    k_hat = _k_hat_from_packed(packed, comps)
    ref = orc.logits(q.float(), k_hat)
    for tables_mode in (False, True):
        s = paged.score(packed, q.cuda(), decode_tables=tables_mode).cpu()
        assert score_rel_error(s[0], ref[0]) < SCORE_TOL
        assert score_rel_error(s[1, :, :, :130], ref[1, :, :, :130]) < SCORE_TOL
        assert float(s[1, :, :, 130:].abs().max()) == 0.0


def _decode_case(lens, hq, hkv, b_avg, tokens_per_split=0, out_dtype=torch.float32, shuffle_pages=False):
    N = max(max(lens), 1)
    keys, comps, _, tables = _setup(hkv, N, b_avg, cfg_layer=5)
    S = len(lens)
    kb = torch.stack([keys.roll(7 * s, 1) for s in range(S)]).cuda()
    g = torch.Generator().manual_seed(1234 + S)
    v = torch.randn(S, hkv, N, 128, generator=g).to(torch.bfloat16)
    q = torch.randn(S, hq, 128, generator=g).to(torch.bfloat16)
    cache = paged.PagedKVCache(tables, [max(n, 1) for n in lens])
    if shuffle_pages:
        perm = torch.randperm(cache.n_pages, generator=g).to(torch.int32).cuda()
        cache.page_table = perm[cache.page_table.long()]
    cache.prefill(kb, v.cuda(), lens)
    out = cache.decode(q.cuda(), out_dtype=out_dtype, tokens_per_split=tokens_per_split).float().cpu()
    paged.check_status(cache.status)
    packed = paged.PackedKeys(tables, cache.k_pool, cache.page_table, cache.seq_lens, list(lens), cache.status)
    k_hat = _k_hat_from_packed(packed, comps)
    ref = torch.zeros(S, hq, 128)
    for s, n in enumerate(lens):
        if n:
            ref[s] = orc.decode_attention(q[s:s + 1], k_hat[s:s + 1, :, :n], v[s:s + 1, :, :n])[0]
    return out, ref


@pytest.mark.parametrize("lens,hq,hkv,b_avg,tps", [
    ([1000, 37, 1, 16], 8, 2, 2.0, 0),
    ([4096], 32, 8, 2.0, 0),
    ([4096], 32, 8, 2.0, 256),
    ([513, 0, 2048], 8, 2, 3.0, 512),
    ([300, 299], 2, 2, 2.5, 0),
    ([700], 16, 2, 3.0, 256),
    ([1500, 900], 8, 2, 1.0, 0),          # the smallest budget: most coordinates carry no bits
    ([1500, 900], 8, 2, 4.0, 0),          # the largest: 64-byte records, 16-level tables throughout
    ([6000, 5000], 32, 8, 2.0, 128)])     # 696 blocks: more than one wave, tables come from the table kernel
def test_decode_matches_oracle(lens, hq, hkv, b_avg, tps):
    out, ref = _decode_case(lens, hq, hkv, b_avg, tps)
    scale = ref.abs().amax(-1, keepdim=True).clamp_min(1e-6)
    err = ((out - ref).abs() / scale).max().item()
    print(f"decode lens={lens} hq={hq} hkv={hkv} bits={b_avg} tps={tps}: max rel err {err:.2e}")
    assert err < OUT_TOL
    for s, n in enumerate(lens):
        if n == 0:
            assert float(out[s].abs().max()) == 0.0


def test_decode_bf16_output_and_page_permutation_invariance():
    a, ref = _decode_case([1500, 640], 8, 2, 2.0, 0, out_dtype=torch.bfloat16)
    b, _ = _decode_case([1500, 640], 8, 2, 2.0, 0, out_dtype=torch.float32, shuffle_pages=True)
    scale = ref.abs().amax(-1, keepdim=True)
    assert ((a - ref).abs() / scale).max().item() < 1e-2          # bf16 rounding of the output
    assert ((b - ref).abs() / scale).max().item() < OUT_TOL


def test_decode_head_dim_64_matches_oracle():
    """The decode kernel's second head size: 64 dims, 8 q / 2 kv heads, two ragged sequences."""
    d, hkv, hq, lens = 64, 2, 8, [1100, 333]
    N = max(lens)
    keys = torch.stack([spectrum_keys(N, config_seed(0, 7, h), d=d) for h in range(hkv)])
    comps, _ = fit_sigma_k_heads(keys, 2.5)
    tables = jq.HeadTables.from_compressors(comps, device="cuda")
    g = torch.Generator().manual_seed(77)
    v = torch.randn(len(lens), hkv, N, d, generator=g).to(torch.bfloat16)
    q = torch.randn(len(lens), hq, d, generator=g).to(torch.bfloat16)
    cache = paged.PagedKVCache(tables, lens)
    cache.prefill(torch.stack([keys.roll(5 * s, 1) for s in range(len(lens))]).cuda(), v.cuda(), lens)
    out = cache.decode(q.cuda()).cpu()
    paged.check_status(cache.status)
    packed = paged.PackedKeys(tables, cache.k_pool, cache.page_table, cache.seq_lens, list(lens), cache.status)
    k_hat = _k_hat_from_packed(packed, comps)
    for s, n in enumerate(lens):
        ref = orc.decode_attention(q[s:s + 1], k_hat[s:s + 1, :, :n], v[s:s + 1, :, :n])[0]
        err = ((out[s] - ref).abs() / ref.abs().amax(-1, keepdim=True).clamp_min(1e-6)).max().item()
        assert err < OUT_TOL, err


def test_decode_from_host_buffers_equals_device_call():
    """PagedKVCache.decode_host (a replayed graph of H2D copy, decode, D2H copy, or one call of
    jqk_decode_attend_host) returns what decode() returns, also with a new query and after the cache
    has grown."""
    keys, comps, sig, tables = _setup(2, 2048, 2.0)
    g = torch.Generator().manual_seed(5)
    v = torch.randn(1, 2, 2048, 128, generator=g).to(torch.bfloat16)
    cache = paged.PagedKVCache(tables, [2048])
    cache.prefill(keys[:, :1500].unsqueeze(0).cuda(), v[:, :, :1500].cuda())
    for rep in range(3):
        q = torch.randn(1, 8, 128, generator=g).to(torch.bfloat16)
        if rep == 2:
            cache.prefill(keys[:, 1500:1501].unsqueeze(0).cuda(), v[:, :, 1500:1501].cuda())   # append one token
        want = cache.decode(q.cuda()).cpu()
        assert torch.equal(cache.decode_host(q).clone(), want)                    # replayed graph of H2D copy, decode, D2H copy
        assert torch.equal(cache.decode_host(q, zero_copy=True).clone(), want)    # one-kernel graph, kernel reads / writes host memory
        assert torch.equal(cache.decode_host(q, zero_copy="out").clone(), want)   # H2D copy, then the kernel writes the host result
        assert torch.equal(cache.decode_host(q, use_graph=False).clone(), want)   # jqk_decode_attend_host with device staging
        assert torch.equal(cache.decode_host(q, use_graph=False, zero_copy=True).clone(), want)   # ... without
    paged.check_status(cache.status)


@pytest.mark.parametrize("hq", [8, 16])
def test_appended_key_attends_exactly_in_its_own_step(hq):
    """Mode B of the reference compresses a decode key after the step that produced it
    (jointqk_press.py:298-304): in that step attention sees the exact key, later steps see its
    reconstruction.  jqk_decode_append_attend with JQK_APPEND_OWN_KEY_EXACT against the oracle's
    attention over [reconstructed history, exact new key]; the retrieval-style query makes the new
    key carry most of the weight, so the choice is visible in the output."""
    H, n0, steps = 2, 700, 5
    keys, comps, sig, tables = _setup(H, 2048, 2.0, dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(17)
    v = torch.randn(1, H, n0 + steps, 128, generator=g).to(torch.bfloat16)
    cache = paged.PagedKVCache(tables, [n0 + steps])
    cache.prefill(keys[:, :n0].unsqueeze(0).cuda(), v[:, :, :n0].cuda())
    for i in range(steps):
        k_new = keys[:, n0 + i].unsqueeze(0)                                     # (1, H, d) bf16
        v_new = v[:, :, n0 + i]
        q = (k_new.float().repeat_interleave(hq // H, 1) * 0.6 + 0.3 * torch.randn(1, hq, 128, generator=g)).to(torch.bfloat16)
        got = cache.generate_step(k_new.unsqueeze(2).cuda(), v_new.unsqueeze(2).cuda(), q.cuda(), own_key_exact=True).cpu()
        packed = paged.PackedKeys(tables, cache.k_pool, cache.page_table, cache.seq_lens, list(cache.lengths), cache.status)
        k_hat = _k_hat_from_packed(packed, comps)                               # (1, H, n0+i+1, d), the new key compressed
        k_own = k_hat.clone()
        k_own[:, :, -1] = k_new.float()
        ref_own = orc.decode_attention(q, k_own, v[:, :, :n0 + i + 1])
        ref_codes = orc.decode_attention(q, k_hat, v[:, :, :n0 + i + 1])
        scale = ref_own.abs().amax(-1, keepdim=True).clamp_min(1e-6)
        err = ((got - ref_own).abs() / scale).max().item()
        gap = ((ref_codes - ref_own).abs() / scale).max().item()
        assert err < OUT_TOL, (i, err)
        assert gap > 2 * OUT_TOL and gap > 4 * err, (gap, err)                    # the two semantics differ measurably here
    paged.check_status(cache.status)


def _wide_setup(H, N, b_avg, n_wide_extra=0):
    """Reference-default allocation (cap 8) on the parity spectrum: the four outlier channels get 5..8
    bits; ``n_wide_extra`` more coordinates are lifted to 8 bits to crowd the table memory."""
    keys = torch.stack([spectrum_keys(N, config_seed(0, 0, h)) for h in range(H)])
    comps, sig = fit_sigma_k_heads(keys, b_avg, max_bits=8)
    if n_wide_extra:
        lifted = []
        for c in comps:
            bits = c.bits_int.clone()
            idx = (bits <= 4).nonzero().flatten()[:n_wide_extra]
            bits[idx] = 8
            lifted.append(jq.PerCoordCompressor(bits, c.stds, c.forward_map, c.inverse_map))
        comps = lifted
    return keys, comps, sig, jq.HeadTables.from_compressors(comps, device="cuda")


@pytest.mark.parametrize("b_avg", [2.0, 2.5, 3.0])
def test_codes_above_4_bits_scores_decode_and_generate(b_avg):
    """The reference's default cap of 8: outlier coordinates carry 5..8-bit codes, a byte each in the
    record and a 256-entry lookup table each in the kernels.  Table scores against the oracle's
    logits, decode attention against the oracle, the one-launch generate step against append + decode."""
    H, N = 4, 3000
    keys, comps, sig, tables = _wide_setup(H, 4096, b_avg)
    assert tables.n_wide >= 4 and tables.decodable
    packed = paged.compress(tables, keys[:, :N].cuda().unsqueeze(0))
    k_hat = _k_hat_from_packed(packed, comps)
    want_codes = torch.stack([orc.nearest_codes(orc.transform(keys[h, :N], comps[h].forward_map), comps[h].codebooks_padded)
                              for h in range(H)])
    assert (paged.unpack_codes(packed)[0].cpu().long() != want_codes).float().mean().item() <= 1e-5
    q = torch.stack([retrieval_queries(keys[h], sig[h], 64, config_seed(0, 0, h) + 7)[0] for h in range(H)]).unsqueeze(0)
    ref = orc.logits(q, k_hat)
    s32 = paged.score(packed, q.cuda()).cpu()
    stab = paged.score(packed, q.cuda(), decode_tables=True).cpu()
    assert score_rel_error(s32, ref) < 1e-5 and score_rel_error(stab, ref) < SCORE_TOL
    g = torch.Generator().manual_seed(19)
    v = torch.randn(1, H, N + 8, 128, generator=g).to(torch.bfloat16)
    for tps in (0, 256):                                       # blocks build their tables / table kernel (48 blocks x 4 heads)
        cache = paged.PagedKVCache(tables, [N + 8])
        cache.prefill(keys[:, :N].unsqueeze(0).cuda(), v[:, :, :N].cuda())
        qd = torch.randn(1, 4 * H, 128, generator=g).to(torch.bfloat16)
        out = cache.decode(qd.cuda(), tokens_per_split=tps).cpu()
        want = orc.decode_attention(qd, k_hat, v[:, :, :N])
        err = ((out - want).abs() / want.abs().amax(-1, keepdim=True).clamp_min(1e-6)).max().item()
        assert err < OUT_TOL, (tps, err)
    plain = paged.PagedKVCache(tables, [N + 8])
    plain.prefill(keys[:, :N].unsqueeze(0).cuda(), v[:, :, :N].cuda())
    for i in range(8):                                         # the new key's wide codes come from the decode kernel itself
        kn, vn = keys[:, N + i].unsqueeze(0).unsqueeze(2).cuda(), v[:, :, N + i:N + i + 1].cuda()
        qd = torch.randn(1, 4 * H, 128, generator=g).to(torch.bfloat16).cuda()
        got = cache.generate_step(kn, vn, qd).clone()
        plain.append(kn, vn)
        want = plain.decode(qd)
        assert (got - want).abs().max().item() <= 1e-4 * want.abs().max().item(), i
    pk = [paged.PackedKeys(tables, c.k_pool, c.page_table, c.seq_lens, list(c.lengths), c.status) for c in (cache, plain)]
    assert torch.equal(paged.unpack_codes(pk[0]), paged.unpack_codes(pk[1]))
    paged.check_status(cache.status)


def test_too_many_wide_columns_for_the_table_memory_are_refused_by_decode_only():
    keys, comps, sig, tables = _wide_setup(2, 4096, 2.0, n_wide_extra=12)       # sixteen 256-entry tables would take 256 of 208 slots
    assert tables.n_wide >= 14 and not tables.decodable
    packed = paged.compress(tables, keys[:, :500].cuda().unsqueeze(0))          # stored, read back, scored from the reconstruction
    k_hat = _k_hat_from_packed(packed, comps)
    q = torch.randn(1, 2, 8, 128)
    assert score_rel_error(paged.score(packed, q.cuda()).cpu(), orc.logits(q, k_hat)) < 1e-5
    with pytest.raises(ValueError, match="max_bits=4"):
        paged.PagedKVCache(tables, [500]).decode(torch.zeros(1, 2, 128, dtype=torch.bfloat16, device="cuda"))


def test_decode_split_invariance_at_context_32768():
    """Full-context property: the result does not depend on how the keys are split over blocks."""
    H, N = 8, 32768
    keys = torch.stack([spectrum_keys(N, config_seed(1, 0, h), device="cuda") for h in range(H)])
    comps, _ = fit_sigma_k_heads(keys[:, :4096].cpu(), 2.0)
    tables = jq.HeadTables.from_compressors(comps, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(5)
    v = torch.randn(1, H, N, 128, generator=g, device="cuda").to(torch.bfloat16)
    q = torch.randn(1, 32, 128, generator=g, device="cuda").to(torch.bfloat16)
    cache = paged.PagedKVCache(tables, [N])
    cache.prefill(keys.unsqueeze(0), v)
    outs = [cache.decode(q, tokens_per_split=t) for t in (0, 1024, 4096, 32768)]
    for o in outs[1:]:
        assert ((o - outs[0]).abs().max() / outs[0].abs().max()).item() < 1e-4
    # repeated calls reuse the workspace (counters return to zero)
    again = cache.decode(q)
    assert torch.equal(again, outs[0])


def test_decode_rejects_bad_arguments():
    keys, comps, _, tables = _setup(2, 64, 2.0)
    cache = paged.PagedKVCache(tables, [64])
    with pytest.raises(ValueError):
        cache.decode(torch.zeros(1, 3, 128, dtype=torch.bfloat16, device="cuda"))     # 3 q heads over 2 kv heads
    with pytest.raises(ValueError):
        cache.decode(torch.zeros(1, 4, 128, dtype=torch.float32, device="cuda"))      # q must be bf16
    with pytest.raises(ValueError):
        cache.decode(torch.zeros(1, 4, 128, dtype=torch.bfloat16, device="cuda"), tokens_per_split=100)
