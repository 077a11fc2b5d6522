"""GPU tests of the paged cache around the kernels: the value-store kernel against a plain torch
statement of the V page layout, appends at every slot offset, page allocation / growth / release,
the status bits for over-long lengths and expired waits, and the lifetime of the split workspace
behind a captured decode graph."""

import pytest
import torch

import jointqk_b200 as jq
from jointqk_b200 import _native, paged
from jointqk_b200.synthetic import config_seed, fit_sigma_k_heads, spectrum_keys
from gpu_util import recon_from_codes
from oracle import reference_port as orc

pytestmark = pytest.mark.gpu


def _tables(H, d=128, b_avg=2.0, layer=9):
    keys = torch.stack([spectrum_keys(2048, config_seed(0, layer, h), d=d) for h in range(H)])
    comps, _ = fit_sigma_k_heads(keys, b_avg)
    return keys, comps, jq.HeadTables.from_compressors(comps, device="cuda")


def _v_reference(v_pool, page_table, s, lengths, H, d):
    """(H, n, d) values of sequence s read back from the pool with the layout formula of the header."""
    n = lengths[s]
    pos = torch.arange(n, device=v_pool.device)
    pages = page_table[s, pos // 16].long()
    offs = paged.v_slot_offsets(d, v_pool.device)[pos % 16]                 # (n, d)
    return v_pool[pages[:, None], :, offs].permute(2, 0, 1)              # (H, n, d)


@pytest.mark.parametrize("dtype,d", [(torch.bfloat16, 128), (torch.float32, 128), (torch.float16, 64)])
def test_value_store_matches_layout_and_append_at_every_offset(dtype, d):
    H = 2
    _, _, tables = _tables(H, d=d)
    g = torch.Generator().manual_seed(3)
    lens = [50, 0, 17]
    cache = paged.PagedKVCache(tables, n_seqs=3)
    v_all = torch.randn(3, H, 200, d, generator=g).to(dtype).cuda()
    k_all = torch.randn(3, H, 200, d, generator=g).cuda()
    cache.prefill(k_all[:, :, :50], v_all[:, :, :50], lens)
    done = list(lens)
    # strided input (a slice of a larger tensor), then one append per slot offset 0..15
    for step, n in enumerate([1, 1, 2, 3, 1, 5, 1, 1, 16, 1, 7, 1, 1, 1, 9, 1, 1]):
        add = [n, 1 if step % 3 == 0 else 0, n]
        ks = torch.stack([k_all[s, :, done[s]:done[s] + max(add)] for s in range(3)])
        vs = torch.stack([v_all[s, :, done[s]:done[s] + max(add)] for s in range(3)])
        cache.prefill(ks, vs, add)
        done = [a + b for a, b in zip(done, add)]
    paged.check_status(cache.status)
    assert cache.lengths == done
    for s in range(3):
        got = _v_reference(cache.v_pool, cache.page_table, s, done, H, d)
        want = v_all[s, :, :done[s]].to(torch.bfloat16)
        assert torch.equal(got, want), f"sequence {s}"


def test_pool_growth_release_and_reuse_keep_results():
    H = 2
    keys, comps, tables = _tables(H)
    g = torch.Generator().manual_seed(4)
    v = torch.randn(2, H, 2048, 128, generator=g).to(torch.bfloat16).cuda()
    q = torch.randn(2, 8, 128, generator=g).to(torch.bfloat16).cuda()
    kk = torch.stack([keys, keys.flip(1)]).cuda()
    fixed = paged.PagedKVCache(tables, [2048, 2048])
    fixed.prefill(kk, v)
    want = fixed.decode(q)
    grown = paged.PagedKVCache(tables, n_seqs=2, initial_pages=3)          # far too small: the pool must grow
    gen0 = grown.pool.generation
    for lo, hi in [(0, 100), (100, 101), (101, 900), (900, 2048)]:
        grown.prefill(kk[:, :, lo:hi], v[:, :, lo:hi])
    assert grown.pool.generation > gen0 and grown.lengths == [2048, 2048]
    assert torch.equal(grown.decode(q), want)
    # release one sequence: its pages go back and are handed out again
    free_before = grown.pool.n_free
    grown.release(0)
    assert grown.pool.n_free == free_before + 128 and grown.lengths[0] == 0
    grown.prefill(kk[:1], v[:1], [2048, 0])
    assert grown.pool.n_free == free_before
    assert torch.equal(grown.decode(q), want)
    paged.check_status(grown.status)


def test_generate_loop_append_equals_prefill():
    """append() (one token per sequence, destinations taken from the lengths on the device) gives the
    cache that a single prefill gives, and decode after every step matches the oracle."""
    H = 2
    keys, comps, tables = _tables(H)
    g = torch.Generator().manual_seed(6)
    n0, steps = 90, 40
    v = torch.randn(2, H, n0 + steps, 128, generator=g).to(torch.bfloat16).cuda()
    kk = torch.stack([keys[:, : n0 + steps], keys.flip(1)[:, : n0 + steps]]).cuda()
    cache = paged.PagedKVCache(tables, n_seqs=2)
    cache.prefill(kk[:, :, :n0], v[:, :, :n0])
    for t in range(n0, n0 + steps):
        cache.append(kk[:, :, t:t + 1], v[:, :, t:t + 1])
    whole = paged.PagedKVCache(tables, [n0 + steps] * 2)
    whole.prefill(kk, v)
    q = torch.randn(2, 8, 128, generator=g).to(torch.bfloat16).cuda()
    out = cache.decode(q)
    assert cache.lengths == [n0 + steps] * 2 and cache.seq_lens.tolist() == [n0 + steps] * 2
    assert torch.equal(out, whole.decode(q))
    packed = paged.PackedKeys(tables, cache.k_pool, cache.page_table, cache.seq_lens, cache.lengths, cache.status)
    codes = paged.unpack_codes(packed).cpu()
    for s in range(2):
        k_hat = torch.stack([recon_from_codes(comps[h], codes[s, h]) for h in range(H)]).unsqueeze(0)
        ref = orc.decode_attention(q[s:s + 1].cpu(), k_hat, v[s:s + 1].cpu())[0]
        assert ((out[s].cpu() - ref).abs() / ref.abs().amax(-1, keepdim=True)).max().item() < 2e-3
    paged.check_status(cache.status)


def test_generate_step_graph_equals_append_then_decode():
    """generate_step in its graph form (append + attend as one replayed graph, recaptured when the context crosses the
    split boundary its grid covers or the pool moves) returns what append() followed by decode()
    returns, step after step."""
    H = 2
    keys, comps, tables = _tables(H)
    g = torch.Generator().manual_seed(12)
    n0, steps = 370, 60                                                     # crosses the 384-key split boundary
    v = torch.randn(2, H, n0 + steps, 128, generator=g).to(torch.bfloat16).cuda()
    kk = torch.stack([keys[:, : n0 + steps], keys.flip(1)[:, : n0 + steps]]).cuda()
    qs = torch.randn(steps, 2, 8, 128, generator=g).to(torch.bfloat16).cuda()
    a = paged.PagedKVCache(tables, n_seqs=2, initial_pages=4)
    b = paged.PagedKVCache(tables, n_seqs=2)
    a.prefill(kk[:, :, :n0], v[:, :, :n0])
    b.prefill(kk[:, :, :n0], v[:, :, :n0])
    captures = set()
    for i, t in enumerate(range(n0, n0 + steps)):
        got = a.generate_step(kk[:, :, t:t + 1], v[:, :, t:t + 1], qs[i], fused_append=False).clone()
        captures.add(id(a._gen_step["graph"]))
        b.append(kk[:, :, t:t + 1], v[:, :, t:t + 1])
        want = b.decode(qs[i])
        assert (got - want).abs().max().item() <= 1e-4 * want.abs().max().item(), f"step {i}"   # the splits may differ
    assert a.lengths == b.lengths == [n0 + steps] * 2 and a.seq_lens.tolist() == b.seq_lens.tolist()
    assert 2 <= len(captures) <= 6                                           # recaptured, but not every step
    paged.check_status(a.status)


@pytest.mark.parametrize("dtype,hq", [(torch.bfloat16, 8), (torch.float32, 8), (torch.bfloat16, 16)])
def test_fused_append_step_equals_the_separate_launches_bit_for_bit(dtype, hq):
    """jqk_decode_append_attend (one launch: append, attend, advance the lengths) against the
    graph of compress + store + length + decode launches on ragged sequences that cross page and
    split boundaries: the same output bits every step, the same codes and value rows in the pages,
    the same lengths; and the codes are the oracle's codes of the appended keys.  16 query heads over
    2 kv heads make two query blocks per head: both keep a copy of the new row, one writes it."""
    H = 2
    keys, comps, tables = _tables(H)
    g = torch.Generator().manual_seed(21)
    n0, steps = [370, 29, 1], 70
    total = max(n0) + steps
    v = torch.randn(3, H, total, 128, generator=g).to(torch.bfloat16).cuda()
    kk = torch.stack([keys[:, :total], keys.flip(1)[:, :total], keys[:, 100:100 + total]]).cuda()
    qs = torch.randn(steps, 3, hq, 128, generator=g).to(torch.bfloat16).cuda()
    caches = [paged.PagedKVCache(tables, [n + steps for n in n0]) for _ in range(2)]
    for c in caches:
        c.prefill(kk[:, :, :max(n0)], v[:, :, :max(n0)], lengths=n0)
    new_k = torch.stack([torch.stack([kk[s, :, n0[s] + i] for s in range(3)]) for i in range(steps)]).to(dtype)   # (steps, 3, H, d)
    new_v = torch.stack([torch.stack([v[s, :, n0[s] + i] for s in range(3)]) for i in range(steps)]).to(dtype)
    for i in range(steps):
        got = caches[0].generate_step(new_k[i].unsqueeze(2), new_v[i].unsqueeze(2), qs[i]).clone()
        want = caches[1].generate_step(new_k[i].unsqueeze(2), new_v[i].unsqueeze(2), qs[i], fused_append=False).clone()
        assert torch.equal(got, want), f"step {i}: {(got - want).abs().max().item()}"
    a, b = caches
    assert a._gen_step["fused"] and not b._gen_step["fused"]
    assert a.lengths == b.lengths == [n + steps for n in n0]
    assert a.seq_lens.tolist() == b.seq_lens.tolist() == a.lengths
    for c in caches:
        paged.check_status(c.status)
    for s in range(3):
        pk = [paged.PackedKeys(c.tables, c.k_pool, c.page_table[s:s + 1], c.seq_lens[s:s + 1], [c.lengths[s]], c.status)
              for c in caches]
        ca, cb = paged.unpack_codes(pk[0]), paged.unpack_codes(pk[1])
        assert torch.equal(ca, cb)
        assert torch.equal(_v_reference(a.v_pool, a.page_table, s, a.lengths, H, 128),
                           _v_reference(b.v_pool, b.page_table, s, b.lengths, H, 128))
        # the appended keys against the oracle's codes (fp32 transform, first-minimum ties)
        rows = new_k[:, s].float().cpu().to(torch.bfloat16 if dtype == torch.bfloat16 else torch.float32).float()   # (steps, H, d)
        for h in range(H):
            want_codes = orc.nearest_codes(orc.transform(rows[:, h], comps[h].forward_map), comps[h].codebooks_padded)
            got_codes = ca[0, h, n0[s]:, :].cpu()
            assert (got_codes.long() != want_codes.long()).float().mean().item() <= 1e-4


def test_fused_append_on_a_grid_of_several_waves():
    """The append launch when the grid exceeds one wave of blocks (tables from the table kernel,
    blocks that start after others have finished): ragged sequences, 180 blocks, three steps in a
    row on one workspace.  Lengths advance once per launch, the appended rows land in the pages, the
    outputs equal a plain decode over the grown cache."""
    H, n_seqs, tps = 2, 3, 384
    keys, comps, tables = _tables(H)
    g = torch.Generator().manual_seed(31)
    n0 = [384 * 30 - 2, 5000, 17]
    total = max(n0) + 8
    reps = -(-total // keys.shape[1])
    kk = torch.stack([keys.repeat(1, reps, 1)[:, :total].roll(7 * s, 1) for s in range(n_seqs)]).cuda()
    v = torch.randn(n_seqs, H, total, 128, generator=g).to(torch.bfloat16).cuda()
    fused = paged.PagedKVCache(tables, [n + 8 for n in n0])
    plain = paged.PagedKVCache(tables, [n + 8 for n in n0])
    for c in (fused, plain):
        c.prefill(kk[:, :, :max(n0)], v[:, :, :max(n0)], lengths=n0)
    covered = 384 * 30 + 384
    assert -(-covered // tps) * H * n_seqs > 148
    ws = paged.DecodeWorkspace(n_seqs, 8, H, -(-covered // tps), "cuda")
    out = torch.empty(n_seqs, 8, 128, device="cuda")
    for i in range(3):
        q = torch.randn(n_seqs, 8, 128, generator=g).to(torch.bfloat16).cuda()
        k_new = torch.stack([kk[s, :, n0[s] + i] for s in range(n_seqs)])
        v_new = torch.stack([v[s, :, n0[s] + i] for s in range(n_seqs)])
        for s in range(n_seqs):
            fused.reserve(s, n0[s] + i + 1)
        got = paged.decode_append_attend(tables, q, k_new, v_new, fused.seq_lens, covered, fused.page_table, fused.k_pool,
                                         fused.v_pool, out, ws, fused.status, tps).clone()
        for s in range(n_seqs):
            fused.lengths[s] += 1
        assert fused.seq_lens.tolist() == fused.lengths
        plain.append(k_new.unsqueeze(2), v_new.unsqueeze(2))
        want = plain.decode(q, tokens_per_split=tps)
        assert torch.equal(got, want), f"step {i}: {(got - want).abs().max().item()}"
    paged.check_status(fused.status)
    for s in range(n_seqs):
        pk = [paged.PackedKeys(c.tables, c.k_pool, c.page_table[s:s + 1], c.seq_lens[s:s + 1], [c.lengths[s]], c.status)
              for c in (fused, plain)]
        assert torch.equal(paged.unpack_codes(pk[0]), paged.unpack_codes(pk[1]))
        assert torch.equal(_v_reference(fused.v_pool, fused.page_table, s, fused.lengths, H, 128),
                           _v_reference(plain.v_pool, plain.page_table, s, plain.lengths, H, 128))


def test_overlong_length_is_clamped_flagged_and_leaves_the_workspace_clean():
    """A seq_lens entry above the max_seq_len the call was sized for: the kernel cuts the context to
    what its grid covers, sets JQK_STATUS_BAD_LENGTH, still merges, and the next call on the same
    workspace is intact.  Every page the clamped context touches is valid; nothing faults."""
    H = 2
    keys, comps, tables = _tables(H)
    g = torch.Generator().manual_seed(8)
    v = torch.randn(1, H, 2048, 128, generator=g).to(torch.bfloat16).cuda()
    q = torch.randn(1, 8, 128, generator=g).to(torch.bfloat16).cuda()
    cache = paged.PagedKVCache(tables, [2048])
    cache.prefill(keys.unsqueeze(0).cuda(), v)
    ws = paged.DecodeWorkspace(1, 8, H, 4, "cuda")
    out = torch.empty(1, 8, 128, device="cuda")
    good = paged.decode_attend(tables, q, cache.seq_lens, 1024, cache.page_table, cache.k_pool, cache.v_pool,
                               torch.empty_like(out), ws, cache.status, 256).clone()          # lengths say 2048!
    torch.cuda.synchronize()
    assert int(cache.status.item()) == _native.STATUS_BAD_LENGTH
    with pytest.raises(RuntimeError, match="sized for"):
        paged.check_status(cache.status)
    # the clamped call attended over the first 1024 keys: same as an honest call on a 1024-key context
    short = torch.tensor([1024], dtype=torch.int32, device="cuda")
    cache.status.zero_()
    ref = paged.decode_attend(tables, q, short, 1024, cache.page_table, cache.k_pool, cache.v_pool,
                              torch.empty_like(out), ws, cache.status, 256)
    assert torch.equal(good, ref)
    assert int(cache.status.item()) == 0
    # a token range past the page-table row is flagged by the page lookup, and skipped
    narrow = torch.zeros(1, 64, dtype=torch.int32, device="cuda")          # a row of 64 pages = 1024 tokens
    narrow.copy_(cache.page_table[:, :64])
    packed = paged.PackedKeys(tables, cache.k_pool, narrow, cache.seq_lens, [2048], cache.status)
    paged.unpack_codes(packed)
    torch.cuda.synchronize()
    assert int(cache.status.item()) == _native.STATUS_BAD_LENGTH


def test_bounded_wait_gives_up_sets_status_and_returns():
    """The wait every kernel uses, on a barrier nothing completes, with a 1 ms limit: the kernel
    returns, the status word carries JQK_STATUS_WAIT_EXPIRED, and the context keeps working."""
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    _native.check(_native.lib.jqk_selftest_bounded_wait(1000, status.data_ptr(), torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert int(status.item()) == _native.STATUS_WAIT_EXPIRED
    with pytest.raises(RuntimeError, match="wait expired"):
        paged.check_status(status)
    assert float((torch.ones(8, device="cuda") * 2).sum()) == 16.0       # the device still answers
    assert _native.lib.jqk_selftest_bounded_wait(0, status.data_ptr(), None) == -1


def test_captured_decode_graph_survives_a_workspace_reallocation():
    H = 2
    keys, comps, tables = _tables(H)
    g = torch.Generator().manual_seed(10)
    v = torch.randn(1, H, 2048, 128, generator=g).to(torch.bfloat16).cuda()
    cache = paged.PagedKVCache(tables, [2048])
    cache.prefill(keys.unsqueeze(0).cuda(), v)
    q = torch.randn(1, 8, 128, generator=g).to(torch.bfloat16)
    first = cache.decode_host(q, 1024).clone()                           # graph captured with a 2-split workspace
    first_call = cache.decode_host(q, 1024, use_graph=False).clone()
    ws_before = cache._ws
    cache.decode(q.cuda(), tokens_per_split=32)                          # needs 64 splits: the workspace is replaced
    assert cache._ws is not ws_before
    junk = [torch.full((1 << 20,), float("nan"), device="cuda") for _ in range(8)]   # reuse whatever was freed
    assert torch.equal(cache.decode_host(q, 1024), first)
    assert torch.equal(cache.decode_host(q, 1024, use_graph=False), first_call)
    del junk
    paged.check_status(cache.status)
