"""The allocation-free decode entry point, called through the C ABI.

``jqk_decode_attend_static`` serves hosts that cannot allocate device memory on the decode path
(an engine whose pool already owns the whole GPU, a plugin inside someone else's memory budget):
its split-key scratch is an array built into the library.  The result must equal what
``jqk_decode_attend`` produces with a caller-owned workspace, on two calls in a row (the second
call finds the scratch as the first one left it), and an oversized request must be refused with
a clear error rather than overrun the array.  This file sorts last on purpose so that a run that
stops at the first failure has already executed every other test.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(n_seqs, lens, hq, hkv, seed):
    import jointqk_b200 as jq
    from jointqk_b200 import paged
    from jointqk_b200.synthetic import config_seed, fit_sigma_k_heads, spectrum_keys

    N = max(lens)
    keys = torch.stack([spectrum_keys(N, config_seed(1, 7, h)) for h in range(hkv)])
    comps, _ = fit_sigma_k_heads(keys, 2.0)
    tables = jq.HeadTables.from_compressors(comps, device="cuda")
    g = torch.Generator().manual_seed(seed)
    v = torch.randn(n_seqs, hkv, N, 128, generator=g).to(torch.bfloat16).cuda()
    q = torch.randn(n_seqs, hq, 128, generator=g).to(torch.bfloat16).cuda()
    cache = paged.PagedKVCache(tables, lens)
    cache.prefill(torch.stack([keys.roll(3 * s, 1) for s in range(n_seqs)]).cuda(), v, lens)
    return tables, cache, q


def _call_static(tables, cache, q, lens, tps, out):
    from jointqk_b200 import _native

    return _native.lib.jqk_decode_attend_static(
        tables.ref, q.data_ptr(), q.shape[0], q.shape[1], cache.seq_lens.data_ptr(), max(lens), tps,
        cache.page_table.data_ptr(), cache.page_table.stride(0), cache.n_pages, cache.k_pool.data_ptr(),
        cache.v_pool.data_ptr(), out.data_ptr(), _native.torch_dtype_code(out.dtype), cache.status.data_ptr(),
        torch.cuda.current_stream().cuda_stream)


def test_static_scratch_decode_matches_workspace_decode_twice():
    from jointqk_b200 import _native, paged

    lens = [3000, 777]
    tables, cache, q = _case(2, lens, 8, 2, seed=11)
    ref = cache.decode(q, tokens_per_split=256)                   # caller-owned workspace, 12 splits
    warm = torch.empty_like(ref)
    _native.check(_call_static(tables, cache, q, lens, 256, warm))   # first call on the device: address look-up
    outs = [torch.full_like(ref, float("nan")) for _ in range(2)]    # torch allocates before the measurement
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for out in outs:                                                  # two calls in a row through the C ABI
        _native.check(_call_static(tables, cache, q, lens, 256, out))
    torch.cuda.synchronize()
    # the entry point took nothing from the device: the driver reports the same free memory
    assert torch.cuda.mem_get_info()[0] == free_before
    paged.check_status(cache.status)
    for call, out in enumerate(outs):
        # same kernel, same split sizes, same merge order: the results are identical
        assert torch.equal(out, ref), f"call {call}: max diff {(out - ref).abs().max().item():.3e}"
    # a different query through the same scratch right after
    q2 = q.flip(1).contiguous()
    ref2 = cache.decode(q2, tokens_per_split=512)
    out2 = torch.empty_like(ref2)
    _native.check(_call_static(tables, cache, q2, lens, 512, out2))
    assert torch.allclose(out2, ref2, rtol=0, atol=0)
    # a single split per sequence still keeps its lookup tables in the scratch
    out3 = torch.empty_like(ref2)
    _native.check(_call_static(tables, cache, q2, lens, 4096, out3))
    assert torch.allclose(out3, cache.decode(q2, tokens_per_split=4096), rtol=1e-6, atol=1e-6)


def test_static_scratch_rejects_oversized_requests():
    from jointqk_b200 import _native

    lens = [3000, 777]
    tables, cache, q = _case(2, lens, 8, 2, seed=12)
    out = torch.empty(q.shape, dtype=torch.float32, device="cuda")
    limit = 8 * 1024 * 1024
    # pretend the context is huge: the size check runs on the host before anything is launched
    big = 40_000_000
    need = _native.lib.jqk_decode_workspace_bytes(2, 8, 2, -(-big // 32))
    assert need > limit
    rc = _native.lib.jqk_decode_attend_static(
        tables.ref, q.data_ptr(), 2, 8, cache.seq_lens.data_ptr(), big, 32, cache.page_table.data_ptr(),
        cache.page_table.stride(0), cache.n_pages, cache.k_pool.data_ptr(), cache.v_pool.data_ptr(),
        out.data_ptr(), 0, cache.status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == -4
    msg = _native.lib.jqk_last_error().decode()
    assert "built-in array" in msg and str(limit) in msg
