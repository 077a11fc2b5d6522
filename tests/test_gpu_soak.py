"""Seeded sweeps over shapes that the hand-picked cases do not enumerate: ragged and empty
sequences, lengths on and around page (16), tile (32) and block (384) boundaries, group sizes that do
and do not fill a query block, head sizes 64 and 128, every bit budget, small and default splits.

* decode attention against fp32 attention over the reconstruction of the same codes (the decompress
  kernel has its own parity tests against the oracle), tolerance as in test_gpu_decode.py;
* the one-launch generate step against the graph of separate launches: same outputs, same codes in
  the pages, same lengths, for bf16 / fp16 / fp32 rows and pools that have to grow;
* the tensor-core compress kernel against the CUDA-core one over arbitrary allocations (widths drawn
  per coordinate, sorted, or in blocks of eight), which drives the read planner through every class
  and into its generic path: the two may only differ where a value sits on a decision threshold."""

import os
import random

import pytest
import torch

import jointqk_b200 as jq
from jointqk_b200 import paged
from jointqk_b200.layout import plan_key_layout
from jointqk_b200.synthetic import config_seed, fit_sigma_k_heads, spectrum_keys

pytestmark = pytest.mark.gpu

EDGE_LENGTHS = [0, 1, 15, 16, 17, 31, 33, 383, 384, 385]
# longer sweeps from other seeds: JQK_SOAK_SCALE=5 JQK_SOAK_SEED=100 python -m pytest tests/test_gpu_soak.py -m gpu
SCALE = int(os.environ.get("JQK_SOAK_SCALE", "1"))
SEED = int(os.environ.get("JQK_SOAK_SEED", "0"))
_TABLES = {}


def _tables(H, b, d=128, cap=4):
    """``cap`` 8: the reference's own cap; outlier coordinates then carry byte-wide codes."""
    key = (H, b, d, cap)
    if key not in _TABLES:
        keys = torch.stack([spectrum_keys(8192, config_seed(0, 5, h), d=d) for h in range(H)])
        comps, _ = fit_sigma_k_heads(keys[:, :4096], b, max_bits=cap)
        _TABLES[key] = (keys, jq.HeadTables.from_compressors(comps, device="cuda"))
    return _TABLES[key]


def test_decode_over_random_shapes():
    rng = random.Random(3 + SEED)
    worst = 0.0
    for it in range(60 * SCALE):
        d = rng.choice([128, 128, 128, 64])
        H, g = rng.choice([1, 2, 4, 8]), rng.choice([1, 2, 4, 5, 8])
        b = rng.choice([1.0, 2.0, 2.5, 3.0, 4.0])
        lens = [rng.choice(EDGE_LENGTHS + [rng.randint(2, 8000)]) for _ in range(rng.randint(1, 6))]
        tps = rng.choice([0, 0, 32, 128, 384, 1024])
        cap = rng.choice([4, 4, 8]) if d == 128 and b <= 3.0 else 4
        keys, tables = _tables(H, b, d, cap)
        N = max(max(lens), 1)
        gen = torch.Generator().manual_seed(it)
        kk = torch.stack([keys[:, :N].roll(3 * s, 1) for s in range(len(lens))]).cuda()
        v = torch.randn(len(lens), H, N, d, generator=gen).to(torch.bfloat16).cuda()
        q = torch.randn(len(lens), H * g, d, generator=gen).to(torch.bfloat16).cuda()
        cache = paged.PagedKVCache(tables, [max(n, 1) for n in lens])
        cache.prefill(kk, v, lens)
        out = cache.decode(q, tokens_per_split=tps)
        paged.check_status(cache.status)
        k_hat = paged.decompress(paged.PackedKeys(tables, cache.k_pool, cache.page_table, cache.seq_lens, list(lens), cache.status))
        for s, n in enumerate(lens):
            if n == 0:
                assert out[s].abs().max().item() == 0.0
                continue
            kh = k_hat[s, :, :n].repeat_interleave(g, 0)
            vv = v[s, :, :n].float().repeat_interleave(g, 0)
            w = (torch.einsum("hd,htd->ht", q[s].float(), kh) / d ** 0.5).softmax(-1)
            ref = torch.einsum("ht,htd->hd", w, vv)
            err = ((out[s] - ref).abs() / ref.abs().amax(-1, keepdim=True).clamp_min(1e-6)).max().item()
            worst = max(worst, err)
            assert err < 2e-3, (it, d, H, g, b, lens, tps, s, err)
    print(f"decode over {60 * SCALE} random shapes: worst relative error {worst:.2e}")


_V_TABLES = {}


def _v_tables(H, cap=4):
    """Value-side tables (eigenbasis of the covariance, 3 bits, mean-centred) for H heads."""
    if (H, cap) not in _V_TABLES:
        from jointqk_b200.synthetic import second_moment

        g = torch.Generator().manual_seed(40 + H)
        vals = torch.stack([spectrum_keys(4096, config_seed(0, 60, h), n_outliers=0 if cap == 4 else 2) for h in range(H)]) \
            + 0.3 * torch.randn(H, 1, 128, generator=g)
        comps = []
        for h in range(H):
            mu = vals[h].double().mean(0).float()
            comps.append(jq.build_v_compressor("v_eigen_waterfill", cov_v_for_head=second_moment(vals[h]) - torch.outer(mu, mu),
                                               head_dim=128, bits=3, seed=42 + h, mu_v_for_head=mu, max_bits=cap))
        _V_TABLES[(H, cap)] = jq.HeadTables.from_compressors([c.inner for c in comps], device="cuda",
                                                      center=torch.stack([c.mu for c in comps]))
    return _V_TABLES[(H, cap)]


@pytest.mark.parametrize("packed_values", [False, True])
def test_fused_generate_step_over_random_shapes(packed_values):
    rng = random.Random(7 + packed_values + SEED)
    for it in range((20 if packed_values else 40) * SCALE):
        H, g = rng.choice([1, 2, 4]), rng.choice([1, 2, 4, 8])
        b = rng.choice([1.0, 2.0, 2.5, 3.0, 4.0])
        n0 = [rng.choice(EDGE_LENGTHS + [rng.randint(2, 3000)]) for _ in range(rng.randint(1, 4))]
        steps = rng.randint(1, 40)
        dtype = rng.choice([torch.bfloat16, torch.float32, torch.float16])
        cap = rng.choice([4, 8]) if b <= 3.0 else 4
        keys, tables = _tables(H, b, cap=cap)
        total = max(n0) + steps
        gen = torch.Generator().manual_seed(it)
        kk = torch.stack([keys[:, :total].roll(3 * s, 1) for s in range(len(n0))]).cuda()
        v = torch.randn(len(n0), H, total, 128, generator=gen).to(torch.bfloat16).cuda()
        vt = _v_tables(H, cap) if packed_values else None
        fused = paged.PagedKVCache(tables, n_seqs=len(n0), initial_pages=rng.choice([1, 8, 64]), v_tables=vt)   # has to grow
        plain = paged.PagedKVCache(tables, n_seqs=len(n0), v_tables=vt)
        for cache in (fused, plain):
            if max(n0) > 0:
                cache.prefill(kk[:, :, :max(n0)], v[:, :, :max(n0)], lengths=n0)
        for i in range(steps):
            q = torch.randn(len(n0), H * g, 128, generator=gen).to(torch.bfloat16).cuda()
            kn = torch.stack([kk[s, :, n0[s] + i] for s in range(len(n0))]).to(dtype).unsqueeze(2)
            vn = torch.stack([v[s, :, n0[s] + i] for s in range(len(n0))]).to(dtype).unsqueeze(2)
            got = fused.generate_step(kn, vn, q).clone()
            want = plain.generate_step(kn, vn, q, fused_append=False)
            # the two caches may size their grids differently (pages reserved ahead), so the splits,
            # and with them the last bits of the merge, may differ
            assert (got - want).abs().max().item() <= 1e-4 * want.abs().max().item(), (it, i)
        assert fused.seq_lens.tolist() == fused.lengths == plain.lengths == [n + steps for n in n0]
        for s in range(len(n0)):
            for t, pool in ((tables, "k_pool"),) + (((vt, "v_pool"),) if packed_values else ()):
                pk = [paged.PackedKeys(t, getattr(c, pool), c.page_table[s:s + 1], c.seq_lens[s:s + 1], [c.lengths[s]], c.status)
                      for c in (fused, plain)]
                assert torch.equal(paged.unpack_codes(pk[0]), paged.unpack_codes(pk[1])), (it, s, pool)
        paged.check_status(fused.status)
        paged.check_status(plain.status)


def test_tensor_core_compress_over_random_allocations():
    rng = random.Random(5 + SEED)
    H, T = 2, 2048
    keys = torch.stack([spectrum_keys(T, config_seed(0, 2, h)) for h in range(H)]).to(torch.bfloat16)
    base, _ = fit_sigma_k_heads(keys.float(), 2.5)
    differ = total = wide_coords = wide_values = 0
    for it in range(60 * SCALE):
        comps = []
        wide_coords = 0
        for c in base:
            mode = rng.choice(["iid", "sorted", "blocks"])
            if mode == "iid":
                bits = torch.tensor(rng.choices([0, 1, 2, 3, 4], weights=[rng.random() for _ in range(5)], k=128))
            elif mode == "sorted":
                cuts = sorted(rng.randint(0, 128) for _ in range(4))
                bits = torch.tensor([4] * cuts[0] + [3] * (cuts[1] - cuts[0]) + [2] * (cuts[2] - cuts[1])
                                    + [1] * (cuts[3] - cuts[2]) + [0] * (128 - cuts[3]))
            else:
                bits = torch.tensor(sum([[rng.choice([0, 1, 2, 3, 4])] * 8 for _ in range(16)], []))
            if int(bits.sum()) == 0:
                bits[0] = 1
            if it % 3 == 2:      # some coordinates at 5..8 bits (a byte each); the record holds 16 words
                for j in rng.sample(range(128), rng.randint(1, 32)):
                    bits[j] = rng.randint(5, 8)
                while True:
                    try:
                        plan_key_layout(bits.numpy())
                        break
                    except ValueError:
                        nz = bits.nonzero().flatten().tolist()
                        bits[rng.choice(nz)] = 0
                wide_coords += int((bits > 4).sum())
            comps.append(jq.PerCoordCompressor(bits, c.stds, c.forward_map, c.inverse_map))
        tables = jq.HeadTables.from_compressors(comps, device="cuda")
        n = rng.choice([T, 1000, 129, 128, 17])
        on_tensor_cores = paged.compress(tables, keys[:, :n].unsqueeze(0).cuda())            # bf16 keys
        on_cuda_cores = paged.compress(tables, keys[:, :n].float().unsqueeze(0).cuda())      # the same values in fp32
        a, b = paged.unpack_codes(on_tensor_cores), paged.unpack_codes(on_cuda_cores)
        differ += int((a != b).sum())
        total += a.numel()
        wide_values += wide_coords * n
        assert (a.int() - b.int()).abs().max().item() <= 1, it          # a threshold tie moves a code by one level
        paged.check_status(on_tensor_cores.status)
    print(f"tensor-core vs CUDA-core codes over {60 * SCALE} allocations: {differ} of {total} differ")
    assert differ <= 1e-5 * total + 1e-4 * wide_values + 2     # 255 thresholds to sit on instead of 15
