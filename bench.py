#!/usr/bin/env python
"""Benchmark of the compress-then-attend key path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline (one JSON line on stdout): compressed-K decode tokens/s on the single-layer decode
config -- GQA 32 q / 8 kv heads, head_dim 128, batch 1 per GPU, context 32768, keys packed at
2.0 bits/coordinate in 16-token pages, bf16 V -- with the HBM roofline of the decode kernel,
the same metric end to end from host buffers (``e2e``), and the reference algorithm's torch
CPU path timed on this box (``cpu_baseline``).  ``extra`` carries decode at batch and the other two stages of the
path on their named shapes: prefill compression (keys/s) and calibration moments
(token-layers/s), each with its own roofline fraction.

With N > 1 (torchrun, one rank per GPU) every rank serves its own sequence of the same shape
(the path shards by sequence with no collective on decode); the time is the max over ranks.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

CTX = 32768
N_Q_HEADS, N_KV_HEADS, HEAD_DIM = 32, 8, 128
B_AVG = 2.0
L2_BYTES = 126 * 2 ** 20
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0


def measured_peaks() -> tuple[float, float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        j = json.loads(p.read_text())
        return float(j["hbm_gbs"]), float(j.get("bf16_tflops_sustained", j.get("bf16_tflops", FALLBACK_BF16_TFLOPS))), "measured"
    return FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, "fallback"


# ----------------------------------------------------------------------------------------------
# clocks sampling through NVML (read-only)
# ----------------------------------------------------------------------------------------------
class ClockSampler:
    REASONS = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
               0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}

    def __init__(self, index: int) -> None:
        self.samples: list[tuple[float, int, int]] = []
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = index
            if visible:
                ids = [x for x in visible.split(",") if x.strip() != ""]
                if index < len(ids) and ids[index].strip().isdigit():
                    phys = int(ids[index])
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nv = None

    def _run(self) -> None:
        nv = self._nv
        while not self._stop.is_set():
            try:
                mhz = int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                rs = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)) if hasattr(
                    nv, "nvmlDeviceGetCurrentClocksEventReasons") else int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h))
                self.samples.append((time.perf_counter(), mhz, rs))
            except Exception:
                pass
            time.sleep(0.002)

    def start(self) -> None:
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(1.0)

    def summary(self, t0: float, t1: float) -> dict:
        inside = [s for s in self.samples if t0 <= s[0] <= t1] or self.samples[-5:]
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        mhz = sorted(s[1] for s in inside)
        bits = 0
        for s in inside:
            bits |= s[2]
        reasons = [n for b, n in self.REASONS.items() if bits & b and n != "gpu_idle"]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": self.max_mhz, "reasons": reasons, "samples": len(inside)}


# ----------------------------------------------------------------------------------------------
# workload: decode, one layer, context 32768, 2.0 bits
# ----------------------------------------------------------------------------------------------
def build_decode_workload(device, rank: int, n_copies: int):
    """Fit the 8 heads on a 4096-key sample of the config's key distribution, compress the full
    context through the product's own prefill path and build ``n_copies`` distinct caches so
    that consecutive steps never find their pages in L2."""
    import jointqk_b200 as jq
    from jointqk_b200 import paged
    from jointqk_b200.synthetic import config_seed, fit_sigma_k_heads, spectrum_keys

    keys = torch.stack([spectrum_keys(CTX, config_seed(1, 0, h) + 100 * rank, device=device) for h in range(N_KV_HEADS)])
    comps, _ = fit_sigma_k_heads(keys[:, :4096].cpu(), B_AVG)
    tables = jq.HeadTables.from_compressors(comps, device=device)
    gen = torch.Generator(device=device)
    gen.manual_seed(config_seed(1, 0, 0) + 7 + rank)
    caches = []
    for c in range(n_copies):
        cache = paged.PagedKVCache(tables, [CTX])
        v = torch.randn(1, N_KV_HEADS, CTX, HEAD_DIM, generator=gen, device=device).to(torch.bfloat16)
        cache.prefill(keys.roll(c * 17, 1).unsqueeze(0), v)
        caches.append(cache)
    q = torch.randn(1, N_Q_HEADS, HEAD_DIM, generator=gen, device=device).to(torch.bfloat16)
    paged.check_status(caches[0].status)
    return tables, comps, caches, q, keys


def decode_algorithmic_bytes(tables) -> dict:
    k_bytes = CTX * N_KV_HEADS * tables.payload_bytes_per_key
    v_bytes = CTX * N_KV_HEADS * HEAD_DIM * 2
    basis = N_KV_HEADS * HEAD_DIM * HEAD_DIM * 4
    small = N_KV_HEADS * 128 * 16 * 4 + N_Q_HEADS * HEAD_DIM * (2 + 4)
    return {"k_codes": k_bytes, "v": v_bytes, "basis": basis, "tables_q_out": small,
            "total": k_bytes + v_bytes + basis + small}


def timed_loop(fn, steps: int, warmup: int, device, world: int):
    """W untimed steps, barrier + synchronize, K steps between two CUDA events on the current
    stream, synchronize + barrier; returns (max-over-ranks ms, host t0, host t1)."""
    import torch.distributed as dist

    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize(device)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for i in range(steps):
        fn(warmup + i)
    e1.record()
    torch.cuda.synchronize(device)
    t1 = time.perf_counter()
    ms = e0.elapsed_time(e1)
    if world > 1:
        dist.barrier()
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms, t0, t1


def prewarm(fn, device, seconds: float = 0.25) -> None:
    """Untimed spin-up so that the SM clock has left idle before the W warm-up steps."""
    end = time.perf_counter() + seconds
    i = 0
    while time.perf_counter() < end:
        for _ in range(50):
            fn(i)
            i += 1
        torch.cuda.synchronize(device)


# ----------------------------------------------------------------------------------------------
# CPU side: the reference algorithm's torch path for one decode step (oracle port)
# ----------------------------------------------------------------------------------------------
def cpu_decode_setup(comps, keys_cpu: torch.Tensor, ctx: int):
    """Reconstructed keys (the reference keeps dequantised floats in its cache), V and q on the host."""
    from oracle import reference_port as orc

    k_hat = torch.stack([orc.roundtrip(keys_cpu[h, :ctx], comps[h].codebooks_padded, comps[h].forward_map,
                                       comps[h].inverse_map)[0] for h in range(N_KV_HEADS)]).unsqueeze(0)
    g = torch.Generator().manual_seed(99)
    v = torch.randn(1, N_KV_HEADS, ctx, HEAD_DIM, generator=g).to(torch.bfloat16)
    q = torch.randn(1, N_Q_HEADS, HEAD_DIM, generator=g).to(torch.bfloat16)
    return k_hat, v, q


def cpu_decode_steps_per_s(comps, keys_cpu, budget_s: float, steps: int | None = None, warmup: int = 1):
    """Times ``orc.decode_attention`` (fp32 matmul / softmax / @V on reconstructed keys).  A step is
    the full context when it fits the time budget, otherwise a leading slice of the context whose
    time is scaled linearly to the full context (the work is linear in context length)."""
    from oracle import reference_port as orc

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    ctx = CTX
    k_hat, v, q = cpu_decode_setup(comps, keys_cpu, ctx)
    t = time.perf_counter()
    orc.decode_attention(q, k_hat, v)
    t_full = time.perf_counter() - t
    n = steps if steps is not None else max(3, min(200, int(budget_s / max(t_full, 1e-6))))
    if (n + warmup) * t_full > budget_s:
        ctx = max(1024, int(CTX * budget_s / ((n + warmup) * t_full)) // 16 * 16)
        k_hat, v = k_hat[:, :, :ctx].contiguous(), v[:, :, :ctx].contiguous()
    for _ in range(warmup):
        orc.decode_attention(q, k_hat, v)
    t = time.perf_counter()
    for _ in range(n):
        orc.decode_attention(q, k_hat, v)
    dt = (time.perf_counter() - t) / n
    per_full_step = dt * (CTX / ctx)
    sample = f"{n} decode steps over {ctx} of {CTX} context keys, 32 q / 8 kv heads, fp32 matmul+softmax+@V on reconstructed keys"
    if ctx != CTX:
        sample += ", time scaled linearly to the full context"
    return 1.0 / per_full_step, per_full_step * 1e3, cores, sample


def cpu_stage_baselines() -> dict:
    """The reference's torch CPU path for the two secondary stages on bounded samples of their bench
    shapes, all host threads (about five seconds each): the per-head ``roundtrip`` loop on 8 heads x
    16384 bf16 keys at 2.5 bits, and the moment sums of 32 q / 8 kv heads x 8192 bf16 tokens."""
    from jointqk_b200.synthetic import config_seed, correlated_qk, fit_sigma_k_heads, spectrum_keys
    from oracle import reference_port as orc

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    out = {}
    T = 16384
    keys = torch.stack([spectrum_keys(T, config_seed(4, 0, h), 8, 20.0, dtype=torch.bfloat16) for h in range(N_KV_HEADS)])
    comps, _ = fit_sigma_k_heads(keys[:, :4096].float(), 2.5)
    run = lambda: [orc.roundtrip(keys[h], comps[h].codebooks_padded, comps[h].forward_map, comps[h].inverse_map)
                   for h in range(N_KV_HEADS)]
    run()
    t = time.perf_counter()
    reps = 0
    while reps < 3 or (time.perf_counter() - t < 4.0 and reps < 50):
        run()
        reps += 1
    dt = (time.perf_counter() - t) / reps
    out["prefill_compress"] = {"value": N_KV_HEADS * T / dt, "unit": "keys compressed/s", "cores": cores, "kind": "port",
                               "sample": f"{reps} passes of the per-head roundtrip (transform, argmin, gather, inverse) over 8 heads x {T} bf16 keys, 2.5 bits/coord"}
    T = 8192
    q, k = correlated_qk(T, N_Q_HEADS, N_KV_HEADS, config_seed(3, 0, 0))
    q, k = q.unsqueeze(0), k.unsqueeze(0)
    orc.moment_sums(q, k)
    t = time.perf_counter()
    reps = 0
    while reps < 3 or (time.perf_counter() - t < 4.0 and reps < 50):
        orc.moment_sums(q, k)
        reps += 1
    dt = (time.perf_counter() - t) / reps
    out["calibration_moments"] = {"value": T / dt, "unit": "calibration token-layers/s", "cores": cores, "kind": "port",
                                  "sample": f"{reps} passes of the three fp32 einsum sums over 32 q / 8 kv heads x {T} bf16 tokens"}
    return out


class _HostFit:
    """What the CPU legs need of a fitted head: codebooks and the two maps (plain tensors)."""

    def __init__(self, codebooks_padded, forward_map, inverse_map):
        self.codebooks_padded, self.forward_map, self.inverse_map = codebooks_padded, forward_map, inverse_map


def host_fit_sigma_k(keys: torch.Tensor, b_avg: float, max_bits: int = 4, eps: float = 1e-4) -> list[_HostFit]:
    """The parity config's fit (Sigma_K eigenbasis, water-fill on its variances, capped tail, Lloyd-Max
    codebooks) from the host-side modules alone.  The reference arm uses this so that it never loads
    the CUDA library."""
    from jointqk_b200.allocation import allocate_bits_for_budget
    from jointqk_b200.basis import eigvec_desc
    from jointqk_b200.codebooks import unit_gaussian_centroids
    from jointqk_b200.synthetic import second_moment
    from oracle import reference_port as orc

    unit = {b: unit_gaussian_centroids(b) for b in range(1, max_bits + 1)}
    out = []
    for h in range(keys.shape[0]):
        sig = second_moment(keys[h].float())
        R = eigvec_desc(sig, eps).float()
        var = (R.T @ sig @ R).diagonal().clamp_min(1e-30)
        bits = allocate_bits_for_budget(var.unsqueeze(0), float(b_avg) * keys.shape[-1], max_bits).squeeze(0)
        out.append(_HostFit(orc.codebooks_padded(bits, var.sqrt(), unit), R, R.T.contiguous()))
    return out


def run_reference_arm(args, rank: int, world: int) -> None:
    """The reference's CPU implementation of the path on this box's host cores (rank 0 only).  Nothing
    here imports a module that binds the CUDA library."""
    if rank != 0:
        return
    from jointqk_b200.synthetic import config_seed, spectrum_keys

    keys = torch.stack([spectrum_keys(CTX, config_seed(1, 0, h)) for h in range(N_KV_HEADS)])
    comps = host_fit_sigma_k(keys[:, :4096], B_AVG)
    value, ms, cores, sample = cpu_decode_steps_per_s(comps, keys, budget_s=150.0, steps=args.steps, warmup=args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


METRIC = "compressed-K decode tokens/s"
UNIT = "tokens/s (one decode step of one layer per sequence)"


def workload_config(n_gpus: int) -> dict:
    return {
        "workload": "decode, 1 layer, Llama-3.1-8B attention shape: 32 q / 8 kv heads, head_dim 128, "
                    "batch 1 per GPU, context 32768, K packed at 2.0 bits/coord in 16-token pages, V bf16",
        "context": CTX, "n_q_heads": N_Q_HEADS, "n_kv_heads": N_KV_HEADS, "head_dim": HEAD_DIM, "bits_per_coord": B_AVG,
        "sequences": n_gpus, "sharding": "by sequence, one per GPU, no collective",
        "l2_policy": "inputs rotate over 8 distinct caches (608 MB > 126 MB L2), so every step reads HBM",
    }


# ----------------------------------------------------------------------------------------------
# secondary stages on their named shapes (reported under "extra")
# ----------------------------------------------------------------------------------------------
def bench_compress(device, hbm_gbs: float, peak_kind: str) -> dict:
    """Prefill compression, one layer of the Qwen3-8B-shaped config: 4 sequences x 8 kv heads x 131072
    bf16 keys (1.07 GB in, > L2), 2.5 bits/coord, 8 outlier channels x20."""
    import jointqk_b200 as jq
    from jointqk_b200 import paged
    from jointqk_b200.synthetic import config_seed, fit_sigma_k_heads, spectrum_keys

    T, B = 131072, 4
    keys = torch.stack([torch.stack([spectrum_keys(T, config_seed(4, b, h), 8, 20.0, device=device, dtype=torch.bfloat16)
                                     for h in range(N_KV_HEADS)]) for b in range(B)])
    comps, _ = fit_sigma_k_heads(keys[0, :, :4096].float().cpu(), 2.5)
    tables = jq.HeadTables.from_compressors(comps, device=device)
    page_table, used = paged.sequential_page_table([T] * B, device)
    k_pool = paged.alloc_k_pool(tables, used)
    n_tok = torch.tensor([T] * B, dtype=torch.int32, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    run = lambda: paged.compress_into(tables, keys, n_tok, T, page_table, k_pool, status)
    for _ in range(3):
        run()
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 10
    e0.record()
    for _ in range(reps):
        run()
    e1.record()
    torch.cuda.synchronize(device)
    ms = e0.elapsed_time(e1) / reps
    n_keys = T * N_KV_HEADS * B
    bytes_per_key = HEAD_DIM * 2 + tables.payload_bytes_per_key
    gbs = n_keys * bytes_per_key / (ms * 1e-3) / 1e9
    res = {"metric": "keys compressed/s", "value": n_keys / (ms * 1e-3), "ms_per_launch": ms,
           "workload": "1 layer x 4 sequences x 8 kv heads x 131072 bf16 keys, 2.5 bits/coord, 16-token pages",
           "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm_gbs, "unit": "GB/s", "frac": gbs / hbm_gbs,
                        "bytes_per_key": bytes_per_key, "peak_kind": peak_kind}}
    # the same keys at the reference's default cap of 8 bits (outlier coordinates: a byte each)
    del k_pool
    comps8, _ = fit_sigma_k_heads(keys[0, :, :4096].float().cpu(), 2.5, max_bits=8)
    tables8 = jq.HeadTables.from_compressors(comps8, device=device)
    k_pool8 = paged.alloc_k_pool(tables8, used)
    run8 = lambda: paged.compress_into(tables8, keys, n_tok, T, page_table, k_pool8, status)
    for _ in range(3):
        run8()
    torch.cuda.synchronize(device)
    e0.record()
    for _ in range(reps):
        run8()
    e1.record()
    torch.cuda.synchronize(device)
    ms8 = e0.elapsed_time(e1) / reps
    bpk8 = HEAD_DIM * 2 + tables8.payload_bytes_per_key
    res["reference_default_cap8"] = {"ms_per_launch": ms8, "value": n_keys / (ms8 * 1e-3), "byte_wide_columns": tables8.n_wide,
                                     "words_per_record": tables8.words_per_record, "bytes_per_key": bpk8,
                                     "frac": n_keys * bpk8 / (ms8 * 1e-3) / 1e9 / hbm_gbs}
    paged.check_status(status)
    return res


def bench_reference_cap8(device, hbm_gbs: float, peak_kind: str) -> dict:
    """The headline decode step, the generate step and the prompt's compression with the reference's
    own allocation: the same 2.0 bits per coordinate, its default cap of 8 bits instead of 4
    (per_coord_quantization.py:367), so the outlier coordinates carry byte-wide codes."""
    import jointqk_b200 as jq
    from jointqk_b200 import paged
    from jointqk_b200.synthetic import config_seed, fit_sigma_k_heads, spectrum_keys

    keys = torch.stack([spectrum_keys(CTX, config_seed(1, 0, h), device=device) for h in range(N_KV_HEADS)])
    comps, _ = fit_sigma_k_heads(keys[:, :4096].cpu(), B_AVG, max_bits=8)
    tables = jq.HeadTables.from_compressors(comps, device=device)
    gen = torch.Generator(device=device)
    gen.manual_seed(config_seed(1, 0, 0) + 7)
    n_copies = 4
    caches = []
    for c in range(n_copies):
        cache = paged.PagedKVCache(tables, [CTX])
        v = torch.randn(1, N_KV_HEADS, CTX, HEAD_DIM, generator=gen, device=device).to(torch.bfloat16)
        cache.prefill(keys.roll(c * 17, 1).unsqueeze(0), v)
        caches.append(cache)
    q = torch.randn(1, N_Q_HEADS, HEAD_DIM, generator=gen, device=device).to(torch.bfloat16)
    tps = paged.default_split(1, N_Q_HEADS, N_KV_HEADS, CTX)
    ws = paged.DecodeWorkspace(1, N_Q_HEADS, N_KV_HEADS, -(-CTX // tps), device)
    out = torch.empty((1, N_Q_HEADS, HEAD_DIM), dtype=torch.float32, device=device)

    def step(i: int) -> None:
        c = caches[i % n_copies]
        paged.decode_attend(tables, q, c.seq_lens, CTX, c.page_table, c.k_pool, c.v_pool, out, ws, c.status, tps)

    stream = torch.cuda.Stream(device)
    with torch.cuda.stream(stream):
        for i in range(n_copies):
            step(i)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(n_copies):
                step(i)
    prewarm(lambda _i: graph.replay(), device, 0.1)
    reps = 100
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize(device)
    ms = e0.elapsed_time(e1) / (reps * n_copies)
    paged.check_status(caches[0].status)
    alg = decode_algorithmic_bytes(tables)["total"]
    res = {"workload": "the headline decode step with the reference's default cap of 8 bits per coordinate "
                       "(%d byte-wide columns per head at most, %d words per record)" % (tables.n_wide, tables.words_per_record),
           "ms_per_step": ms, "value": 1.0 / (ms * 1e-3), "unit": UNIT,
           "roofline": {"bound": "hbm", "achieved": alg / (ms * 1e-3) / 1e9, "peak": hbm_gbs, "unit": "GB/s",
                        "frac": alg / (ms * 1e-3) / 1e9 / hbm_gbs, "peak_kind": peak_kind}}
    # the generate step (one launch: append, attend, advance)
    steps = 128
    new_k = torch.randn(1, N_KV_HEADS, steps + 8, HEAD_DIM, generator=gen, device=device)
    new_v = torch.randn(1, N_KV_HEADS, steps + 8, HEAD_DIM, generator=gen, device=device).to(torch.bfloat16)
    cache = caches[0]
    for t in range(8):
        cache.generate_step(new_k[:, :, t:t + 1], new_v[:, :, t:t + 1], q)
    torch.cuda.synchronize(device)
    e0.record()
    for t in range(8, 8 + steps):
        cache.generate_step(new_k[:, :, t:t + 1], new_v[:, :, t:t + 1], q)
    e1.record()
    torch.cuda.synchronize(device)
    res["generate_step_ms"] = e0.elapsed_time(e1) / steps
    paged.check_status(cache.status)
    return res


def bench_decode_batch(device, hbm_gbs: float, peak_kind: str) -> dict:
    """Decode at batch: one layer of one rank's share of the 64-sequence config (8 ragged sequences
    assigned by longest-processing-time, lengths U{4096..65536}), 32 q / 8 kv heads, at 3.0 and at
    2.0 bits per coordinate.  The pools hold random codes and values: the kernel's work does not
    depend on their content, and two caches alternate so that every step reads HBM."""
    import jointqk_b200 as jq
    from jointqk_b200 import paged
    from jointqk_b200.synthetic import config_seed, fit_sigma_k_heads, lpt_shards, spectrum_keys, uniform_lengths

    lens_all = uniform_lengths(64, 4096, 65536, config_seed(2, 0, 0))
    shard = [lens_all[i] for i in lpt_shards(lens_all, 8)[0]]
    gen = torch.Generator(device=device)
    gen.manual_seed(config_seed(2, 0, 0) + 1)
    q = torch.randn(len(shard), N_Q_HEADS, HEAD_DIM, generator=gen, device=device).to(torch.bfloat16)
    out = {"workload": "1 layer, 8 sequences of %d..%d keys (%d in total), 32 q / 8 kv heads, 16-token pages"
                       % (min(shard), max(shard), sum(shard)), "lengths": shard}
    for b_avg in (3.0, 2.0):
        keys = torch.stack([spectrum_keys(4096, config_seed(2, 0, h)) for h in range(N_KV_HEADS)])
        comps, _ = fit_sigma_k_heads(keys, b_avg)
        tables = jq.HeadTables.from_compressors(comps, device=device)
        caches = []
        for _ in range(2):
            cache = paged.PagedKVCache(tables, shard)
            cache.k_pool.random_(0, 2 ** 31 - 1, generator=gen)
            cache.v_pool.normal_(generator=gen)
            cache.lengths = list(shard)
            cache.seq_lens[:] = torch.tensor(shard, dtype=torch.int32, device=device)
            caches.append(cache)
        for c in caches:
            c.decode(q)
        torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 40
        e0.record()
        for i in range(reps):
            caches[i % 2].decode(q)
        e1.record()
        torch.cuda.synchronize(device)
        ms = e0.elapsed_time(e1) / reps
        paged.check_status(caches[0].status)
        nbytes = sum(shard) * N_KV_HEADS * (tables.record_bytes + HEAD_DIM * 2)
        gbs = nbytes / (ms * 1e-3) / 1e9
        out["%.1f bits" % b_avg] = {
            "ms_per_layer_step": ms, "tokens_per_split": paged.split_for_lengths(shard, N_Q_HEADS, N_KV_HEADS),
            "layer_steps_x_sequences_per_s": len(shard) / (ms * 1e-3),
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm_gbs, "unit": "GB/s", "frac": gbs / hbm_gbs,
                         "algorithmic_bytes_per_launch": nbytes, "peak_kind": peak_kind}}
        del caches
        torch.cuda.empty_cache()
    return out


def bench_moments(device, hbm_gbs: float, tflops: float, peak_kind: str) -> dict:
    """Calibration moments: one layer, 32 q / 8 kv heads, 131072 bf16 tokens per launch (1.3 GB in)."""
    from jointqk_b200.moments import KeyPathMoments
    from jointqk_b200.synthetic import config_seed, correlated_qk

    T = 131072
    q, k = correlated_qk(T, N_Q_HEADS, N_KV_HEADS, config_seed(3, 0, 0), device=device)

    def time_variant(**kw) -> float:
        acc = KeyPathMoments(1, N_Q_HEADS, N_KV_HEADS, HEAD_DIM, device, **kw)
        run = lambda _i: acc.update(0, q, k)
        for i in range(2):
            run(i)
        return region_ms(run, 5, device, 1) / 5

    ms = time_variant(first_moments=False)                 # the three second moments (the named config)
    ms_first = time_variant(first_moments=True)            # plus sum_q / sum_k from the same pass
    ms_chain512 = time_variant(first_moments=False, max_chain_tokens=512)   # 512-token accumulation chains
    bytes_per_tl = (N_Q_HEADS + N_KV_HEADS) * HEAD_DIM * 2
    flop_per_tl = (N_Q_HEADS + 2 * N_KV_HEADS) * 2 * HEAD_DIM * HEAD_DIM
    gbs = T * bytes_per_tl / (ms * 1e-3) / 1e9
    tf = T * flop_per_tl / (ms * 1e-3) / 1e12
    return {"metric": "calibration token-layers/s", "value": T / (ms * 1e-3), "ms_per_launch": ms,
            "ms_per_launch_with_first_moments": ms_first, "ms_per_launch_chains_of_512_tokens": ms_chain512,
            "workload": "1 layer, 32 q / 8 kv heads, 131072 bf16 tokens, head_dim 128",
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm_gbs, "unit": "GB/s", "frac": gbs / hbm_gbs,
                         "tensor_tflops": tf, "tensor_frac": tf / tflops, "peak_kind": peak_kind}}



# ----------------------------------------------------------------------------------------------
# the three partitioned workloads, run at every N (reported under "extra.scale")
# ----------------------------------------------------------------------------------------------
def region_ms(fn, reps: int, device, world: int) -> float:
    """barrier + synchronize, `reps` calls of fn between two CUDA events, synchronize + barrier;
    the max over ranks of the event time, in ms."""
    import torch.distributed as dist

    torch.cuda.synchronize(device)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(reps):
        fn(i)
    e1.record()
    torch.cuda.synchronize(device)
    ms = e0.elapsed_time(e1)
    if world > 1:
        dist.barrier()
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def scale_decode_batch64(device, rank: int, world: int, hbm_gbs: float, peak_kind: str) -> dict:
    """The 64-sequence decode config, strong scaling: 32 layer-steps over the rank's share of 64
    sequences (context U{4096..65536}, K at 3.0 bits, bf16 V), sequences dealt by longest-processing-
    time, no collective; two caches alternate between layer-steps so every launch reads HBM."""
    import jointqk_b200 as jq
    from jointqk_b200 import paged
    from jointqk_b200.synthetic import config_seed, fit_sigma_k_heads, lpt_shards, spectrum_keys, uniform_lengths

    n_layers, b_avg = 32, 3.0
    lens_all = uniform_lengths(64, 4096, 65536, config_seed(2, 0, 0))
    shards = lpt_shards(lens_all, world)
    shard = [lens_all[i] for i in shards[rank]]
    gen = torch.Generator(device=device)
    gen.manual_seed(config_seed(2, 0, 0) + 1 + rank)
    q = torch.randn(len(shard), N_Q_HEADS, HEAD_DIM, generator=gen, device=device).to(torch.bfloat16)
    keys = torch.stack([spectrum_keys(4096, config_seed(2, 0, h)) for h in range(N_KV_HEADS)])
    comps, _ = fit_sigma_k_heads(keys, b_avg)
    tables = jq.HeadTables.from_compressors(comps, device=device)
    caches = []
    for _ in range(2):
        cache = paged.PagedKVCache(tables, shard)
        cache.k_pool.random_(0, 2 ** 31 - 1, generator=gen)
        cache.v_pool.normal_(generator=gen)
        cache.lengths = list(shard)
        cache.seq_lens[:] = torch.tensor(shard, dtype=torch.int32, device=device)
        caches.append(cache)

    def step(_i: int) -> None:
        for layer in range(n_layers):
            caches[layer % 2].decode(q)

    step(0)
    reps = max(2, math.ceil(50.0 / (45.0 / world)))                     # >= 50 ms timed
    ms = region_ms(step, reps, device, world) / reps
    paged.check_status(caches[0].status)
    bytes_per_step = sum(lens_all) * N_KV_HEADS * (tables.record_bytes + HEAD_DIM * 2) * n_layers
    gbs = bytes_per_step / (ms * 1e-3) / 1e9
    loads = [sum(lens_all[i] for i in sh) for sh in shards]
    del caches
    torch.cuda.empty_cache()
    return {"workload": "decode, 32 layers, 64 sequences, context U{4096..65536} (%d keys), 3.0 bits K, bf16 V" % sum(lens_all),
            "sharding": "sequences by longest-processing-time over %d rank(s), no collective" % world, "scaling": "strong",
            "value": 64 / (ms * 1e-3), "unit": "tokens/s (one 32-layer decode step per sequence)", "ms_per_step": ms,
            "timed_steps": reps, "rank_imbalance": max(loads) / (sum(loads) / world),
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm_gbs * world, "unit": "GB/s",
                         "frac": gbs / (hbm_gbs * world), "peak_kind": peak_kind, "algorithmic_bytes_per_step": bytes_per_step}}


def scale_calibration(device, rank: int, world: int, hbm_gbs: float, tflops: float, peak_kind: str) -> dict:
    """The calibration config, strong scaling: 2 097 152 tokens x 32 layers of bf16 q (32 heads) / k (8
    heads), tokens split evenly over the ranks, streamed as 65536-token chunks from a pool of 8
    distinct chunks (5.4 GB, generation untimed), then one NCCL all-reduce of the [32][3][8][128][128]
    fp32 block (50.3 MB) plus first moments and counts.  Kernels and collective are timed apart.  A
    small separate case checks the sharded sums against a single-rank pass."""
    import torch.distributed as dist
    from jointqk_b200.moments import KeyPathMoments
    from jointqk_b200.synthetic import config_seed, correlated_qk

    n_layers, total, chunk = 32, 2097152, 65536
    per_rank = total // world
    n_chunks = per_rank // chunk
    pool = [correlated_qk(chunk, N_Q_HEADS, N_KV_HEADS, config_seed(3, 0, c) + 50 * rank, device=device) for c in range(8)]
    acc = KeyPathMoments(n_layers, N_Q_HEADS, N_KV_HEADS, HEAD_DIM, device, first_moments=False)

    def kernels(_i: int) -> None:
        for layer in range(n_layers):
            for c in range(n_chunks):
                q, k = pool[(layer + c) % 8]
                acc.update(layer, q, k)

    for layer in range(2):                                               # warm-up: a few chunks
        for c in range(4):
            acc.update(layer, *pool[c])
    acc.all_reduce()
    acc.sums.zero_()
    acc.firsts.zero_()
    acc.tokens.zero_()
    k_ms = region_ms(kernels, 1, device, world)
    c_ms = region_ms(lambda _i: acc.all_reduce(), 1, device, world)
    acc.finalize()
    # parity of the sharded path on a distinct small case: every rank a token slice, all-reduce, and
    # rank 0's own pass over all tokens
    T = 8192 * max(1, world)
    qs, ks = correlated_qk(T, N_Q_HEADS, N_KV_HEADS, config_seed(3, 1, 0), device=device)
    part = KeyPathMoments(1, N_Q_HEADS, N_KV_HEADS, HEAD_DIM, device, first_moments=False)
    lo, hi = rank * T // world, (rank + 1) * T // world
    part.update(0, qs[:, lo:hi], ks[:, lo:hi])
    part.all_reduce()
    whole = KeyPathMoments(1, N_Q_HEADS, N_KV_HEADS, HEAD_DIM, device, first_moments=False)
    whole.update(0, qs, ks)
    err = float((part.sums.double() - whole.sums.double()).norm() / whole.sums.double().norm())
    same_tokens = float(part.tokens[0]) == float(T)
    tl = total * n_layers
    bytes_tl = (N_Q_HEADS + N_KV_HEADS) * HEAD_DIM * 2
    flop_tl = (N_Q_HEADS + 2 * N_KV_HEADS) * 2 * HEAD_DIM * HEAD_DIM
    step_ms = k_ms + c_ms
    gbs, tf = tl * bytes_tl / (k_ms * 1e-3) / 1e9, tl * flop_tl / (k_ms * 1e-3) / 1e12
    payload = acc.sums.numel() * 4
    del pool
    torch.cuda.empty_cache()
    return {"workload": "calibration moments, 2097152 tokens x 32 layers, 32 q / 8 kv heads, bf16, 65536-token chunks from a pool of 8",
            "sharding": "tokens split evenly over %d rank(s), one all-reduce of the sums" % world, "scaling": "strong",
            "value": tl / (step_ms * 1e-3), "unit": "calibration token-layers/s", "ms_kernels": k_ms, "ms_allreduce": c_ms,
            "allreduce_share": c_ms / step_ms, "allreduce_bytes": payload,
            "allreduce_busbw_gbs": (payload * 2 * (world - 1) / world / (c_ms * 1e-3) / 1e9) if world > 1 else None,
            "sharded_vs_single_pass_rel_err": err, "sharded_token_count_ok": same_tokens,
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm_gbs * world, "unit": "GB/s", "frac": gbs / (hbm_gbs * world),
                         "tensor_tflops": tf, "tensor_frac": tf / (tflops * world), "peak_kind": peak_kind,
                         "note": "kernel time only; the all-reduce is reported beside it"}}


def scale_prefill_compress(device, rank: int, world: int, hbm_gbs: float, peak_kind: str) -> dict:
    """The prefill-compression config, strong scaling: 36 layers x (4 sequences x 8 kv heads) x 131072 bf16
    keys, 2.5 bits.  The 32 (sequence, head) units of a layer are dealt to the ranks by kv head (rank r
    takes the heads h with h % N == r, all four sequences), layers iterate locally, no collective."""
    import jointqk_b200 as jq
    from jointqk_b200 import paged
    from jointqk_b200.synthetic import config_seed, fit_sigma_k_heads, spectrum_keys

    T, B, n_layers = 131072, 4, 36
    if world > N_KV_HEADS:
        return {"skipped": "more ranks than kv heads"}
    heads = [h for h in range(N_KV_HEADS) if h % world == rank]
    keys = torch.stack([torch.stack([spectrum_keys(T, config_seed(4, b, h), 8, 20.0, device=device, dtype=torch.bfloat16)
                                     for h in heads]) for b in range(B)])
    comps, _ = fit_sigma_k_heads(keys[0, :, :4096].float().cpu(), 2.5)
    tables = jq.HeadTables.from_compressors(comps, device=device)
    page_table, used = paged.sequential_page_table([T] * B, device)
    k_pool = paged.alloc_k_pool(tables, used)
    n_tok = torch.tensor([T] * B, dtype=torch.int32, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)

    def step(_i: int) -> None:
        for _layer in range(n_layers):
            paged.compress_into(tables, keys, n_tok, T, page_table, k_pool, status)

    step(0)
    reps = max(2, math.ceil(50.0 / (17.0 / world)))
    ms = region_ms(step, reps, device, world) / reps
    paged.check_status(status)
    n_keys = T * N_KV_HEADS * B * n_layers
    bytes_per_key = HEAD_DIM * 2 + tables.payload_bytes_per_key
    gbs = n_keys * bytes_per_key / (ms * 1e-3) / 1e9
    del keys, k_pool
    torch.cuda.empty_cache()
    return {"workload": "prefill compression, 36 layers x 4 sequences x 8 kv heads x 131072 bf16 keys, 2.5 bits/coord",
            "sharding": "(sequence, kv head) units by head over %d rank(s): %d units per rank, no collective" % (world, len(heads) * B),
            "scaling": "strong", "value": n_keys / (ms * 1e-3), "unit": "keys compressed/s", "ms_per_step": ms, "timed_steps": reps,
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm_gbs * world, "unit": "GB/s", "frac": gbs / (hbm_gbs * world),
                         "bytes_per_key": bytes_per_key, "peak_kind": peak_kind}}


def bench_generate_loop(device, tables, cache, hbm_gbs: float) -> dict:
    """The decode step as a generate loop on the headline shape: every step appends one new token per
    sequence (compress it into the tail page, store its value, advance the length on the device) and
    then attends over the whole context.  Timed end to end over 256 steps, launches included."""
    from jointqk_b200 import paged

    steps, H = 256, N_KV_HEADS
    gen = torch.Generator(device=device)
    gen.manual_seed(4242)
    new_k = torch.randn(1, H, steps + 8, HEAD_DIM, generator=gen, device=device)
    new_v = torch.randn(1, H, steps + 8, HEAD_DIM, generator=gen, device=device).to(torch.bfloat16)
    q = torch.randn(1, N_Q_HEADS, HEAD_DIM, generator=gen, device=device).to(torch.bfloat16)
    for t in range(8):                                                   # warm-up (also reserves the next page)
        cache.append(new_k[:, :, t:t + 1], new_v[:, :, t:t + 1])
        cache.decode(q)
    torch.cuda.synchronize(device)
    t0 = time.perf_counter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for t in range(8, 8 + steps):
        cache.append(new_k[:, :, t:t + 1], new_v[:, :, t:t + 1])
        out = cache.decode(q)
    e1.record()
    torch.cuda.synchronize(device)
    wall = time.perf_counter() - t0
    ms = e0.elapsed_time(e1) / steps
    # the same step through PagedKVCache.generate_step: the four launches replayed as one CUDA graph
    # (inputs staged), then the single launch that appends, attends and advances the lengths itself
    def graph_loop(fused: bool):
        more_k = torch.randn(1, H, steps + 8, HEAD_DIM, generator=gen, device=device)
        more_v = torch.randn(1, H, steps + 8, HEAD_DIM, generator=gen, device=device).to(torch.bfloat16)
        for t in range(8):
            cache.generate_step(more_k[:, :, t:t + 1], more_v[:, :, t:t + 1], q, fused_append=fused)
        torch.cuda.synchronize(device)
        t0 = time.perf_counter()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for t in range(8, 8 + steps):
            cache.generate_step(more_k[:, :, t:t + 1], more_v[:, :, t:t + 1], q, fused_append=fused)
        e1.record()
        torch.cuda.synchronize(device)
        return e0.elapsed_time(e1) / steps, (time.perf_counter() - t0) / steps * 1e3

    ms_g4, wall_g4 = graph_loop(False)
    ms_g, wall_g = graph_loop(True)
    # the fused launch called directly, rows read in place (no staging copies, no graph): what a model
    # whose projection kernels write k, v and q into fixed buffers pays per layer and step
    n_direct = steps
    rows_k = torch.randn(n_direct + 8, 1, H, HEAD_DIM, generator=gen, device=device).to(torch.bfloat16)
    rows_v = torch.randn(n_direct + 8, 1, H, HEAD_DIM, generator=gen, device=device).to(torch.bfloat16)
    cache.reserve(0, cache.lengths[0] + n_direct + 8)
    covered = cache.lengths[0] + n_direct + 8
    tps = paged.split_for_lengths([covered], N_Q_HEADS, H)
    ws = paged.DecodeWorkspace(1, N_Q_HEADS, H, -(-covered // tps), device)
    out = torch.empty(1, N_Q_HEADS, HEAD_DIM, device=device)

    def direct(i):
        paged.decode_append_attend(tables, q, rows_k[i], rows_v[i], cache.seq_lens, covered, cache.page_table,
                                   cache.k_pool, cache.v_pool, out, ws, cache.status, tps)

    for i in range(8):
        direct(i)
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(8, 8 + n_direct):
        direct(i)
    e1.record()
    torch.cuda.synchronize(device)
    ms_d = e0.elapsed_time(e1) / n_direct
    cache.lengths[0] += n_direct + 8
    assert cache.seq_lens[0].item() == cache.lengths[0]
    paged.check_status(cache.status)
    return {"workload": "generate loop on the headline shape: append 1 token (K compress + V store + length), then decode, context %d -> %d"
                        % (cache.lengths[0] - 4 * steps - 32, cache.lengths[0]),
            "value": 1.0 / (ms_g * 1e-3), "unit": UNIT, "ms_per_step": ms_g, "wall_ms_per_step": wall_g,
            "how": "PagedKVCache.generate_step: one launch per step (jqk_decode_append_attend appends the row, attends and advances the lengths), rows read in place",
            "fused_launch_direct": {"ms_per_step": ms_d, "launches_per_step": 1,
                                    "note": "back-to-back jqk_decode_append_attend launches reading the new rows in place, no graph"},
            "graph_of_four_launches": {"ms_per_step": ms_g4, "wall_ms_per_step": wall_g4},
            "separate_launches": {"ms_per_step": ms, "wall_ms_per_step": wall / steps * 1e3, "launches_per_step": 4},
            "steps": steps}


def bench_isolated_launch(step, device, alg_bytes: float, hbm_gbs: float) -> dict:
    """One decode step at a time: launch, wait for it, launch the next.  Nothing of the next step can
    overlap the tail of this one, unlike the back-to-back replay of the headline; both are real uses
    (a step that waits for its result, a pipeline of independent steps)."""
    times = []
    for i in range(40):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(device)
        e0.record()
        step(i)
        e1.record()
        torch.cuda.synchronize(device)
        times.append(e0.elapsed_time(e1))
    times = sorted(times[8:])
    ms = times[len(times) // 2]
    return {"ms_per_step": ms, "frac_of_hbm": alg_bytes / (ms * 1e-3) / 1e9 / hbm_gbs,
            "note": "median of 32 single launches, each synchronised before and after (event overhead of ~2 us included)"}


def bench_decode_packed_values(device, hbm_gbs: float, peak_kind: str) -> dict:
    """The headline decode shape with the values stored as packed codes too: K at 2.0 bits, V at 3.0
    bits (eigenbasis of Cov[V], water-fill, mean-centred), 80 bytes per key and head instead of 288.
    The pools hold random codes (the kernel's work does not depend on their content); 8 caches rotate."""
    import jointqk_b200 as jq
    from jointqk_b200 import paged
    from jointqk_b200.synthetic import config_seed, fit_sigma_k_heads, second_moment, spectrum_keys

    keys = torch.stack([spectrum_keys(4096, config_seed(1, 0, h)) for h in range(N_KV_HEADS)])
    comps, _ = fit_sigma_k_heads(keys, B_AVG)
    tables = jq.HeadTables.from_compressors(comps, device=device)
    vals = torch.stack([spectrum_keys(4096, config_seed(1, 1, h), n_outliers=0) for h in range(N_KV_HEADS)]) + 0.1
    v_comps = []
    for h in range(N_KV_HEADS):
        mu = vals[h].double().mean(0).float()
        v_comps.append(jq.build_v_compressor("v_eigen_waterfill", cov_v_for_head=second_moment(vals[h]) - torch.outer(mu, mu),
                                             head_dim=HEAD_DIM, bits=3, mu_v_for_head=mu, max_bits=4))
    v_tables = jq.HeadTables.from_compressors([c.inner for c in v_comps], device=device, center=torch.stack([c.mu for c in v_comps]))
    gen = torch.Generator(device=device)
    gen.manual_seed(5)
    q = torch.randn(1, N_Q_HEADS, HEAD_DIM, generator=gen, device=device).to(torch.bfloat16)
    caches = []
    for _ in range(8):
        c = paged.PagedKVCache(tables, [CTX], v_tables=v_tables)
        c.k_pool.random_(0, 2 ** 31 - 1, generator=gen)
        c.v_pool.random_(0, 2 ** 31 - 1, generator=gen)
        c.lengths = [CTX]
        c.seq_lens[:] = CTX
        caches.append(c)
    run = lambda i: caches[i % 8].decode(q)
    for i in range(16):
        run(i)
    ms = region_ms(run, 200, device, 1) / 200
    paged.check_status(caches[0].status)
    nbytes = CTX * N_KV_HEADS * (tables.payload_bytes_per_key + v_tables.payload_bytes_per_key) + 2 * N_KV_HEADS * HEAD_DIM * HEAD_DIM * 4
    gbs = nbytes / (ms * 1e-3) / 1e9
    return {"workload": "decode, 1 layer, 32 q / 8 kv heads, context 32768, K 2.0 bits and V 3.0 bits packed (80 B per key and head)",
            "value": 1.0 / (ms * 1e-3), "unit": UNIT, "ms_per_step": ms, "cache_bytes_per_step": nbytes,
            "cache_bytes_vs_bf16_values": nbytes / (CTX * N_KV_HEADS * (tables.payload_bytes_per_key + 2 * HEAD_DIM)),
            "roofline": {"bound": "shared memory (dequantisation), not hbm", "achieved": gbs, "peak": hbm_gbs, "unit": "GB/s",
                         "frac": gbs / hbm_gbs, "peak_kind": peak_kind}}


def bench_value_store(device, hbm_gbs: float, peak_kind: str) -> dict:
    """Values of one layer of the prefill config into pages: 4 sequences x 8 kv heads x 131072 bf16 rows,
    one pass of the store kernel (256 B read + 256 B written per row)."""
    import jointqk_b200 as jq
    from jointqk_b200 import paged
    from jointqk_b200.synthetic import config_seed, fit_sigma_k_heads, spectrum_keys

    T, B = 131072, 4
    keys = torch.stack([spectrum_keys(4096, config_seed(4, 0, h)) for h in range(N_KV_HEADS)])
    comps, _ = fit_sigma_k_heads(keys, 2.5)
    tables = jq.HeadTables.from_compressors(comps, device=device)
    gen = torch.Generator(device=device)
    gen.manual_seed(7)
    v = torch.randn(B, N_KV_HEADS, T, HEAD_DIM, generator=gen, device=device).to(torch.bfloat16)
    page_table, used = paged.sequential_page_table([T] * B, device)
    v_pool = paged.alloc_v_pool(tables, used)
    n_tok = torch.tensor([T] * B, dtype=torch.int32, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    run = lambda _i: paged.store_values_into(v, n_tok, T, page_table, v_pool, status)
    for i in range(3):
        run(i)
    ms = region_ms(run, 10, device, 1) / 10
    rows = T * N_KV_HEADS * B
    gbs = rows * 512 / (ms * 1e-3) / 1e9
    return {"metric": "value rows stored/s", "value": rows / (ms * 1e-3), "ms_per_launch": ms,
            "workload": "1 layer x 4 sequences x 8 kv heads x 131072 bf16 value rows into 16-token pages",
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm_gbs, "unit": "GB/s", "frac": gbs / hbm_gbs,
                         "bytes_per_row": 512, "peak_kind": peak_kind}}


def run_scale_blocks(device, rank: int, world: int) -> dict:
    hbm_gbs, tflops, peak_kind = measured_peaks()
    out = {}
    for name, fn in (("decode_batch64", lambda: scale_decode_batch64(device, rank, world, hbm_gbs, peak_kind)),
                     ("calibration", lambda: scale_calibration(device, rank, world, hbm_gbs, tflops, peak_kind)),
                     ("prefill_compress", lambda: scale_prefill_compress(device, rank, world, hbm_gbs, peak_kind))):
        out[name] = fn()
    return out

# ----------------------------------------------------------------------------------------------
# main arm
# ----------------------------------------------------------------------------------------------
# dram__bytes_read.sum + dram__bytes_write.sum of one decode_kernel launch of the headline workload,
# from one ncu capture of that launch (76.20 MB + 1.20 MB, mean of the two captured launches)
DECODE_DRAM_TRAFFIC_BYTES = 77.40e6


def run_ours(args, rank: int, local_rank: int, world: int) -> None:
    import torch.distributed as dist
    from jointqk_b200 import paged

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product path has no CPU implementation")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    hbm_gbs, tflops, peak_kind = measured_peaks()
    n_copies = 8
    tables, comps, caches, q, keys = build_decode_workload(device, rank, n_copies)
    tps = args.tokens_per_split or paged.default_split(1, N_Q_HEADS, N_KV_HEADS, CTX)
    max_splits = -(-CTX // tps)
    ws = paged.DecodeWorkspace(1, N_Q_HEADS, N_KV_HEADS, max_splits, device)
    out = torch.empty((1, N_Q_HEADS, HEAD_DIM), dtype=torch.float32, device=device)

    def step(i: int) -> None:
        c = caches[i % n_copies]
        paged.decode_attend(tables, q, c.seq_lens, CTX, c.page_table, c.k_pool, c.v_pool, out, ws, c.status, tps)

    # Launch-bound loop: capture n_copies consecutive steps in a CUDA graph and replay it.
    stream = torch.cuda.Stream(device)
    with torch.cuda.stream(stream):
        for i in range(n_copies):
            step(i)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(n_copies):
                step(i)
    torch.cuda.synchronize(device)
    full, rest = divmod(args.steps, n_copies)

    def replay(_i: int) -> None:
        if args.no_graph:
            for i in range(n_copies):
                step(i)
        else:
            graph.replay()

    sampler = ClockSampler(local_rank)
    sampler.start()
    prewarm(replay, device, 0.05 if args.no_graph else 0.25)
    # W warm-up steps and exactly K timed steps (graph replays of 8 steps plus single launches)
    def run_steps(n: int, base: int) -> None:
        f, r = divmod(n, n_copies)
        for _ in range(f):
            replay(0)
        for i in range(r):
            step(base + i)

    run_steps(args.warmup, 0)
    # R repeats of the K-step region, each bracketed by barrier + synchronize and timed with CUDA events
    # (max over ranks); the reported step time is the median region.  One region of K steps is short
    # (K x ~20 us), so a single one would mostly measure jitter.
    region_list = []
    t0 = time.perf_counter()
    for _rep in range(max(1, args.repeats)):
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        run_steps(args.steps, 0)
        e1.record()
        torch.cuda.synchronize(device)
        r_ms = e0.elapsed_time(e1)
        if world > 1:
            dist.barrier()
            t = torch.tensor([r_ms], dtype=torch.float64, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            r_ms = float(t.item())
        region_list.append(r_ms)
    t1 = time.perf_counter()
    ordered = sorted(region_list)
    ms = ordered[len(ordered) // 2]
    sampler.stop()
    clocks = sampler.summary(t0, t1)
    paged.check_status(caches[0].status)

    # end to end through the public call with host buffers: PagedKVCache.decode_host stages the query
    # in pinned memory and replays a graph of {H2D copy, decode launch, D2H copy}, then waits for it
    q_host = q.cpu()
    e2e_steps = max(20, min(args.steps, 500))
    for c in caches:
        c.decode_host(q_host, tps)                               # capture outside the timed region
    e2e_out = [None]

    def e2e_step(i: int) -> None:
        e2e_out[0] = caches[i % n_copies].decode_host(q_host, tps)   # the next token depends on this result

    e2e_ms, _, _ = timed_loop(e2e_step, e2e_steps, max(3, args.warmup), device, world)
    # the same step with no copy commands: the kernel reads the query from page-locked host memory and
    # writes the result there itself (an option of decode_host; reported beside the default)
    for c in caches:
        c.decode_host(q_host, tps, zero_copy=True)
    e2e_zc_ms, _, _ = timed_loop(lambda i: caches[i % n_copies].decode_host(q_host, tps, zero_copy=True),
                                 e2e_steps, max(3, args.warmup), device, world)
    for c in caches:
        c.decode_host(q_host, tps, zero_copy="out")
    e2e_zo_ms, _, _ = timed_loop(lambda i: caches[i % n_copies].decode_host(q_host, tps, zero_copy="out"),
                                 e2e_steps, max(3, args.warmup), device, world)

    alg = decode_algorithmic_bytes(tables)
    per_launch_ms = ms / args.steps
    achieved = alg["total"] / (per_launch_ms * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": world * args.steps / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_launch_ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16 q/V, 0-4 bit K codes (fixed-point 16-bit lookup tables), fp32 accumulate",
        "data": "synthetic", "config": workload_config(world), "clocks": clocks,
        "e2e": {"value": world * e2e_steps / (e2e_ms * 1e-3), "unit": UNIT,
                "h2d_bytes_per_step": q_host.numel() * 2, "d2h_bytes_per_step": e2e_out[0].numel() * 4,
                "steps": e2e_steps, "value_zero_copy": world * e2e_steps / (e2e_zc_ms * 1e-3),
                "value_zero_copy_out": world * e2e_steps / (e2e_zo_ms * 1e-3),
                "note": "host query in, pinned-host result out through PagedKVCache.decode_host (replayed graph of H2D copy, decode, D2H copy; "
                        "stream wait per step); value_zero_copy: the same step as a one-kernel graph that reads the query from and writes the "
                        "result to page-locked host memory itself"},
        "gpu_launches": args.steps,
        "repeats": {"regions": len(region_list), "steps_per_region": args.steps, "ms_per_step_median": per_launch_ms,
                    "ms_per_step_min": ordered[0] / args.steps, "ms_per_step_max": ordered[-1] / args.steps},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_gbs, "unit": "GB/s", "frac": achieved / hbm_gbs,
                     "traffic": DECODE_DRAM_TRAFFIC_BYTES, "peak_kind": peak_kind, "kernel": "decode_kernel",
                     "algorithmic_bytes_per_launch": alg, "tokens_per_split": tps},
    }
    if not args.no_extra:
        extra = {}
        if world == 1:
            extra["isolated_launch"] = bench_isolated_launch(step, device, alg["total"], hbm_gbs)
            extra["generate_loop"] = bench_generate_loop(device, tables, caches[0], hbm_gbs)
        del caches[1:]
        torch.cuda.empty_cache()
        if world == 1:
            extra["prefill_compress"] = bench_compress(device, hbm_gbs, peak_kind)
            extra["prefill_values"] = bench_value_store(device, hbm_gbs, peak_kind)
            extra["calibration_moments"] = bench_moments(device, hbm_gbs, tflops, peak_kind)
            extra["decode_batch"] = bench_decode_batch(device, hbm_gbs, peak_kind)
            extra["decode_packed_values"] = bench_decode_packed_values(device, hbm_gbs, peak_kind)
            extra["reference_default_cap8"] = bench_reference_cap8(device, hbm_gbs, peak_kind)
        del caches[:]
        torch.cuda.empty_cache()
        # the partitioned workloads run at every N: sequences, tokens and (sequence, head) units over the ranks
        extra["scale"] = run_scale_blocks(device, rank, world)
        line["extra"] = extra
    if rank == 0:
        if world == 1 and not args.no_cpu:
            v, cms, cores, sample = cpu_decode_steps_per_s(comps, keys.cpu(), budget_s=20.0)
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample,
                                    "ms_per_step": cms}
            if "extra" in line:
                for stage, base in cpu_stage_baselines().items():
                    if stage in line["extra"]:
                        line["extra"][stage]["cpu_baseline"] = base
        print(json.dumps(line), flush=True)


def run_batch64(args, rank: int, local_rank: int, world: int) -> None:
    """Opt-in workload (``--workload batch64``): the 64-sequence decode config.  One step = 32 layer-steps
    over the rank's share of 64 sequences with context lengths U{4096..65536}, K packed at 3.0 bits,
    bf16 V.  Sequences are dealt to the ranks by longest-processing-time; there is no collective on the
    step.  Two caches alternate between layer-steps, so every launch reads HBM.  Strong scaling: the
    64 sequences are fixed, ``value`` = 64 sequences x steps / max-over-ranks time."""
    import jointqk_b200 as jq
    from jointqk_b200 import paged
    from jointqk_b200.synthetic import config_seed, fit_sigma_k_heads, lpt_shards, spectrum_keys, uniform_lengths

    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    hbm_gbs, _, peak_kind = measured_peaks()
    n_layers, b_avg = 32, 3.0
    lens_all = uniform_lengths(64, 4096, 65536, config_seed(2, 0, 0))
    shard = [lens_all[i] for i in lpt_shards(lens_all, world)[rank]]
    gen = torch.Generator(device=device)
    gen.manual_seed(config_seed(2, 0, 0) + 1 + rank)
    q = torch.randn(len(shard), N_Q_HEADS, HEAD_DIM, generator=gen, device=device).to(torch.bfloat16)
    keys = torch.stack([spectrum_keys(4096, config_seed(2, 0, h)) for h in range(N_KV_HEADS)])
    comps, _ = fit_sigma_k_heads(keys, b_avg)
    tables = jq.HeadTables.from_compressors(comps, device=device)
    caches = []
    for _ in range(2):
        cache = paged.PagedKVCache(tables, shard)
        cache.k_pool.random_(0, 2 ** 31 - 1, generator=gen)
        cache.v_pool.normal_(generator=gen)
        cache.lengths = list(shard)
        cache.seq_lens[:] = torch.tensor(shard, dtype=torch.int32, device=device)
        caches.append(cache)

    def step(_i: int) -> None:
        for layer in range(n_layers):
            caches[layer % 2].decode(q)

    steps, warmup = min(args.steps, 20), max(3, min(args.warmup, 5))
    sampler = ClockSampler(local_rank)
    sampler.start()
    ms, t0, t1 = timed_loop(step, steps, warmup, device, world)
    sampler.stop()
    paged.check_status(caches[0].status)
    per_step_ms = ms / steps
    bytes_per_step = sum(lens_all) * N_KV_HEADS * (tables.record_bytes + HEAD_DIM * 2) * n_layers
    gbs = bytes_per_step / (per_step_ms * 1e-3) / 1e9
    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": 64 * steps / (ms * 1e-3), "unit": "tokens/s (one 32-layer decode step per sequence)",
            "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": per_step_ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16 q/V, 0-4 bit K codes (fixed-point 16-bit lookup tables), fp32 accumulate", "data": "synthetic",
            "config": {"workload": "decode, 32 layers, 64 sequences with context U{4096..65536} (%d keys in all), 32 q / 8 kv heads, "
                                   "head_dim 128, K packed at 3.0 bits/coord in 16-token pages, V bf16" % sum(lens_all),
                       "sharding": "by sequence, longest-processing-time over %d rank(s), no collective" % world,
                       "rank0_lengths": shard, "l2_policy": "two caches alternate between layer-steps"},
            "clocks": sampler.summary(t0, t1), "gpu_launches": steps * n_layers,
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm_gbs * world, "unit": "GB/s",
                         "frac": gbs / (hbm_gbs * world), "peak_kind": peak_kind, "kernel": "decode_kernel",
                         "algorithmic_bytes_per_step": bytes_per_step}}), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--repeats", type=int, default=10, help="timed regions of --steps steps each; the median is reported")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extra", action="store_true", help="skip the compress / moments stages")
    ap.add_argument("--no-cpu", action="store_true", help="skip the timed CPU baseline")
    ap.add_argument("--no-graph", action="store_true", help="launch every step directly instead of replaying a CUDA graph")
    ap.add_argument("--tokens-per-split", type=int, default=0, help="override the decode split size (0 = library default)")
    ap.add_argument("--workload", default="headline", choices=["headline", "batch64"],
                    help="headline: the single-layer context-32768 step (default, what the JSON contract names); "
                         "batch64: the 32-layer, 64-sequence decode config sharded by sequence over the ranks")
    ap.add_argument("--stage", default="all", choices=["all", "compress", "moments", "decode_batch", "values", "packed_values", "generate", "cap8", "scale"],
                    help="run only one of the secondary stages (or the three partitioned workloads) and print its JSON")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        if args.steps > 200:
            args.steps = 200
        run_reference_arm(args, rank, world)
        return
    if args.stage not in ("all", "scale"):
        dev = torch.device("cuda", local_rank)
        torch.cuda.set_device(dev)
        hbm, tf, kind = measured_peaks()
        if args.stage == "generate":
            tables, _comps, caches, _q, _keys = build_decode_workload(dev, 0, 1)
            print(json.dumps(bench_generate_loop(dev, tables, caches[0], hbm)), flush=True)
            return
        res = (bench_compress(dev, hbm, kind) if args.stage == "compress" else
               bench_decode_batch(dev, hbm, kind) if args.stage == "decode_batch" else
               bench_value_store(dev, hbm, kind) if args.stage == "values" else
               bench_decode_packed_values(dev, hbm, kind) if args.stage == "packed_values" else
               bench_reference_cap8(dev, hbm, kind) if args.stage == "cap8" else bench_moments(dev, hbm, tf, kind))
        print(json.dumps(res), flush=True)
        return
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        if args.stage == "scale":
            dev = torch.device("cuda", local_rank)
            torch.cuda.set_device(dev)
            res = run_scale_blocks(dev, rank, world)
            if rank == 0:
                print(json.dumps(res), flush=True)
        elif args.workload == "batch64":
            run_batch64(args, rank, local_rank, world)
        else:
            run_ours(args, rank, local_rank, world)
    finally:
        if world > 1:
            import torch.distributed as dist

            dist.destroy_process_group()


if __name__ == "__main__":
    main()
