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
    n = steps if steps is not None else max(3, min(50, int(budget_s / max(t_full, 1e-6))))
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


def run_reference_arm(args, rank: int, world: int) -> None:
    """The reference's CPU implementation of the path on this box's host cores (rank 0 only)."""
    if rank != 0:
        return
    from jointqk_b200.synthetic import config_seed, fit_sigma_k_heads, spectrum_keys

    keys = torch.stack([spectrum_keys(CTX, config_seed(1, 0, h)) for h in range(N_KV_HEADS)])
    comps, _ = fit_sigma_k_heads(keys[:, :4096], B_AVG)
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
    return {"metric": "keys compressed/s", "value": n_keys / (ms * 1e-3), "ms_per_launch": ms,
            "workload": "1 layer x 4 sequences x 8 kv heads x 131072 bf16 keys, 2.5 bits/coord, 16-token pages",
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm_gbs, "unit": "GB/s", "frac": gbs / hbm_gbs,
                         "bytes_per_key": bytes_per_key, "peak_kind": peak_kind}}


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
    acc = KeyPathMoments(1, N_Q_HEADS, N_KV_HEADS, HEAD_DIM, device)
    run = lambda: acc.update(0, q, k)
    for _ in range(2):
        run()
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 3
    e0.record()
    for _ in range(reps):
        run()
    e1.record()
    torch.cuda.synchronize(device)
    ms = e0.elapsed_time(e1) / reps
    bytes_per_tl = (N_Q_HEADS + N_KV_HEADS) * HEAD_DIM * 2
    flop_per_tl = (N_Q_HEADS + 2 * N_KV_HEADS) * 2 * HEAD_DIM * HEAD_DIM
    gbs = T * bytes_per_tl / (ms * 1e-3) / 1e9
    tf = T * flop_per_tl / (ms * 1e-3) / 1e12
    return {"metric": "calibration token-layers/s", "value": T / (ms * 1e-3), "ms_per_launch": ms,
            "workload": "1 layer, 32 q / 8 kv heads, 131072 bf16 tokens, head_dim 128",
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm_gbs, "unit": "GB/s", "frac": gbs / hbm_gbs,
                         "tensor_tflops": tf, "tensor_frac": tf / tflops, "peak_kind": peak_kind}}


# ----------------------------------------------------------------------------------------------
# main arm
# ----------------------------------------------------------------------------------------------
# dram__bytes_read.sum + dram__bytes_write.sum of one decode_kernel launch of the headline workload,
# from one ncu capture of that launch (76.20 MB + 1.38 MB)
DECODE_DRAM_TRAFFIC_BYTES = 77.58e6


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
    torch.cuda.synchronize(device)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    run_steps(args.steps, 0)
    e1.record()
    torch.cuda.synchronize(device)
    t1 = time.perf_counter()
    ms = e0.elapsed_time(e1)
    if world > 1:
        dist.barrier()
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
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

    alg = decode_algorithmic_bytes(tables)
    per_launch_ms = ms / args.steps
    achieved = alg["total"] / (per_launch_ms * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": world * args.steps / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_launch_ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16 q/V, 0-4 bit K codes, fp32 accumulate",
        "data": "synthetic", "config": workload_config(world), "clocks": clocks,
        "e2e": {"value": world * e2e_steps / (e2e_ms * 1e-3), "unit": UNIT,
                "h2d_bytes_per_step": q_host.numel() * 2, "d2h_bytes_per_step": e2e_out[0].numel() * 4,
                "steps": e2e_steps, "note": "host query in, pinned-host result out through PagedKVCache.decode_host (replayed graph of H2D copy, decode, D2H copy; stream wait per step)"},
        "gpu_launches": args.steps,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_gbs, "unit": "GB/s", "frac": achieved / hbm_gbs,
                     "traffic": DECODE_DRAM_TRAFFIC_BYTES, "peak_kind": peak_kind, "kernel": "decode_kernel",
                     "algorithmic_bytes_per_launch": alg, "tokens_per_split": tps},
    }
    if world == 1 and not args.no_extra:
        del caches[1:]
        torch.cuda.empty_cache()
        line["extra"] = {"prefill_compress": bench_compress(device, hbm_gbs, peak_kind),
                         "calibration_moments": bench_moments(device, hbm_gbs, tflops, peak_kind),
                         "decode_batch": bench_decode_batch(device, hbm_gbs, peak_kind)}
    if rank == 0:
        if world == 1 and not args.no_cpu:
            v, cms, cores, sample = cpu_decode_steps_per_s(comps, keys.cpu(), budget_s=20.0)
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample,
                                    "ms_per_step": cms}
            if "extra" in line:
                for stage, base in cpu_stage_baselines().items():
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
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16 q/V, 0-4 bit K codes, fp32 accumulate", "data": "synthetic",
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
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extra", action="store_true", help="skip the compress / moments stages")
    ap.add_argument("--no-cpu", action="store_true", help="skip the timed CPU baseline")
    ap.add_argument("--no-graph", action="store_true", help="launch every step directly instead of replaying a CUDA graph")
    ap.add_argument("--tokens-per-split", type=int, default=0, help="override the decode split size (0 = library default)")
    ap.add_argument("--workload", default="headline", choices=["headline", "batch64"],
                    help="headline: the single-layer context-32768 step (default, what the JSON contract names); "
                         "batch64: the 32-layer, 64-sequence decode config sharded by sequence over the ranks")
    ap.add_argument("--stage", default="all", choices=["all", "compress", "moments", "decode_batch"],
                    help="profiling aid: run only one of the secondary stages and print its JSON")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        if args.steps > 200:
            args.steps = 200
        run_reference_arm(args, rank, world)
        return
    if args.stage != "all":
        dev = torch.device("cuda", local_rank)
        torch.cuda.set_device(dev)
        hbm, tf, kind = measured_peaks()
        res = (bench_compress(dev, hbm, kind) if args.stage == "compress" else
               bench_decode_batch(dev, hbm, kind) if args.stage == "decode_batch" else bench_moments(dev, hbm, tf, kind))
        print(json.dumps(res), flush=True)
        return
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        if args.workload == "batch64":
            run_batch64(args, rank, local_rank, world)
        else:
            run_ours(args, rank, local_rank, world)
    finally:
        if world > 1:
            import torch.distributed as dist

            dist.destroy_process_group()


if __name__ == "__main__":
    main()
