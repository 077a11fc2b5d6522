"""Multi-rank host logic on CPU ranks (gloo, world_size 2): token-sharded moments reduce to the
single-rank result, and the sequence / head partitions cover the work exactly once."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from jointqk_b200.synthetic import correlated_qk, lpt_shards, uniform_lengths
from oracle import reference_port as orc


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from jointqk_b200.moments import KeyPathMoments

        q, k = correlated_qk(512, 4, 2, seed=77, dtype=torch.float32, d=32)
        acc = KeyPathMoments(1, 4, 2, 32, device="cpu")
        lo, hi = rank * 256, (rank + 1) * 256
        part = orc.moment_sums(q[None, :, lo:hi], k[None, :, lo:hi])     # this rank's token shard
        acc.sums[0, 0], acc.sums[0, 1], acc.sums[0, 2] = part["sq_sum"][0], part["sk_sum"][0], part["cqk_sum"][0]
        acc.firsts[0, 0] = q[:, lo:hi].reshape(2, 2, hi - lo, 32).sum((1, 2))
        acc.firsts[0, 1] = k[:, lo:hi].sum(1)
        acc.tokens[0] = hi - lo
        acc.all_reduce()
        fin = acc.finalize()
        full = orc.normalise_moments(orc.moment_sums(q[None], k[None]), group=2, tokens=512)
        ok = all(torch.allclose(fin[n][0], full[n][0], rtol=1e-5, atol=1e-5) for n in ("sigma_q", "sigma_k", "cqk"))
        ok = ok and float(fin["total_tokens"][0]) == 512.0
        ok = ok and torch.allclose(fin["mu_k"][0], k.mean(1), rtol=1e-5, atol=1e-6)
        ok = ok and torch.allclose(fin["mu_q"][0], q.reshape(2, 2, 512, 32).mean((1, 2)), rtol=1e-5, atol=1e-6)
        out[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_token_sharded_moments_allreduce():
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        out = mgr.dict()
        with socket.socket() as sock:                     # a port the kernel says is free right now
            sock.bind(("127.0.0.1", 0))
            port = sock.getsockname()[1]
        procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0
        assert dict(out) == {0: True, 1: True}


def test_moment_status_word_is_read_on_finalize():
    """An expired wait in the moment kernel reaches the caller: every finalize reads the status word."""
    from jointqk_b200 import _native, moments

    key = ("cpu", None)
    moments._STATUS[key] = torch.tensor([_native.STATUS_WAIT_EXPIRED], dtype=torch.int32)
    try:
        with pytest.raises(RuntimeError, match="wait expired"):
            moments.check_status()
        acc = moments.QueryMomentsAccumulator()
        acc.sum_q, acc.sum_outer, acc.total_count = torch.zeros(1, 1, 4), torch.zeros(1, 1, 4, 4), 3
        with pytest.raises(RuntimeError, match="wait expired"):
            acc.finalize()
        cross = moments.CrossMomentsAccumulator()
        cross.sum_qk, cross.total_count = torch.zeros(1, 4, 4), 3
        with pytest.raises(RuntimeError, match="wait expired"):
            cross.finalize()
    finally:
        del moments._STATUS[key]
    assert moments.check_status() is None


def test_lpt_partition_covers_everything_once():
    lens = uniform_lengths(64, 4096, 65536, seed=1)
    assert len(lens) == 64 and min(lens) >= 4096 and max(lens) <= 65536
    shards = lpt_shards(lens, 8)
    flat = sorted(i for s in shards for i in s)
    assert flat == list(range(64))
    loads = [sum(lens[i] for i in s) for s in shards]
    assert max(loads) <= 1.05 * (sum(lens) / 8)
    assert lpt_shards(lens, 1) == [sorted(range(64), key=lambda i: -lens[i])]
