"""world_size-2 gloo test of the multi-GPU host logic on CPU: (batch*head) shards are disjoint and
cover the batch, each rank's gradients are its slice of the full problem, and d(lambda) is the host
sum of the per-rank fp32 partials."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import diffattn_oracle as oracle


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from triton_diff_attn_b200 import shard_batch, sum_dlambda_on_host
    torch.set_num_threads(1)
    b, h, n, d = 4, 2, 64, 16
    q1, q2, k1, k2, v, dy = oracle.make_inputs(b, h, n, d, seed=99, dtype=torch.float32)
    lam = torch.tensor([0.5])
    lo, hi = shard_batch(b, h, rank, world)
    part = oracle.backward_closed_form(*(t[lo:hi] for t in (q1, q2, k1, k2, v)), lam, dy[lo:hi], 0.8, True)
    total = sum_dlambda_on_host(part["dlambda"].float())
    full = oracle.backward_closed_form(q1, q2, k1, k2, v, lam, dy, 0.8, True)
    ok = abs(total - float(full["dlambda"])) <= 1e-4 * max(1.0, abs(float(full["dlambda"])))
    ok = ok and torch.allclose(part["dq1"], full["dq1"][lo:hi], atol=1e-6)
    ok = ok and torch.allclose(part["dv"], full["dv"][lo:hi], atol=1e-6)
    q.put((rank, lo, hi, bool(ok)))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_sharding_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert [(r[1], r[2]) for r in res] == [(0, 2), (2, 4)]
    assert all(r[3] for r in res)


def test_shard_range_covers_everything():
    from triton_diff_attn_b200 import shard_range
    for total in (0, 1, 7, 64, 2048):
        for world in (1, 2, 3, 8):
            spans = [shard_range(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(8, 2, 2)
