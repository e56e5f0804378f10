"""Data-parallel host logic on CPU ranks (gloo, world size 2): row sharding, the gradient
all-reduce convention (per-rank gradients of the GLOBAL-mean loss, summed), timing reduction, and
a rank that fails on the host before the collective (the others get an error, not a hang)."""

import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, mode, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    from difflut_b200.distributed import allreduce_sum_, init_from_env, max_over_ranks, shard_rows
    from oracle import difflut_oracle as O

    torch.set_num_threads(1)
    r, w, _ = init_from_env(backend="gloo", timeout_s=20.0)
    assert (r, w) == (rank, world)
    if mode == "fail" and rank == 1:
        raise SystemExit(3)  # leaves before the collective, on the host
    g = torch.Generator().manual_seed(0)
    B, I, k, tau = 50, 24, 5, 2.0
    bits = (torch.rand(B, I, generator=g) > 0.5).float()
    labels = torch.randint(0, k, (B,), generator=g)
    maps = [O.random_mapping(I, 20, 6, 0), O.random_mapping(20, 10, 6, 1)]
    tabs = [torch.randn(20, 1, 64, generator=g), torch.randn(10, 1, 64, generator=g)]
    alpha, beta = 0.5 * 0.75 ** 5, 0.25 / 0.75

    def table_grads(rows, labs, denom):
        logits, acts = O.dwn_network_forward(rows, maps, tabs, k, tau)
        lg = logits.clone().requires_grad_(True)
        loss = torch.nn.functional.cross_entropy(lg, labs, reduction="sum") / denom
        loss.backward()
        gr = O.dwn_network_backward(acts, maps, tabs, lg.grad, k, tau, alpha, beta)
        return torch.cat([x.reshape(-1) for x in gr]), loss.detach()

    lo, hi = shard_rows(B, rank, world)
    flat, loss = table_grads(bits[lo:hi], labels[lo:hi], B)  # local rows, global denominator
    if mode == "fail":
        try:
            allreduce_sum_(flat)
        except Exception:
            raise SystemExit(7)  # expected: the peer is gone
        raise SystemExit(0)
    allreduce_sum_(flat)
    loss_t = loss.clone().reshape(1)
    allreduce_sum_(loss_t)
    full, full_loss = table_grads(bits, labels, B)
    torch.testing.assert_close(flat, full, rtol=1e-5, atol=1e-7)
    torch.testing.assert_close(loss_t[0], full_loss, rtol=1e-6, atol=1e-7)
    assert max_over_ranks(float(rank + 1)) == float(world)
    dist.barrier()
    with open(os.path.join(out_dir, f"ok{rank}"), "w") as f:
        f.write("ok")


def test_shard_rows_partitions_exactly():
    from difflut_b200.distributed import shard_rows

    for total, world in ((8192, 8), (10, 3), (5, 8), (1, 1)):
        spans = [shard_rows(total, r, world) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == total
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        sizes = [b - a for a, b in spans]
        assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_rows(10, 3, 3)


def test_two_rank_gradient_allreduce_matches_full_batch(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, "ok", str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()


def test_rank_leaving_on_the_host_ends_the_collective_with_an_error(tmp_path):
    port = _free_port()
    ctx = mp.spawn(_worker, args=(2, port, "fail", str(tmp_path)), nprocs=2, join=False)
    for p in ctx.processes:
        p.join(timeout=90)
    codes = sorted(p.exitcode for p in ctx.processes)
    assert all(c is not None for c in codes), "a rank is still waiting: the collective hung"
    assert codes == [3, 7], codes
