"""The peer-memory optimiser step (gradient sum + Adam + parameter broadcast in one kernel per layer).

Two GPUs (skipped otherwise; the ranks are child processes): two ranks train a small DWN classifier for
three steps with it and, separately, with the NCCL all-reduce path and as ONE process on the whole batch;
tables must agree between the ranks bit for bit, and with the other two runs to fp32 rounding.

One GPU: the exchange kernel with a world of one rank must reproduce dl_adam_step bit for bit (slices,
channels, state advance), and with a peer whose flags nothing writes it must give up after the limit,
report the peer and leave parameters, moments and optimiser state untouched."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

WORKER = r"""
import os, sys, warnings
warnings.simplefilter("ignore")
import torch
import torch.distributed as dist
sys.path.insert(0, os.environ["DIFFLUT_ROOT"])
from difflut_b200.distributed import init_from_env, shard_rows
from difflut_b200.encoder import ThermometerEncoder
from difflut_b200.layers import RandomLayer
from difflut_b200.network import DWNNetwork
from difflut_b200.nodes import DWNNode, NodeConfig
from difflut_b200.utils import GroupSum

rank, world, local = init_from_env(timeout_s=60)
dev = torch.device("cuda", local)
gen = torch.Generator().manual_seed(0)
B, F, Tb, k = 600, 12, 3, 4
x = torch.rand(B, F, generator=gen)
y = torch.randint(0, k, (B,), generator=gen)
sizes = [70, 40, 20]
tabs = [torch.randn(N, 1, 64, generator=gen) for N in sizes]
lo, hi = shard_rows(B, rank, world)
results = {}
for peer in (True, False):
    enc = ThermometerEncoder(num_bits=Tb).fit(x)
    layers, I = [], F * Tb
    for li, N in enumerate(sizes):
        l = RandomLayer(I, N, DWNNode, NodeConfig(input_dim=6, output_dim=1), seed=li).to(dev)
        with torch.no_grad():
            l.luts.copy_(tabs[li].to(dev))
        layers.append(l)
        I = N
    net = DWNNetwork(enc, layers, GroupSum(k=k, tau=2.0, use_randperm=False), lr=1e-2, peer_optimizer=peer)
    assert net.peer_optimizer == peer
    for step in range(3):
        net.train_step(x[lo:hi].to(dev), y[lo:hi].to(dev), use_graph=(step > 0))
    torch.cuda.synchronize()
    assert net.peer_status() == 0
    results[peer] = torch.cat([t.reshape(-1) for t in net.tables]).clone()
# the same three steps in one process on the whole batch (no exchange at all)
enc = ThermometerEncoder(num_bits=Tb).fit(x)
layers, I = [], F * Tb
for li, N in enumerate(sizes):
    l = RandomLayer(I, N, DWNNode, NodeConfig(input_dim=6, output_dim=1), seed=li).to(dev)
    with torch.no_grad():
        l.luts.copy_(tabs[li].to(dev))
    layers.append(l)
    I = N
solo = DWNNetwork(enc, layers, GroupSum(k=k, tau=2.0, use_randperm=False), lr=1e-2, distributed=False)
for step in range(3):
    solo.train_step(x.to(dev), y.to(dev))
torch.cuda.synchronize()
single = torch.cat([t.reshape(-1) for t in solo.tables]).clone()
torch.testing.assert_close(results[True], single, rtol=1e-5, atol=2e-6)
mine = results[True]
both = [torch.empty_like(mine) for _ in range(world)]
dist.all_gather(both, mine)
assert torch.equal(both[0], both[1]), "ranks disagree after the peer-memory step"
torch.testing.assert_close(results[True], results[False], rtol=1e-5, atol=1e-6)
assert not torch.equal(results[True], torch.cat([t.reshape(-1) for t in tabs]).to(dev)), "tables did not move"
dist.barrier()
print(f"rank {rank} ok", flush=True)
os._exit(0)
"""


def test_peer_optimizer_matches_allreduce_path(tmp_path):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, DIFFLUT_ROOT=root, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29533", str(script)]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert "rank 0 ok" in out.stdout and "rank 1 ok" in out.stdout


def test_barrier_wait_runs_out_and_reports():
    """A barrier whose peer never arrives (its flag array is a local buffer nothing writes) gives up after the
    wall-clock limit, records which rank was missing and leaves the context usable."""
    import ctypes
    import time

    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from difflut_b200 import _native

    dev = torch.device("cuda", 0)
    mine = torch.zeros(8, dtype=torch.int32, device=dev)
    absent = torch.zeros(8, dtype=torch.int32, device=dev)  # stands in for rank 1's flag array
    ctrl = torch.zeros(2, dtype=torch.int32, device=dev)
    ptrs = (ctypes.c_void_p * 2)(mine.data_ptr(), absent.data_ptr())
    t0 = time.time()
    with torch.cuda.device(dev):
        _native.call("dl_p2p_barrier", ctypes.addressof(ptrs), 0, 2, ctrl, 200)
    torch.cuda.synchronize()
    waited = time.time() - t0
    assert 0.15 < waited < 5.0
    assert ctrl.tolist() == [1, 2]  # epoch advanced; status = 1 + the missing rank
    assert int(absent[0]) == 1  # this rank did publish its arrival
    # a barrier of one rank with itself passes at once and the context still works
    ctrl.zero_()
    solo = (ctypes.c_void_p * 1)(mine.data_ptr())
    with torch.cuda.device(dev):
        _native.call("dl_p2p_barrier", ctypes.addressof(solo), 0, 1, ctrl, 200)
    assert ctrl.tolist() == [1, 0]
    assert float(torch.ones(4, device=dev).sum()) == 4.0


def _exchange_args(dev, count, world):
    import ctypes

    g = torch.Generator().manual_seed(11)
    grads = torch.randn(count, generator=g).to(dev) * 1e-3
    params = torch.randn(count, generator=g).to(dev)
    flags = torch.zeros(8 * 2 * 8, dtype=torch.int32, device=dev)
    absent = torch.zeros(8 * 2 * 8, dtype=torch.int32, device=dev)  # stands in for a rank that never runs
    m = torch.zeros(count // world, device=dev)
    v = torch.zeros(count // world, device=dev)
    state = torch.ones(2, dtype=torch.float64, device=dev)
    ctrl = torch.zeros(17, dtype=torch.int32, device=dev)

    def table(*tensors):
        arr = (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])
        return arr

    return grads, params, flags, absent, m, v, state, ctrl, table


def test_exchange_kernel_with_one_rank_equals_adam_step():
    import ctypes

    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from difflut_b200 import _native

    dev = torch.device("cuda", 0)
    count = 3 * 4096 + 512  # two "layers": slices of 4096*2 and the rest
    grads, params, flags, _, m, v, state, ctrl, table = _exchange_args(dev, count, 1)
    ref_p, ref_m, ref_v = params.clone(), m.clone(), v.clone()
    ref_state = state.clone()
    tg, tp, tf = table(grads), table(params), table(flags)
    split = 8192
    with torch.cuda.device(dev):
        for step in range(3):
            grads.mul_(-0.7).add_(1e-4)  # a different gradient every step
            _native.call("dl_adam_step", ref_p, grads, ref_m, ref_v, ref_state, count, 1e-2, 0.9, 0.999, 1e-8, 1.0)
            # upper slice first on channel 1, lower slice last on channel 0 (it advances the state)
            _native.call("dl_p2p_exchange_adam", ctypes.addressof(tg), ctypes.addressof(tp), ctypes.addressof(tf),
                         m, v, state, ctrl, split, count - split, 1, 0, 1, 1, 0, 1, 1e-2, 0.9, 0.999, 1e-8, 1.0, 200)
            _native.call("dl_p2p_exchange_adam", ctypes.addressof(tg), ctypes.addressof(tp), ctypes.addressof(tf),
                         m, v, state, ctrl, 0, split, 0, 1, 0, 0, 0, 1, 1e-2, 0.9, 0.999, 1e-8, 1.0, 200)
            torch.cuda.synchronize()
            assert torch.equal(state, ref_state), (step, state.tolist(), ref_state.tolist())
            for name, got, want in (("m", m, ref_m), ("v", v, ref_v), ("params", params, ref_p)):
                bad = (got != want).nonzero().flatten()
                assert bad.numel() == 0, (f"step {step}: {name} differs at {bad.numel()} places, first {int(bad[0])}: "
                                          f"{float(got[bad[0]])!r} vs {float(want[bad[0]])!r}")
    with torch.cuda.device(dev):  # the deferred half of channel 1's rendezvous: every rank (this one) is done
        _native.call("dl_p2p_wait_done", ctypes.addressof(tf), ctrl, 1, 0, 1, 200)
    torch.cuda.synchronize()
    c = ctrl.tolist()
    assert c[0] == 0 and c[1] == 3 and c[3] == 3 and c[2] == 0 and c[4] == 0  # status, epochs, counters reset


def test_exchange_kernel_gives_up_and_touches_nothing():
    import ctypes
    import time

    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from difflut_b200 import _native

    dev = torch.device("cuda", 0)
    count = 8 * 1024
    grads, params, flags, absent, m, v, state, ctrl, table = _exchange_args(dev, count, 2)
    m.fill_(0.25)
    v.fill_(0.5)
    before = (params.clone(), m.clone(), v.clone(), state.clone())
    peer_grads, peer_params = torch.zeros_like(grads), params.clone()
    tg, tp, tf = table(grads, peer_grads), table(params, peer_params), table(flags, absent)
    args = (ctypes.addressof(tg), ctypes.addressof(tp), ctypes.addressof(tf), m, v, state, ctrl, 0, count, 0, 1, 0, 0, 0, 2,
            1e-2, 0.9, 0.999, 1e-8, 1.0, 200)
    t0 = time.time()
    with torch.cuda.device(dev):
        _native.call("dl_p2p_exchange_adam", *args)
    torch.cuda.synchronize()
    waited = time.time() - t0
    assert 0.15 < waited < 5.0
    assert int(ctrl[0]) == 2  # 1 + the rank that never arrived
    assert int(absent[0]) == 1  # this rank did publish its arrival (channel 0, "arrive", slot of rank 0)
    for now, was in zip((params, m, v, state), before):
        assert torch.equal(now, was)
    assert torch.equal(peer_params, before[0])
    # the status is sticky: the next call returns at once and still changes nothing
    t0 = time.time()
    with torch.cuda.device(dev):
        _native.call("dl_p2p_exchange_adam", *args)
    torch.cuda.synchronize()
    assert time.time() - t0 < 0.15
    for now, was in zip((params, m, v, state), before):
        assert torch.equal(now, was)
    # the three-kernel form: a status left by a barrier stops the reduce + Adam kernel as well
    bctrl = torch.tensor([1, 2], dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        _native.call("dl_p2p_reduce_adam", ctypes.addressof(tg), ctypes.addressof(tp), m, v, state, bctrl, count, 0, 2,
                     1e-2, 0.9, 0.999, 1e-8, 1.0)
    torch.cuda.synchronize()
    for now, was in zip((params, m, v, state), before):
        assert torch.equal(now, was)
    # the deferred wait gives up the same way: an epoch nobody has reported "done" for
    ctrl2 = torch.zeros(17, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        _native.call("dl_p2p_wait_done", ctypes.addressof(tf), ctrl2, 3, 0, 2, 200)  # before any exchange: returns at once
    torch.cuda.synchronize()
    assert int(ctrl2[0]) == 0
    ctrl2[1 + 2 * 3] = 1
    t0 = time.time()
    with torch.cuda.device(dev):
        _native.call("dl_p2p_wait_done", ctypes.addressof(tf), ctrl2, 3, 0, 2, 200)
    torch.cuda.synchronize()
    assert 0.15 < time.time() - t0 < 5.0 and int(ctrl2[0]) in (1, 2)
    assert float(torch.ones(4, device=dev).sum()) == 4.0  # the context is still usable
