"""The allocation-free variant of the GroupSum-fused last layer.

`dl_dwn_fwd_groupsum_noalloc_t` serves hosts that cannot give the library a scratch buffer (their
device memory is owned by another component, or they cannot afford cudaMalloc's device-wide
synchronisation).  It keeps its partial sums in a fixed array inside the library, so the checks here
are: same logits as the caller-scratch entry point, on two calls in a row (the second call finds the
first call's leftovers in the shared array), and a clear refusal beyond the array's capacity.
This file sorts last on purpose: a run that stops at the first failure has then run everything else.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(dev, seed, B, I, N, k, with_host_copies=False):
    from difflut_b200 import _native
    from difflut_b200.layers.random_layer import draw_random_mapping

    gen = torch.Generator().manual_seed(seed)
    Bp = _native.padded_batch(B)
    x_host = torch.rand(B, I, generator=gen)
    x = x_host.to(dev)
    bits = torch.empty(I, Bp // 32, device=dev, dtype=torch.int32)
    _native.call("dl_pack_rows_to_t", x, bits, B, I, Bp, 0.5)
    map_host = draw_random_mapping(I, N, 6, seed, True)
    mapping = map_host.to(device=dev, dtype=torch.int32).contiguous()
    tab_host = torch.randn(N, 64, generator=gen)
    tables = tab_host.to(dev)
    if with_host_copies:
        return bits, mapping, tables, Bp, (x_host, map_host, tab_host)
    return bits, mapping, tables, Bp


def test_noalloc_matches_caller_scratch_twice_in_a_row():
    from difflut_b200 import _native

    dev = torch.device("cuda", 0)
    lib = _native.lib()
    # two different problems back to back: the second must not be disturbed by what the first left behind
    for seed, B, I, N, k, tau in ((0, 700, 96, 130, 10, 3.0), (1, 300, 64, 45, 4, 1.0)):
        bits, mapping, tables, Bp = _case(dev, seed, B, I, N, k)
        S = lib.dl_dwn_groupsum_splits(N, k)
        partial = torch.empty(k * S, Bp, device=dev)
        want = torch.empty(k, Bp, device=dev)
        _native.call("dl_dwn_fwd_groupsum_t", bits, mapping, tables, partial, want, N, 6, k, tau, Bp)
        for _ in range(2):
            got = torch.full((k, Bp), float("nan"), device=dev)
            _native.call("dl_dwn_fwd_groupsum_noalloc_t", bits, mapping, tables, got, N, 6, k, tau, Bp)
            torch.cuda.synchronize()
            # same kernels, same summation order: bit-identical (the suite's tolerance for this
            # forward is rtol 1e-5, this is stricter)
            assert torch.equal(got, want)


def test_noalloc_rejects_sizes_beyond_its_array():
    from difflut_b200 import _native

    dev = torch.device("cuda", 0)
    bits, mapping, tables, Bp = _case(dev, 2, 256, 64, 45, 4)
    out = torch.empty(4, Bp, device=dev)
    # 4000 nodes, 10 classes, 16384 samples would need 31 MiB of partial sums: more than the array holds
    with pytest.raises(RuntimeError, match="capacity"):
        _native.call("dl_dwn_fwd_groupsum_noalloc_t", bits, mapping, tables, out, 4000, 6, 10, 1.0, 16384)


def test_noalloc_logits_match_the_oracle():
    """The chain closed in this file: the allocation-free entry point against the CPU oracle's logits
    (table look-up of every node, difflut/nodes/dwn_node.py:138-165, then GroupSum,
    difflut/utils/modules.py:116-163)."""
    from difflut_b200 import _native
    from oracle import difflut_oracle as O

    dev = torch.device("cuda", 0)
    B, I, N, k, tau = 700, 96, 130, 10, 3.0
    bits, mapping, tables, Bp, (x, idx, tab) = _case(dev, 5, B, I, N, k, with_host_copies=True)
    got = torch.full((k, Bp), float("nan"), device=dev)
    _native.call("dl_dwn_fwd_groupsum_noalloc_t", bits, mapping, tables, got, N, 6, k, tau, Bp)
    torch.cuda.synchronize()
    vals = O.dwn_forward(O.gather_mapping(x, idx), tab.unsqueeze(1)).reshape(B, N)
    want = O.groupsum(vals, k, tau)
    torch.testing.assert_close(got[:, :B].t().cpu(), want, rtol=1e-5, atol=1e-5)
