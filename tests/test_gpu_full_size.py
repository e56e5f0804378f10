"""The benchmarked configurations at their full sizes, value for value against the CPU oracle.

Config 4 (`bench.py`'s default line): 784 features -> 8-threshold thermometer -> RandomLayer+DWN
16000 / 8000 / 4000 (n=6) -> GroupSum(10, tau=33) -> cross-entropy -> Adam, batch 8192, built exactly
as `bench.build_network` builds it and stepped under a CUDA graph.  This is the path whose kernels
walk the nodes with a persistent grid and add eight 1024-sample groups into the table gradient in
place; the small fixtures never reach those loops.  Config 5: the same network's bit-packed hard
inference at 2^14 samples against the reference's eval semantics (difflut/nodes/dwn_node.py:457-483,
difflut/utils/modules.py:158-163, restated in the oracle).

The oracle walks the batch in row chunks (about a minute of host time for config 4).
"""

import warnings

import numpy as np
import pytest
import torch

from oracle import difflut_oracle as O
from parity_util import close_normwise

pytestmark = pytest.mark.gpu
warnings.simplefilter("ignore")


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda", 0)


@pytest.fixture(scope="module")
def c4(dev):
    """Network, inputs and the oracle's answers for one training step of config 4."""
    import bench

    net, x, labels = bench.build_network(dev, 0, 1)
    assert x.shape == (8192, 784) and net.N == [16000, 8000, 4000] and net.fused_backward
    thr = O.thermometer_thresholds(x, bench.THERMO_BITS)
    assert torch.equal(thr, net.encoder.thresholds.reshape(thr.shape).cpu())
    maps = [l._mapping_indices.cpu() for l in net.layers]
    tables = [l.luts.detach().cpu().clone() for l in net.layers]
    for li, (m, I) in enumerate(zip(maps, net.I)):
        assert torch.equal(m.long(), O.random_mapping(I, net.N[li], 6, li, True).long()), "seeded map"
    alpha, beta = net.alpha[0], net.beta[0]
    logits, loss, grads = O.dwn_network_train_reference(x, labels, thr, maps, tables, net.k, net.tau, alpha, beta,
                                                        chunk_rows=512)
    return {"net": net, "x": x, "labels": labels, "tables": tables, "logits": logits, "loss": loss, "grads": grads,
            "thr": thr, "maps": maps}


def test_config4_logits_full_size(c4, dev):
    got = c4["net"].logits(c4["x"].to(dev)).cpu()
    # a logit is a sum of 400 table values / tau: same values, different summation order
    close_normwise(got, c4["logits"], "config-4 logits (8192 x 10)")


def test_config4_train_step_under_graph_full_size(c4, dev):
    net = c4["net"]
    x, labels = c4["x"].to(dev), c4["labels"].to(dev)
    loss = net.train_step(x, labels, use_graph=True)
    torch.cuda.synchronize()
    assert net._graph is not None, "the step must have been captured and replayed"
    close_normwise(loss.cpu().reshape(()), c4["loss"], "config-4 loss")
    for li in range(3):
        got = net.grads[li].cpu()
        assert got.shape == c4["grads"][li].shape
        close_normwise(got, c4["grads"][li], f"config-4 table gradient of layer {li + 1} ({net.N[li]} x 64)")
    # tables after the step: Adam's first step from zero moments, from the oracle's gradients
    for li in range(3):
        p0, g = c4["tables"][li], c4["grads"][li]
        ref, _, _ = O.adam_step(p0, g, torch.zeros_like(g), torch.zeros_like(g), 1, net.lr)
        got = net.layers[li].luts.detach().cpu()
        assert got.shape == ref.shape
        # the first Adam step moves every visited entry by lr * g / (|g| + eps): an entry whose gradient
        # cancels to about eps (1e-8) amplifies a last-bit difference of the gradient by up to lr / eps, so
        # the bound on the tables is absolute: 1e-5 of their scale
        close_normwise(got, ref, f"config-4 tables of layer {li + 1} after one Adam step")
    # a second replay of the same graph keeps working on the updated tables: gradients change, stay finite
    before = net.flat_grad.clone()
    net.train_step(x, labels, use_graph=True)
    torch.cuda.synchronize()
    assert bool(torch.isfinite(net.flat_grad).all()) and not torch.equal(before, net.flat_grad)


def test_config4_layer_api_full_size_equals_oracle_gradients(c4, dev):
    """The reference-shaped call sequence (encoder -> three RandomLayers -> GroupSum -> autograd) on the
    same batch, with the step's ORIGINAL tables: logits and table gradients against the oracle."""
    from difflut_b200.encoder import ThermometerEncoder
    from difflut_b200.layers import RandomLayer
    from difflut_b200.nodes import DWNNode, NodeConfig
    from difflut_b200.utils import GroupSum

    net = c4["net"]
    x, labels = c4["x"].to(dev), c4["labels"].to(dev)
    enc = ThermometerEncoder(num_bits=8).fit(c4["x"]).to(dev)
    layers, I = [], 6272
    for li, N in enumerate(net.N):
        l = RandomLayer(I, N, DWNNode, NodeConfig(input_dim=6, output_dim=1), seed=li).to(dev)
        with torch.no_grad():
            l.luts.copy_(c4["tables"][li].to(dev))
        l.train()
        layers.append(l)
        I = N
    h = enc(x)
    for l in layers:
        h = l(h)
    logits = GroupSum(k=net.k, tau=net.tau, use_randperm=False)(h)
    close_normwise(logits.detach().cpu(), c4["logits"], "layer-API logits at config-4 size")
    torch.nn.functional.cross_entropy(logits, labels.long()).backward()
    for li in range(3):
        close_normwise(layers[li].luts.grad.cpu(), c4["grads"][li], f"layer-API table gradient of layer {li + 1}")


def test_config5_hard_counts_full_width(c4, dev):
    """2^14 samples through the binarised 16000/8000/4000 network: class counts bit-exact."""
    net = c4["net"]
    B = 1 << 14
    gen = torch.Generator().manual_seed(5)
    x = torch.rand(B, 784, generator=gen)
    tables = [l.luts.detach().cpu().clone() for l in net.layers]  # the tables as they are now (after the steps)
    ref = []
    for lo in range(0, B, 1024):
        bits = O.thermometer_encode(x[lo:lo + 1024], c4["thr"])
        ref.append(O.dwn_network_hard_counts(bits, c4["maps"], tables, net.k))
    ref = torch.cat(ref)
    got = net.hard_counts(x.to(dev)).cpu()
    assert got.dtype == torch.int32 and got.shape == (B, net.k)
    assert torch.equal(got, ref)
    # the same through the packed-rows input (config 5's input format: 196 uint32 words per sample)
    bits_all = torch.cat([O.thermometer_encode(x[lo:lo + 4096], c4["thr"]) for lo in range(0, B, 4096)])
    packed = torch.from_numpy(O.pack_bits_row_major(bits_all).view(np.int32)).to(dev)
    assert packed.shape == (B, 196)
    assert torch.equal(net.hard_counts(packed_rows=packed).cpu(), ref)
    # a ragged batch size walks the padded tail of the last 128-sample chunk
    got_ragged = net.hard_counts(x[:5000].to(dev)).cpu()
    assert torch.equal(got_ragged, ref[:5000])
