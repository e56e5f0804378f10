"""GPU parity: every CUDA path, called through the public API (which calls the C ABI), against the
golden fixtures produced by the reference and against the CPU oracle on seeded inputs.

Bars: bit-exact for bits, addresses (observable through exact table values), index maps and hard
outputs; rtol 1e-5 (+ small atol for near-zero sums) for fp32 outputs; gradients that are long sums
over the batch (different summation order than the reference) are held to 1e-5 norm-wise:
max|got - ref| <= 1e-5 * max|ref|, with the measured ratio recorded (tests/parity_util.py).
"""

import warnings

import numpy as np
import pytest
import torch

from oracle import difflut_oracle as O
from parity_util import close_normwise

pytestmark = pytest.mark.gpu
warnings.simplefilter("ignore")


def T(a):
    return torch.from_numpy(np.asarray(a))


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda", 0)


def _layer(dev, I, N, n, O_, node, mapping, extra=None):
    from difflut_b200.layers import RandomLayer
    from difflut_b200.nodes import NodeConfig

    cfg = NodeConfig(input_dim=n, output_dim=O_, extra_params=extra or {})
    return RandomLayer(I, N, node, cfg, seed=0, mapping_indices=mapping).to(dev)


# ------------------------------------------------------------------------------ encoder
def test_thermometer_bits_exact(golden, dev):
    from difflut_b200.encoder import ThermometerEncoder

    g = golden("thermometer")
    for nb in (1, 3, 8):
        enc = ThermometerEncoder(num_bits=nb).fit(T(g[f"x_fit_T{nb}"]))
        assert torch.equal(enc.thresholds, T(g[f"thr_T{nb}"]))
        x = T(g[f"x_T{nb}"]).to(dev)
        bits = enc.to(dev).encode(x)
        assert bits.dtype == torch.float32 and bits.shape == (x.shape[0], x.shape[1] * nb)
        assert np.array_equal(bits.cpu().numpy().astype(np.uint8), g[f"bits_T{nb}"])
        packed_t = enc.encode_packed_t(x).cpu().numpy().view(np.uint32)
        ref_t = O.pack_bits_feature_major(T(g[f"bits_T{nb}"]).float())
        assert np.array_equal(packed_t[:, : ref_t.shape[1]], ref_t)
        assert not packed_t[:, ref_t.shape[1]:].any(), "padding words must be zero"
        packed_r = enc.encode_packed(x).cpu().numpy().view(np.uint32)
        assert np.array_equal(packed_r, O.pack_bits_row_major(T(g[f"bits_T{nb}"]).float()))
        enc3 = ThermometerEncoder(num_bits=nb, flatten=False).fit(T(g[f"x_fit_T{nb}"])).to(dev)
        assert enc3.encode(x).shape == (x.shape[0], x.shape[1], nb)


def test_thermometer_fit_variants_bits_exact(golden, dev):
    from difflut_b200.encoder import DistributiveThermometerEncoder, GaussianThermometerEncoder

    g = golden("thermometer")
    x_fit, x = T(g["variant_x_fit"]), T(g["variant_x"]).to(dev)
    for tag, cls in (("gauss", GaussianThermometerEncoder), ("distr", DistributiveThermometerEncoder)):
        enc = cls(num_bits=4).fit(x_fit).to(dev)
        assert np.array_equal(enc.encode(x).cpu().numpy().astype(np.uint8), g[f"{tag}_bits"])


def test_thermometer_unfitted_raises(dev):
    from difflut_b200.encoder import ThermometerEncoder

    with pytest.raises(RuntimeError):
        ThermometerEncoder(num_bits=2).encode(torch.rand(3, 4, device=dev))


def test_layout_round_trips(dev):
    from difflut_b200 import _native

    gen = torch.Generator().manual_seed(1)
    for B, F in ((1, 1), (37, 45), (300, 70), (129, 33)):
        Bp = _native.padded_batch(B)
        x = torch.rand(B, F, generator=gen).to(dev)
        t = torch.full((F, Bp), 7.0, device=dev)
        _native.call("dl_f32_rows_to_t", x, t, B, F, Bp)
        assert torch.equal(t[:, :B].t(), x) and not t[:, B:].any()
        back = torch.empty_like(x)
        _native.call("dl_f32_t_to_rows", t, back, B, F, Bp)
        assert torch.equal(back, x)
        bits = torch.empty(F, Bp // 32, device=dev, dtype=torch.int32)
        _native.call("dl_pack_rows_to_t", x, bits, B, F, Bp, 0.5)
        ref = O.pack_bits_feature_major((x.cpu() >= 0.5).float())
        got = bits.cpu().numpy().view(np.uint32)
        assert np.array_equal(got[:, : ref.shape[1]], ref) and not got[:, ref.shape[1]:].any()
        rows = torch.empty(B, F, device=dev)
        _native.call("dl_bits_t_to_rows", bits, rows, B, F, Bp)
        assert torch.equal(rows, (x >= 0.5).float())
        pr = torch.from_numpy(O.pack_bits_row_major((x.cpu() >= 0.5).float()).view(np.int32)).to(dev)
        bits2 = torch.empty_like(bits)
        _native.call("dl_bits_rows_to_t", pr, bits2, B, F, pr.shape[1], Bp)
        assert torch.equal(bits2, bits)


# ------------------------------------------------------------------------------ DWN
@pytest.mark.parametrize("tag", ["n6", "n4o2", "n2"])
def test_dwn_layer_matches_reference(golden, dev, tag):
    from difflut_b200.nodes import DWNNode

    g = golden("dwn_layer")
    x, idx, tab = T(g[f"{tag}_x"]), T(g[f"{tag}_map"]), T(g[f"{tag}_tables"])
    N, O_, L = tab.shape
    n = int(np.log2(L))
    layer = _layer(dev, x.shape[1], N, n, O_, DWNNode, idx)
    with torch.no_grad():
        layer.luts.copy_(tab.to(dev))
    assert torch.equal(layer._mapping_indices.cpu(), idx)
    xg = x.to(dev).requires_grad_(True)
    layer.train()
    y = layer(xg)
    assert torch.equal(y.cpu(), T(g[f"{tag}_y"])), "table values must be exact (addresses bit-exact)"
    y.backward(T(g[f"{tag}_gy"]).to(dev))
    torch.testing.assert_close(xg.grad.cpu(), T(g[f"{tag}_gx"]), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(layer.luts.grad.cpu(), T(g[f"{tag}_gtables"]), rtol=1e-5, atol=1e-6)
    layer.eval()
    ye = layer((x >= 0.5).float().to(dev))
    assert np.array_equal(ye.cpu().numpy().astype(np.uint8), g[f"{tag}_y_eval"])
    # the materialised path (get_mapping + node arithmetic) gives the same numbers
    layer.train()
    xg2 = x.to(dev).requires_grad_(True)
    y2 = layer._run_nodes(layer.get_mapping(xg2))
    assert torch.equal(y2, y)
    y2.backward(T(g[f"{tag}_gy"]).to(dev))
    torch.testing.assert_close(xg2.grad.cpu(), T(g[f"{tag}_gx"]), rtol=1e-5, atol=1e-6)
    # per-node views: node(node_input) equals the layer's column
    node = layer.nodes[1]
    yn = node(layer.get_mapping(x.to(dev))[:, 1, :])
    assert torch.equal(yn, y.detach().reshape(x.shape[0], N, O_)[:, 1, :])


@pytest.mark.parametrize("tag", ["n6", "n4o2", "n3"])
def test_dwn_stable_layer_matches_reference(golden, dev, tag):
    from difflut_b200.nodes import DWNStableNode

    g = golden("dwn_stable_layer")
    x, idx, raw = T(g[f"{tag}_x"]), T(g[f"{tag}_map"]), T(g[f"{tag}_raw"])
    scale = float(g[f"{tag}_scale"][0])
    N, O_, L = raw.shape
    n = int(np.log2(L))
    layer = _layer(dev, x.shape[1], N, n, O_, DWNStableNode, idx, extra={"gradient_scale": scale})
    assert layer.gradient_scale.shape == (N,) and float(layer.gradient_scale[0]) == pytest.approx(scale)
    with torch.no_grad():
        layer.raw_luts.copy_(raw.to(dev))
    xg = x.to(dev).requires_grad_(True)
    layer.train()
    y = layer(xg)
    torch.testing.assert_close(y.cpu(), T(g[f"{tag}_y"]), rtol=0, atol=2e-7)  # sigmoid on the device
    y.backward(T(g[f"{tag}_gy"]).to(dev))
    torch.testing.assert_close(xg.grad.cpu(), T(g[f"{tag}_gx"]), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(layer.raw_luts.grad.cpu(), T(g[f"{tag}_graw"]), rtol=1e-5, atol=1e-6)
    assert layer.gradient_scale.grad is None  # the reference reads it with .item(): no gradient
    layer.eval()
    ye = layer((x >= 0.5).float().to(dev))
    assert np.array_equal(ye.cpu().numpy().astype(np.uint8), g[f"{tag}_y_eval"])
    # materialised path and per-node views
    layer.train()
    xg2 = x.to(dev).requires_grad_(True)
    y2 = layer._run_nodes(layer.get_mapping(xg2))
    assert torch.equal(y2, y)
    y2.backward(T(g[f"{tag}_gy"]).to(dev))
    torch.testing.assert_close(xg2.grad.cpu(), T(g[f"{tag}_gx"]), rtol=1e-5, atol=1e-6)
    node = layer.nodes[1]
    yn = node(layer.get_mapping(x.to(dev))[:, 1, :])
    assert torch.equal(yn, y.detach().reshape(x.shape[0], N, O_)[:, 1, :])
    # reference-format state dict round trip
    sd = layer.state_dict()
    assert f"nodes.{N - 1}.raw_luts" in sd and f"nodes.0.gradient_scale" in sd and "raw_luts" not in sd
    other = _layer(dev, x.shape[1], N, n, O_, DWNStableNode, idx)
    other.load_state_dict(sd)
    assert torch.equal(other.raw_luts, layer.raw_luts) and torch.equal(other.gradient_scale, layer.gradient_scale)


@pytest.mark.parametrize("tag", ["n6", "n4o2", "n2"])
def test_hybrid_layer_matches_reference(golden, dev, tag):
    from difflut_b200.nodes import HybridNode

    g = golden("hybrid_layer")
    x, idx, raw = T(g[f"{tag}_x"]), T(g[f"{tag}_map"]), T(g[f"{tag}_raw"])
    N, O_, L = raw.shape
    n = int(np.log2(L))
    layer = _layer(dev, x.shape[1], N, n, O_, HybridNode, idx)
    with torch.no_grad():
        layer.raw_luts.copy_(raw.to(dev))
    xg = x.to(dev).requires_grad_(True)
    layer.train()
    y = layer(xg)
    torch.testing.assert_close(y.cpu(), T(g[f"{tag}_y"]), rtol=0, atol=2e-7)  # sigmoid on the device
    y.backward(T(g[f"{tag}_gy"]).to(dev))
    gx_ref = T(g[f"{tag}_gx"])
    torch.testing.assert_close(xg.grad.cpu(), gx_ref, rtol=1e-5, atol=1e-6)
    assert torch.count_nonzero(xg.grad[0, : x.shape[1] // 2]) == 0  # exactly binary inputs: zero gradient
    torch.testing.assert_close(layer.raw_luts.grad.cpu(), T(g[f"{tag}_graw"]), rtol=1e-5, atol=1e-6)
    layer.eval()
    ye = layer((x >= 0.5).float().to(dev))
    assert np.array_equal(ye.cpu().numpy().astype(np.uint8), g[f"{tag}_y_eval"])
    # materialised path and per-node views
    layer.train()
    xg2 = x.to(dev).requires_grad_(True)
    y2 = layer._run_nodes(layer.get_mapping(xg2))
    assert torch.equal(y2, y)
    y2.backward(T(g[f"{tag}_gy"]).to(dev))
    torch.testing.assert_close(xg2.grad.cpu(), gx_ref, rtol=1e-5, atol=1e-6)
    node = layer.nodes[1]
    yn = node(layer.get_mapping(x.to(dev))[:, 1, :])
    assert torch.equal(yn, y.detach().reshape(x.shape[0], N, O_)[:, 1, :])
    assert node.binary_combinations.shape == (L, n)
    sd = layer.state_dict()
    assert f"nodes.{N - 1}.raw_luts" in sd and "nodes.0.binary_combinations" in sd and "raw_luts" not in sd
    other = _layer(dev, x.shape[1], N, n, O_, HybridNode, idx)
    other.load_state_dict(sd)
    assert torch.equal(other.raw_luts, layer.raw_luts)


@pytest.mark.parametrize("n,O_", [(5, 2), (8, 1), (9, 2)])
def test_hybrid_standalone_node_vs_oracle(dev, n, O_):
    """n <= 6: the layer kernel; wider nodes: the per-sample kernel on materialised inputs."""
    from difflut_b200.nodes import HybridNode

    gen = torch.Generator().manual_seed(31)
    B = 70
    x = torch.rand(B, n, generator=gen)
    x[0, :] = (torch.rand(n, generator=gen) > 0.5).float()  # exactly binary inputs: the 1e-8 guard decides
    node = HybridNode(input_dim=n, output_dim=O_).to(dev)
    tab = torch.sigmoid(node.raw_luts.detach()).cpu()
    xg = x.to(dev).requires_grad_(True)
    y = node.train()(xg)
    assert torch.equal(y.cpu(), O.dwn_forward(x.unsqueeze(1), tab.unsqueeze(0)).squeeze(1))
    gy = torch.randn(B, O_, generator=gen)
    y.backward(gy.to(dev))
    if n <= 6:
        gxm, gl = O.hybrid_backward(x.unsqueeze(1), tab.unsqueeze(0), gy.unsqueeze(1))
    else:
        # 2^n terms of mixed sign per input gradient: in fp32 the reference's own sum is only good to about 1e-5
        # here, so the wide kernel (double accumulation) is held to the formula evaluated in float64
        gxm, gl = O.hybrid_backward(x.double().unsqueeze(1), tab.double().unsqueeze(0), gy.double().unsqueeze(1))
        gxm, gl = gxm.float(), gl.float()
    close_normwise(xg.grad.cpu(), gxm.squeeze(1), f"hybrid node n={n}: input gradient")
    close_normwise(node.raw_luts.grad.cpu(), gl.squeeze(0) * tab * (1 - tab), f"hybrid node n={n}: table gradient")
    with pytest.raises(ValueError):
        HybridNode(input_dim=17, output_dim=1)


@pytest.mark.parametrize("n,O_", [(1, 1), (3, 2), (6, 1), (8, 1), (10, 2)])
def test_dwn_stable_standalone_node_vs_oracle(dev, n, O_):
    from difflut_b200.nodes import DWNStableNode

    gen = torch.Generator().manual_seed(20 + n)
    B = 50
    x = torch.rand(B, n, generator=gen)
    node = DWNStableNode(input_dim=n, output_dim=O_, gradient_scale=0.9).to(dev)
    raw = torch.randn(O_, 2 ** n, generator=gen)
    with torch.no_grad():
        node.raw_luts.copy_(raw.to(dev))
    tab = torch.sigmoid(node.raw_luts.detach()).cpu()  # the device's sigmoid, so look-ups compare exactly
    xg = x.to(dev).requires_grad_(True)
    node.train()
    y = node(xg)
    assert torch.equal(y.cpu(), O.dwn_forward(x.unsqueeze(1), tab.unsqueeze(0)).squeeze(1))
    gy = torch.randn(B, O_, generator=gen)
    y.backward(gy.to(dev))
    gxm, gl = O.dwn_stable_backward(x.unsqueeze(1), tab.unsqueeze(0), gy.unsqueeze(1), 0.9)
    close_normwise(xg.grad.cpu(), gxm.squeeze(1), "xg.grad.cpu()")
    close_normwise(node.raw_luts.grad.cpu(), (gl.squeeze(0) * tab * (1 - tab)), "node.raw_luts.grad.cpu()")
    node.eval()
    xb = (x >= 0.5).float()
    assert torch.equal(node(xb.to(dev)).cpu(), O.dwn_forward_eval(xb.unsqueeze(1), tab.unsqueeze(0)).squeeze(1))
    with pytest.raises(ValueError):
        DWNStableNode(input_dim=17, output_dim=1)


@pytest.mark.parametrize("kind", ["dwn_stable", "hybrid"])
def test_wide_node_layers_vs_oracle(dev, kind):
    """RandomLayer with 8-input DWNStable / Hybrid nodes (beyond the 6 inputs of the layer kernels): forward,
    eval and both gradients through the gather against the oracle."""
    from difflut_b200.nodes import DWNStableNode, HybridNode

    gen = torch.Generator().manual_seed(77)
    B, I, N, n, O_ = 40, 30, 9, 8, 2
    node = DWNStableNode if kind == "dwn_stable" else HybridNode
    extra = {"gradient_scale": 1.1} if kind == "dwn_stable" else None
    layer = _layer(dev, I, N, n, O_, node, None, extra)
    idx = layer._mapping_indices.cpu()
    x = torch.rand(B, I, generator=gen)
    tab = torch.sigmoid(layer.raw_luts.detach()).cpu()
    xg = x.to(dev).requires_grad_(True)
    layer.train()
    y = layer(xg)
    xm = O.gather_mapping(x, idx)
    assert torch.equal(y.cpu(), O.dwn_forward(xm, tab).reshape(B, -1))
    gy = torch.randn(B, N * O_, generator=gen)
    y.backward(gy.to(dev))
    if kind == "dwn_stable":
        gxm, gl = O.dwn_stable_backward(xm, tab, gy.view(B, N, O_), 1.1)
    else:  # the formula in float64 (see test_hybrid_standalone_node_vs_oracle)
        gxm, gl = O.hybrid_backward(xm.double(), tab.double(), gy.view(B, N, O_).double())
        gxm, gl = gxm.float(), gl.float()
    close_normwise(xg.grad.cpu(), O.gather_mapping_backward(gxm, idx, I), f"{kind} n=8 layer: input gradient")
    close_normwise(layer.raw_luts.grad.cpu(), gl * tab * (1 - tab), f"{kind} n=8 layer: table gradient")
    layer.eval()
    xb = (x >= 0.5).float()
    assert torch.equal(layer(xb.to(dev)).cpu(), O.dwn_forward_eval(O.gather_mapping(xb, idx), tab).reshape(B, -1))


@pytest.mark.parametrize("n,O_", [(1, 1), (3, 2), (6, 1), (8, 1), (10, 2)])
def test_dwn_standalone_node_vs_oracle(dev, n, O_):
    from difflut_b200.nodes import DWNNode

    gen = torch.Generator().manual_seed(n)
    B = 50
    x = torch.rand(B, n, generator=gen)
    node = DWNNode(input_dim=n, output_dim=O_).to(dev)
    tab = torch.randn(O_, 2 ** n, generator=gen)
    with torch.no_grad():
        node.luts.copy_(tab.to(dev))
    xg = x.to(dev).requires_grad_(True)
    node.train()
    y = node(xg)
    y_ref = O.dwn_forward(x.unsqueeze(1), tab.unsqueeze(0)).squeeze(1)
    assert torch.equal(y.cpu(), y_ref)
    gy = torch.randn(B, O_, generator=gen)
    y.backward(gy.to(dev))
    alpha, beta = 0.5 * 0.75 ** (n - 1), 0.25 / 0.75
    gxm, gl = O.dwn_backward(x.unsqueeze(1), tab.unsqueeze(0), gy.unsqueeze(1), alpha, beta)
    close_normwise(xg.grad.cpu(), gxm.squeeze(1), "xg.grad.cpu()")
    torch.testing.assert_close(node.luts.grad.cpu(), gl.squeeze(0), rtol=1e-5, atol=1e-6)
    node.eval()
    xb = (x >= 0.5).float()
    ye = node(xb.to(dev))
    assert torch.equal(ye.cpu(), O.dwn_forward_eval(xb.unsqueeze(1), tab.unsqueeze(0)).squeeze(1))


def test_dwn_residual_tables_pass_bit0(golden, dev):
    from difflut_b200.nodes import DWNNode

    node = DWNNode(input_dim=6, output_dim=1).to(dev).eval()
    with torch.no_grad():
        node.luts.copy_(T(golden("dwn_layer")["residual_tables"]).to(dev))
    a = torch.arange(64)
    pats = ((a[:, None] >> torch.arange(6)) & 1).float().to(dev)
    assert torch.equal(node(pats)[:, 0], pats[:, 0])
    import itertools

    assert node.export_bitstream() == [p[0] for p in itertools.product([0, 1], repeat=6)]


def test_dwn_config1_full_size_vs_oracle(dev):
    """BASELINE config 1: B=256 x 784, T=3, 2000 nodes, multinomial map, loss = sum of outputs."""
    from difflut_b200.encoder import ThermometerEncoder
    from difflut_b200.layers import RandomLayer
    from difflut_b200.nodes import DWNNode, NodeConfig

    gen = torch.Generator().manual_seed(0)
    x = torch.rand(256, 784, generator=gen)
    enc = ThermometerEncoder(num_bits=3).fit(x)
    layer = RandomLayer(2352, 2000, DWNNode, NodeConfig(input_dim=6, output_dim=1), seed=0,
                        ensure_full_input_coverage=False).to(dev)
    tab = torch.randn(2000, 1, 64, generator=gen)
    with torch.no_grad():
        layer.luts.copy_(tab.to(dev))
    bits_ref = O.thermometer_encode(x, O.thermometer_thresholds(x, 3))
    bits = enc.to(dev)(x.to(dev))
    assert torch.equal(bits.cpu(), bits_ref)
    idx = O.random_mapping(2352, 2000, 6, 0, False)
    assert torch.equal(layer._mapping_indices.cpu(), idx)
    bg = bits.clone().requires_grad_(True)
    y = layer(bg)
    xm = O.gather_mapping(bits_ref, idx)
    assert torch.equal(y.cpu(), O.dwn_forward(xm, tab).reshape(256, -1))
    y.sum().backward()
    gxm, gl = O.dwn_backward(xm, tab, torch.ones(256, 2000, 1), 0.5 * 0.75 ** 5, 0.25 / 0.75)
    torch.testing.assert_close(layer.luts.grad.cpu(), gl, rtol=1e-5, atol=1e-6)
    close_normwise(bg.grad.cpu(), O.gather_mapping_backward(gxm, idx, 2352), "bg.grad.cpu()")


# ------------------------------------------------------------------------------ probabilistic
def test_prob_layer_matches_reference(golden, dev):
    from difflut_b200.nodes import ProbabilisticNode
    from difflut_b200.utils import GroupSum

    g = golden("prob_layer")
    x, idx, raw = T(g["x"]), T(g["map"]), T(g["raw"])
    layer = _layer(dev, x.shape[1], raw.shape[0], 6, 1, ProbabilisticNode, idx)
    with torch.no_grad():
        layer.raw_weights.copy_(raw.to(dev))
    layer.train()
    xg = x.to(dev).requires_grad_(True)
    y = layer(xg)
    torch.testing.assert_close(y.cpu(), T(g["y"]), rtol=1e-5, atol=1e-6)
    logits = GroupSum(k=10, tau=1.0, use_randperm=False)(y)
    torch.testing.assert_close(logits.cpu(), T(g["logits"]), rtol=1e-5, atol=1e-5)
    loss = torch.nn.functional.cross_entropy(logits, T(g["labels"]).to(dev))
    loss.backward()
    torch.testing.assert_close(loss.detach().cpu(), T(g["loss"]), rtol=1e-5, atol=1e-6)
    close_normwise(xg.grad.cpu(), T(g["gx"]), "xg.grad.cpu()")
    close_normwise(layer.raw_weights.grad.cpu(), T(g["graw"]), "layer.raw_weights.grad.cpu()")
    # fused with GroupSum: same logits and gradients without the (B, N) tensor
    layer.raw_weights.grad = None
    xg2 = x.to(dev).requires_grad_(True)
    logits2 = layer.forward_groupsum(xg2, 10, 1.0)
    torch.testing.assert_close(logits2.cpu(), T(g["logits"]), rtol=1e-5, atol=1e-5)
    torch.nn.functional.cross_entropy(logits2, T(g["labels"]).to(dev)).backward()
    close_normwise(xg2.grad.cpu(), T(g["gx"]), "xg2.grad.cpu()")
    close_normwise(layer.raw_weights.grad.cpu(), T(g["graw"]), "layer.raw_weights.grad.cpu()")
    layer.eval()
    ye = layer((x >= 0.5).float().to(dev))
    assert np.array_equal(ye.cpu().numpy().astype(np.uint8), g["y_eval"])


def test_prob_layer_temperature_multi_output(golden, dev):
    from difflut_b200.nodes import ProbabilisticNode

    g = golden("prob_layer")
    x, idx, raw = T(g["t_x"]), T(g["t_map"]), T(g["t_raw"])
    layer = _layer(dev, x.shape[1], raw.shape[0], 3, 2, ProbabilisticNode, idx, {"temperature": 0.5})
    with torch.no_grad():
        layer.raw_weights.copy_(raw.to(dev))
    layer.train()
    xg = x.to(dev).requires_grad_(True)
    y = layer(xg)
    torch.testing.assert_close(y.cpu(), T(g["t_y"]), rtol=1e-5, atol=1e-6)
    y.backward(T(g["t_gy"]).to(dev))
    close_normwise(xg.grad.cpu(), T(g["t_gx"]), "xg.grad.cpu()")
    close_normwise(layer.raw_weights.grad.cpu(), T(g["t_graw"]), "layer.raw_weights.grad.cpu()")
    # standalone node on mapped inputs
    node = ProbabilisticNode(input_dim=3, output_dim=2, temperature=0.5).to(dev)
    with torch.no_grad():
        node.raw_weights.copy_(raw[0].to(dev))
    xm = O.gather_mapping(x, idx)[:, 0, :]
    out = node(xm.to(dev))
    torch.testing.assert_close(out.cpu(), T(g["t_y"]).reshape(x.shape[0], -1, 2)[:, 0, :], rtol=1e-5, atol=1e-6)


def test_prob_edge_inputs_finite(dev):
    """x exactly 0 or 1: the product-rule gradient stays finite (the reference's autograd path)."""
    from difflut_b200.nodes import ProbabilisticNode

    node = ProbabilisticNode(input_dim=6, output_dim=1).to(dev)
    x = torch.tensor([[0.0, 1.0, 0.0, 1.0, 0.5, 0.0], [1.0] * 6, [0.0] * 6], device=dev, requires_grad=True)
    y = node(x)
    y.sum().backward()
    xr = x.detach().cpu().requires_grad_(True)
    yr = O.prob_forward(xr.unsqueeze(1), node.raw_weights.detach().cpu().unsqueeze(0), 1.0)
    yr.sum().backward()
    assert torch.isfinite(x.grad).all()
    torch.testing.assert_close(y.detach().cpu(), yr.detach().reshape(3, 1), rtol=1e-5, atol=1e-6)
    close_normwise(x.grad.cpu(), xr.grad, "x.grad.cpu()")


# ------------------------------------------------------------------------------ learnable
def test_learnable_layer_matches_reference(golden, dev):
    from difflut_b200.layers import LearnableLayer
    from difflut_b200.nodes import DWNNode, NodeConfig

    g = golden("learnable_layer")
    x, W, tab = T(g["x"]), T(g["W"]), T(g["tables"])
    layer = LearnableLayer(x.shape[1], tab.shape[0], DWNNode, NodeConfig(input_dim=6, output_dim=1)).to(dev)
    with torch.no_grad():
        layer.mapping.W.copy_(W.to(dev))
        layer.luts.copy_(tab.to(dev))
    layer.train()
    xg = x.to(dev).requires_grad_(True)
    m = layer.get_mapping(xg)
    torch.testing.assert_close(m.detach().cpu(), T(g["m"]), rtol=1e-2, atol=1e-4)
    y = layer(xg)
    # soft selections close to 0.5 could flip an address under a low-precision GEMM; the fixture has none
    torch.testing.assert_close(y.cpu(), T(g["y"]), rtol=1e-5, atol=1e-6)
    y.backward(T(g["gy"]).to(dev))
    torch.testing.assert_close(layer.luts.grad.cpu(), T(g["gtables"]), rtol=1e-5, atol=1e-6)
    # the backward GEMMs run on bf16 operands: 1e-2 of the gradient's scale
    gx_ref, gW_ref = T(g["gx"]), T(g["gW"])
    torch.testing.assert_close(xg.grad.cpu(), gx_ref, rtol=1e-2, atol=1e-2 * float(gx_ref.abs().max()))
    torch.testing.assert_close(layer.mapping.W.grad.cpu(), gW_ref, rtol=1e-2, atol=1e-2 * float(gW_ref.abs().max()))
    layer.eval()
    assert np.array_equal(layer.get_mapping_matrix().cpu().numpy(), g["hard_idx"])
    ye = layer(x.to(dev))
    assert np.array_equal(ye.cpu().numpy().astype(np.uint8), g["y_eval"])
    layer.update_tau(500)
    assert abs(layer.tau - float(g["tau_500"][0])) < 1e-12


def test_learnable_feature_major_path_equals_row_path(dev):
    """Batches that are a multiple of 128 train through the swapped-operand contraction; same outputs and
    gradients as the row-major path (bf16 contractions: 1e-2 of the gradient's scale), for DWN and
    DWNStable nodes, and against the fp32 oracle."""
    from difflut_b200.layers import LearnableLayer
    from difflut_b200.nodes import DWNNode, DWNStableNode, NodeConfig

    gen = torch.Generator().manual_seed(9)
    B, I, N = 256, 72, 40
    x = torch.bernoulli(torch.full((B, I), 0.5), generator=gen)
    # two outputs per node: the connection plan is no longer disjoint per virtual node, so the input gradient
    # takes the general kernel and the fp32 hand-over while the forward still receives packed bits
    for node, out_dim in ((DWNNode, 1), (DWNStableNode, 1), (DWNNode, 2)):
        gy = torch.randn(B, N * out_dim, generator=gen).to(dev)
        layer = LearnableLayer(I, N, node, NodeConfig(input_dim=6, output_dim=out_dim)).to(dev).train()
        with torch.no_grad():
            layer.mapping.W.copy_((torch.randn(N * 6, I, generator=gen) * 2.0).to(dev))
        xa = x.to(dev).requires_grad_(True)
        ya = layer(xa)  # feature-major path
        ya.backward(gy)
        grads_a = {k: p.grad.clone() for k, p in layer.named_parameters() if p.grad is not None}
        gxa = xa.grad.clone()
        for p in layer.parameters():
            p.grad = None
        xb = x.to(dev).requires_grad_(True)
        yb = layer._run_nodes(layer.get_mapping(xb))  # row-major path
        assert float((ya != yb).float().mean()) < 1e-3  # same addresses up to selections that sit at 0.5
        yb.backward(gy)
        for k, p in layer.named_parameters():
            if p.grad is None:
                continue
            scale = float(p.grad.abs().max())
            torch.testing.assert_close(grads_a[k], p.grad, rtol=1e-2, atol=1e-2 * scale + 1e-12)
        torch.testing.assert_close(gxa, xb.grad, rtol=1e-2, atol=1e-2 * float(xb.grad.abs().max()))
        if node is DWNNode:
            m = O.learnable_soft_mapping(x, layer.mapping.W.detach().cpu(), layer.tau).view(B, N, 6)
            y_ref = O.dwn_forward(m, layer.luts.detach().cpu()).reshape(B, N * out_dim)
            assert float((ya.cpu() != y_ref).float().mean()) < 1e-3


# ------------------------------------------------------------------------------ GroupSum
def test_groupsum_known_answers(golden, dev):
    from difflut_b200.utils import GroupSum

    g = golden("groupsum")
    x = T(g["x"]).to(dev).requires_grad_(True)
    out = GroupSum(k=4, tau=2.0, use_randperm=False)(x)
    torch.testing.assert_close(out.cpu(), T(g["k4_tau2"]), rtol=1e-6, atol=1e-6)
    out.sum().backward()
    assert torch.allclose(x.grad, torch.full_like(x.grad, 0.5))
    out1 = GroupSum(k=1, tau=1.0, use_randperm=False)(x.detach())
    torch.testing.assert_close(out1.cpu(), T(g["k1_tau1"]), rtol=1e-6, atol=1e-6)
    ones = torch.ones(3, 12, device=dev)
    assert torch.equal(GroupSum(k=4, tau=1.0, use_randperm=False)(ones), torch.full((3, 4), 3.0, device=dev))
    with pytest.raises(ValueError):
        GroupSum(k=2, tau=1.0, use_randperm=False)(torch.ones(3, device=dev))


# ------------------------------------------------------------------------------ fused network
def _build_net3(g, dev, lr=1e-2, fused_backward=True):
    from difflut_b200.encoder import ThermometerEncoder
    from difflut_b200.layers import RandomLayer
    from difflut_b200.network import DWNNetwork
    from difflut_b200.nodes import DWNNode, NodeConfig
    from difflut_b200.utils import GroupSum

    x = T(g["x"])
    k, tau = int(g["k_tau"][0]), float(g["k_tau"][1])
    enc = ThermometerEncoder(num_bits=4).fit(x)
    layers, I = [], x.shape[1] * 4
    for li, N in enumerate(g["sizes"].tolist()):
        l = RandomLayer(I, N, DWNNode, NodeConfig(input_dim=6, output_dim=1), seed=li).to(dev)
        assert torch.equal(l._mapping_indices.cpu(), T(g[f"map{li}"])), "seeded map must equal the reference's"
        with torch.no_grad():
            l.luts.copy_(T(g[f"tables{li}"]).to(dev))
        layers.append(l)
        I = N
    net = DWNNetwork(enc, layers, GroupSum(k=k, tau=tau, use_randperm=False), lr=lr, fused_backward=fused_backward)
    return net, layers, enc


@pytest.mark.parametrize("use_graph,fused", [(False, True), (True, True), (False, False)])
def test_dwn_net3_two_adam_steps_match_reference(golden, dev, use_graph, fused):
    g = golden("dwn_net3")
    net, layers, enc = _build_net3(g, dev, fused_backward=fused)
    x, labels = T(g["x"]).to(dev), T(g["labels"]).to(dev)
    for step in range(2):
        logits = net.logits(x)
        torch.testing.assert_close(logits.cpu(), T(g[f"logits_step{step}"]), rtol=1e-5, atol=1e-5)
        loss = net.train_step(x, labels, use_graph=use_graph)
        torch.testing.assert_close(loss.cpu()[0], T(g[f"loss_step{step}"]), rtol=1e-5, atol=1e-6)
        for li in range(3):
            close_normwise(layers[li].luts.grad.cpu(), T(g[f"gtables{li}_step{step}"]), "layers[li].luts.grad.cpu()")
            torch.testing.assert_close(layers[li].luts.detach().cpu(), T(g[f"tables{li}_after{step}"]), rtol=1e-5, atol=2e-6)
    counts = net.hard_counts(x)
    assert np.array_equal(counts.cpu().numpy(), g["eval_counts"])
    packed = enc.to(dev).encode_packed(x)
    assert torch.equal(net.hard_counts(packed_rows=packed), counts)


def test_graph_on_a_recurring_input_tensor_reads_it_in_place(golden, dev):
    """From its second appearance on, an input tensor gets a graph captured on its own address (no copy into the
    static buffer).  Five graph steps on one tensor whose CONTENT changes between steps must leave the same
    tables, bit for bit, as five eager steps on the same inputs; a fresh tensor afterwards takes the general
    graph again."""
    g = golden("dwn_net3")
    net_a, layers_a, _ = _build_net3(g, dev)
    net_b, layers_b, _ = _build_net3(g, dev)
    x0, labels = T(g["x"]).to(dev), T(g["labels"]).to(dev)
    gen = torch.Generator().manual_seed(7)
    inputs = [x0.clone()] + [torch.rand(x0.shape, generator=gen).to(dev) for _ in range(4)]
    buf = torch.empty_like(x0)
    for step, xi in enumerate(inputs):
        buf.copy_(xi)
        la = net_a.train_step(buf, labels, use_graph=True).clone()
        lb = net_b.train_step(xi, labels, use_graph=False).clone()
        assert torch.equal(la, lb), step
    assert len(net_a._direct_graphs) == 1
    for la_, lb_ in zip(layers_a, layers_b):
        assert torch.equal(la_.luts.detach(), lb_.luts.detach())
    extra = torch.rand(x0.shape, generator=gen).to(dev)
    assert torch.equal(net_a.train_step(extra, labels, use_graph=True), net_b.train_step(extra, labels, use_graph=False))
    assert len(net_a._direct_graphs) == 1


def test_host_pipeline_trains_on_the_batches_in_order(golden, dev):
    """DWNNetwork.host_pipeline: every step() is one graph launch that trains on the batch fetched during the
    previous step and fetches the batch now in the pinned buffers.  Four batches written one step ahead must
    give the same losses and tables, bit for bit, as four train_step calls on the same batches."""
    g = golden("dwn_net3")
    net_a, layers_a, _ = _build_net3(g, dev)
    net_b, layers_b, _ = _build_net3(g, dev)
    x0, labels = T(g["x"]), T(g["labels"]).to(torch.int32)
    gen = torch.Generator().manual_seed(11)
    batches = [x0] + [torch.rand(x0.shape, generator=gen) for _ in range(3)]
    x_pin, y_pin = torch.empty_like(x0).pin_memory(), labels.clone().pin_memory()
    x_pin.copy_(batches[0])
    pipe = net_a.host_pipeline(x_pin, y_pin)
    for k in range(4):
        if k + 1 < len(batches):
            x_pin.copy_(batches[k + 1])  # the next batch goes into the staging buffer before the step that fetches it
        loss = pipe.step()
        torch.cuda.synchronize()
        want = net_b.train_step(batches[k].to(dev), labels.to(dev)).cpu()
        assert torch.equal(loss.clone(), want), k
    for la, lb in zip(layers_a, layers_b):
        assert torch.equal(la.luts.detach(), lb.luts.detach())


def test_layer_api_equals_fused_network(golden, dev):
    """The per-layer fp32 API and the bit-packed executor compute the same logits and table gradients."""
    from difflut_b200.utils import GroupSum

    g = golden("dwn_net3")
    net, layers, enc = _build_net3(g, dev)
    x, labels = T(g["x"]).to(dev), T(g["labels"]).to(dev)
    k, tau = int(g["k_tau"][0]), float(g["k_tau"][1])
    h = enc.to(dev)(x)
    for l in layers:
        l.train()
        l.luts.grad = None
        h = l(h)
    logits = GroupSum(k=k, tau=tau, use_randperm=False)(h)
    torch.testing.assert_close(logits.cpu(), T(g["logits_step0"]), rtol=1e-5, atol=1e-5)
    torch.nn.functional.cross_entropy(logits, labels).backward()
    for li in range(3):
        close_normwise(layers[li].luts.grad.cpu(), T(g[f"gtables{li}_step0"]), "layers[li].luts.grad.cpu()")


def test_full_size_properties(dev):
    """Config-4 shapes (B=8192, 6272 -> 16000 -> 8000 -> 4000): size-independent properties.

    (1) two runs are bit-identical (no atomics anywhere); (2) per node the table gradient sums to
    the sum of the node's output gradient (a checksum of the histogram); (3) the hard path equals
    thresholding the training path's table values for the first layer (bit-sliced LUT vs lookup).
    """
    from difflut_b200 import _native
    from difflut_b200.layers.fused_ops import ConnectionPlan
    from difflut_b200.layers.random_layer import draw_random_mapping

    gen = torch.Generator().manual_seed(0)
    B, I, N = 8192, 6272, 16000
    Bp = _native.padded_batch(B)
    bits_rows = (torch.rand(B, I, generator=gen) > 0.5).float().to(dev)
    bits = torch.empty(I, Bp // 32, device=dev, dtype=torch.int32)
    _native.call("dl_pack_rows_to_t", bits_rows, bits, B, I, Bp, 0.5)
    plan = ConnectionPlan(draw_random_mapping(I, N, 6, 0, True), I, 1, dev)
    tab = torch.randn(N, 64, generator=gen).to(dev)
    g_t = torch.randn(N, Bp, generator=gen).to(dev)
    g_t[:, B:] = 0
    outs = []
    for _ in range(2):
        gt = torch.empty(N, 64, device=dev)
        addr = torch.empty(N, Bp, device=dev, dtype=torch.uint8)
        _native.call("dl_dwn_bwd_tables_t", bits, plan.map_nodes, g_t, 1, 1.0, gt, addr, N, 6, Bp)
        efd = torch.empty(N, 6, 32, device=dev)
        _native.call("dl_dwn_prepare", tab, efd, None, N, 6, 0.1, 1 / 3)
        gx = torch.empty(I, Bp, device=dev)
        _native.call("dl_dwn_bwd_input_t", addr, g_t, 1, 1.0, efd, plan.inv_ptr_virtual, plan.inv_ent8_virtual, gx, I, 6, Bp)
        outs.append((gt, gx, addr))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    torch.testing.assert_close(outs[0][0].sum(1), g_t.sum(1), rtol=1e-3, atol=1e-2)
    vals = torch.empty(N, Bp, device=dev)
    _native.call("dl_dwn_fwd_vals_t", bits, plan.map_nodes, tab, vals, None, N, 6, Bp)
    masks = torch.empty(N, device=dev, dtype=torch.int64)
    _native.call("dl_dwn_prepare", tab, None, masks, N, 6, 0.0, 0.0)
    hard = torch.empty(N, Bp // 32, device=dev, dtype=torch.int32)
    _native.call("dl_dwn_fwd_bits_t", bits, plan.map_nodes, masks, hard, N, 6, Bp)
    hard_rows = torch.empty(B, N, device=dev)
    _native.call("dl_bits_t_to_rows", hard, hard_rows, B, N, Bp)
    assert torch.equal(hard_rows, (vals[:, :B].t() >= 0.5).float())
    # addresses agree with a direct computation on a slice of nodes
    sl = slice(0, 64)
    ref_addr = O.dwn_addresses(O.gather_mapping(bits_rows.cpu(), plan.map_nodes.cpu()[sl]))
    assert torch.equal(outs[0][2][sl, :B].t().cpu().long(), ref_addr)


@pytest.mark.parametrize("B", [4096, 12288, 5000])
def test_bit_sliced_forward_whole_tiles_equals_oracle(dev, B):
    """Batches of one and three whole 4096-sample tiles take the persistent kernel of dl_dwn_fwd_bits_t, the
    ragged one the one-item-per-thread kernel: both against the oracle's eval forward (dwn_node.py:457-483),
    bit for bit, with a node count that is no multiple of the grid's warp count."""
    from difflut_b200 import _native
    from difflut_b200.layers.random_layer import draw_random_mapping

    gen = torch.Generator().manual_seed(B)
    I, N = 100, 777
    Bp = _native.padded_batch(B)
    rows = (torch.rand(B, I, generator=gen) > 0.5).float()
    idx = draw_random_mapping(I, N, 6, 3, True)
    tab = torch.randn(N, 64, generator=gen)
    bits = torch.empty(I, Bp // 32, device=dev, dtype=torch.int32)
    _native.call("dl_pack_rows_to_t", rows.to(dev), bits, B, I, Bp, 0.5)
    masks = torch.empty(N, device=dev, dtype=torch.int64)
    _native.call("dl_dwn_prepare", tab.to(dev), None, masks, N, 6, 0.0, 0.0)
    hard = torch.full((N, Bp // 32), -1, device=dev, dtype=torch.int32)
    _native.call("dl_dwn_fwd_bits_t", bits, idx.to(device=dev, dtype=torch.int32).contiguous(), masks, hard, N, 6, Bp)
    got = torch.empty(B, N, device=dev)
    _native.call("dl_bits_t_to_rows", hard, got, B, N, Bp)
    want = O.dwn_forward_eval(O.gather_mapping(rows, idx), tab.unsqueeze(1)).reshape(B, N)
    assert torch.equal(got.cpu(), want)


def test_error_codes(dev):
    from difflut_b200 import _native

    a = torch.zeros(4, device=dev)
    with pytest.raises(RuntimeError, match="invalid argument"):
        _native.call("dl_f32_rows_to_t", a, a, 1, 4, 100)  # Bp not a multiple of 128
    with pytest.raises(RuntimeError, match="unsupported"):
        _native.call("dl_dwn_prepare", a, a, None, 1, 9, 0.1, 0.3)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        _native.call("dl_f32_rows_to_t", torch.zeros(4), a, 1, 4, 128)


@pytest.mark.parametrize("B,sizes", [
    (2500, [96, 50, 33]),        # ragged tail: general fused kernel; 33 is not a multiple of k
    (2048, [96, 50, 33]),        # whole blocks: pipelined kernel, nodes with 3 and 4 readers (extra-reader path)
    (4096, [6200, 1500, 333]),   # pipelined kernel, first layer with two blocks per item, nodes with 0-2 readers
])
def test_fused_backward_equals_separate_kernels_multi_group(dev, B, sizes):
    """Several 1024-sample groups: the fused per-layer backward (general kernel for a ragged batch, the
    software-pipelined one for whole blocks) and the separate table / input gradient kernels give the same
    table gradients; both match the oracle."""
    from difflut_b200.encoder import ThermometerEncoder
    from difflut_b200.layers import RandomLayer
    from difflut_b200.network import DWNNetwork
    from difflut_b200.nodes import DWNNode, NodeConfig
    from difflut_b200.utils import GroupSum

    gen = torch.Generator().manual_seed(3)
    F, Tb, k, tau = 16, 4, 5, 2.0
    x = torch.rand(B, F, generator=gen)
    labels = torch.randint(0, k, (B,), generator=gen)
    grads = {}
    tabs0 = [torch.randn(N, 1, 64, generator=gen) for N in sizes]
    for fused in (True, False):
        enc = ThermometerEncoder(num_bits=Tb).fit(x)
        layers, I = [], F * Tb
        for li, N in enumerate(sizes):
            l = RandomLayer(I, N, DWNNode, NodeConfig(input_dim=6, output_dim=1), seed=10 + li).to(dev)
            with torch.no_grad():
                l.luts.copy_(tabs0[li].to(dev))
            layers.append(l)
            I = N
        net = DWNNetwork(enc, layers, GroupSum(k=k, tau=tau, use_randperm=False), lr=1e-3, fused_backward=fused)
        net.train_step(x.to(dev), labels.to(dev))
        grads[fused] = [gr.cpu().clone() for gr in net.grads]
        maps = [l._mapping_indices.cpu() for l in layers]
    for li, (a, b) in enumerate(zip(grads[True], grads[False])):
        close_normwise(a, b, f"fused vs separate kernels, table gradient of layer {li + 1}", tol=2e-6)
    bits = O.thermometer_encode(x, O.thermometer_thresholds(x, Tb))
    logits, acts = O.dwn_network_forward(bits, maps, tabs0, k, tau)
    lg = logits.clone().requires_grad_(True)
    torch.nn.functional.cross_entropy(lg, labels).backward()
    ref = O.dwn_network_backward(acts, maps, tabs0, lg.grad, k, tau, 0.5 * 0.75 ** 5, 0.25 / 0.75)
    for li, (a, r) in enumerate(zip(grads[True], ref)):
        close_normwise(a, r, f"fused backward vs oracle, table gradient of layer {li + 1}")


@pytest.mark.parametrize("B,k", [(1024, 10), (2500, 7), (200, 3)])
def test_groupsum_ce_fused_entry_equals_separate_calls(dev, B, k):
    """dl_dwn_fwd_groupsum_ce_s = dl_dwn_fwd_groupsum_s + dl_ce_t, bit for bit (logits, their gradient, per-sample
    losses), with a ragged batch, a class count that does not divide the nodes and an out-of-range label."""
    from difflut_b200 import _native
    from difflut_b200.layers.fused_ops import ConnectionPlan
    from difflut_b200.layers.random_layer import draw_random_mapping

    gen = torch.Generator().manual_seed(B + k)
    I, N, n, tau = 90, 101, 6, 2.5
    Bp = _native.padded_batch(B)
    Ws = int(_native.lib().dl_swizzled_words(Bp))
    x = torch.rand(B, I, generator=gen).to(dev)
    nat = torch.empty(I, Bp // 32, dtype=torch.int32, device=dev)
    _native.call("dl_pack_rows_to_t", x, nat, B, I, Bp, 0.5)
    bits = torch.empty(I, Ws, dtype=torch.int32, device=dev)
    _native.call("dl_bits_swizzle_t", nat, bits, I, Bp)
    plan = ConnectionPlan(draw_random_mapping(I, N, n, 3, True), I, 1, dev)
    tab = torch.randn(N, 64, generator=gen).to(dev)
    labels = torch.randint(0, k, (B,), generator=gen, dtype=torch.int32)
    labels[1] = k + 5  # no such class
    labels = labels.to(dev)
    S = int(_native.lib().dl_dwn_groupsum_splits(N, k))
    outs = []
    for fused in (False, True):
        partial = torch.empty(k * S, Bp, device=dev)
        logits = torch.full((k, Bp), 7.0, device=dev)
        dlog = torch.full((k, Bp), 7.0, device=dev)
        rows = torch.full((Bp,), 7.0, device=dev)
        if fused:
            _native.call("dl_dwn_fwd_groupsum_ce_s", bits, plan.map_nodes, tab, partial, logits, labels, dlog, rows, N, n, k,
                         tau, B, 3 * B, Bp)
        else:
            _native.call("dl_dwn_fwd_groupsum_s", bits, plan.map_nodes, tab, partial, logits, N, n, k, tau, Bp)
            _native.call("dl_ce_t", logits, labels, dlog, rows, None, B, 3 * B, k, Bp)
        outs.append((logits, dlog, rows))
    for a, b in zip(outs[0], outs[1]):
        assert torch.equal(torch.nan_to_num(a, nan=-1.0), torch.nan_to_num(b, nan=-1.0))
    assert bool(torch.isnan(outs[1][2][1])) and not bool(outs[1][1][:, 1].any())  # the bad label: NaN loss, no gradient
    assert not bool(outs[1][1][:, B:].any()) and not bool(outs[1][2][B:].any())  # padding: zeros


@pytest.mark.parametrize("n", [2, 4, 5, 6])
def test_last_layer_groupsum_for_every_node_width_vs_oracle(dev, n):
    """dl_dwn_fwd_groupsum_t / _s for n = 2, 4, 5 (the build of the kernel that reads n at run time) and n = 6
    (the compile-time build), natural and chunk-interleaved bits, ragged batch: logits against the oracle's
    table look-up (difflut/nodes/dwn_node.py:138-165) + GroupSum (difflut/utils/modules.py:116-163)."""
    from difflut_b200 import _native
    from difflut_b200.layers.random_layer import draw_random_mapping

    gen = torch.Generator().manual_seed(40 + n)
    B, I, N, k, tau = 1300, 80, 123, 5, 1.7
    Bp = _native.padded_batch(B)
    x = torch.rand(B, I, generator=gen)
    idx = draw_random_mapping(I, N, n, 2, True)
    tab = torch.randn(N, 1 << n, generator=gen)
    nat = torch.empty(I, Bp // 32, dtype=torch.int32, device=dev)
    _native.call("dl_pack_rows_to_t", x.to(dev), nat, B, I, Bp, 0.5)
    swz = torch.empty(I, int(_native.lib().dl_swizzled_words(Bp)), dtype=torch.int32, device=dev)
    _native.call("dl_bits_swizzle_t", nat, swz, I, Bp)
    xm = O.gather_mapping((x >= 0.5).float(), idx)
    want = O.groupsum(O.dwn_forward(xm, tab.unsqueeze(1)).reshape(B, N), k, tau)
    S = int(_native.lib().dl_dwn_groupsum_splits(N, k))
    mp = idx.to(device=dev, dtype=torch.int32).contiguous()
    for entry, bits in (("dl_dwn_fwd_groupsum_t", nat), ("dl_dwn_fwd_groupsum_s", swz)):
        partial = torch.empty(k * S, Bp, device=dev)
        logits = torch.full((k, Bp), float("nan"), device=dev)
        _native.call(entry, bits, mp, tab.to(dev), partial, logits, N, n, k, tau, Bp)
        torch.testing.assert_close(logits[:, :B].t().cpu(), want, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("B", [128, 1024, 2500])
def test_bits_swizzle_layout(dev, B):
    """Chunk-interleaved layout: bit c + 8r of word w of a 1024-sample block is sample 128c + 4w + r."""
    from difflut_b200 import _native

    gen = torch.Generator().manual_seed(B)
    F = 7
    bits = (torch.rand(B, F, generator=gen) > 0.5).float()
    Bp = _native.padded_batch(B)
    nat = torch.from_numpy(O.pack_bits_feature_major(
        torch.cat([bits, torch.zeros(Bp - B, F)])).view(np.int32)).to(dev)
    Ws = int(_native.lib().dl_swizzled_words(Bp))
    assert Ws == 32 * ((Bp + 1023) // 1024)
    out = torch.full((F, Ws), -1, dtype=torch.int32, device=dev)
    _native.call("dl_bits_swizzle_t", nat, out, F, Bp)
    got = out.cpu().numpy().view(np.uint32)
    padded = np.zeros((Ws * 32, F), dtype=np.uint32)
    padded[:B] = bits.numpy().astype(np.uint32)
    want = np.zeros((F, Ws), dtype=np.uint32)
    for g in range(Ws // 32):
        blk = padded[g * 1024:(g + 1) * 1024].reshape(8, 32, 4, F)  # [c][w][r][f]
        for c in range(8):
            for r in range(4):
                want[:, g * 32:(g + 1) * 32] |= (blk[c, :, r, :].T << np.uint32(c + 8 * r)).astype(np.uint32)
    assert np.array_equal(got, want)
    # the encoder's direct-to-interleaved kernel = natural pack followed by the conversion
    Fx, Tb = 11, 5
    x = torch.rand(B, Fx, generator=gen)
    thr = torch.sort(torch.rand(Fx, Tb, generator=gen), dim=1).values.contiguous()
    nat2 = torch.empty(Fx * Tb, Bp // 32, dtype=torch.int32, device=dev)
    _native.call("dl_thermo_pack_t", x.to(dev), thr.to(dev), nat2, B, Fx, Tb, Bp)
    via = torch.empty(Fx * Tb, Ws, dtype=torch.int32, device=dev)
    _native.call("dl_bits_swizzle_t", nat2, via, Fx * Tb, Bp)
    direct = torch.full((Fx * Tb, Ws), -1, dtype=torch.int32, device=dev)
    _native.call("dl_thermo_pack_s", x.to(dev), thr.to(dev), direct, B, Fx, Tb, Bp)
    assert torch.equal(direct, via)


@pytest.mark.parametrize("B,F", [(1024, 12), (3000, 784), (8192, 296), (8192, 298), (1000, 7)])
def test_thermo_pack_interleaved_all_kernel_variants(dev, B, F):
    """dl_thermo_pack_s picks 16-byte or 4-byte loads (whole quads of features per row or not) and 8 or 4
    features per CTA (large or small grids): every variant = natural pack followed by the layout conversion,
    and the natural pack equals the oracle's bits."""
    from difflut_b200 import _native

    gen = torch.Generator().manual_seed(B + F)
    Tb = 3
    x = torch.rand(B, F, generator=gen)
    thr = torch.sort(torch.rand(F, Tb, generator=gen), dim=1).values.contiguous()
    x[0, :] = thr[:, 0]  # equality with a threshold encodes as 0 (strict comparison)
    # values for which a comparison and a subtraction's sign could disagree if handled carelessly
    thr[0, 0] = -0.0
    x[1, 0], x[2, 0], x[3, 0], x[4, 0] = 0.0, -0.0, float("nan"), float("inf")
    x[5, 0], x[6, 0] = -float("inf"), 1e-42  # a denormal above zero
    Bp = _native.padded_batch(B)
    Ws = int(_native.lib().dl_swizzled_words(Bp))
    nat = torch.empty(F * Tb, Bp // 32, dtype=torch.int32, device=dev)
    _native.call("dl_thermo_pack_t", x.to(dev), thr.to(dev), nat, B, F, Tb, Bp)
    ref = O.pack_bits_feature_major(O.thermometer_encode(x, thr))
    got = nat.cpu().numpy().view(np.uint32)
    assert np.array_equal(got[:, : ref.shape[1]], ref) and not got[:, ref.shape[1]:].any()
    via = torch.empty(F * Tb, Ws, dtype=torch.int32, device=dev)
    _native.call("dl_bits_swizzle_t", nat, via, F * Tb, Bp)
    direct = torch.full((F * Tb, Ws), -1, dtype=torch.int32, device=dev)
    _native.call("dl_thermo_pack_s", x.to(dev), thr.to(dev), direct, B, F, Tb, Bp)
    assert torch.equal(direct, via)


@pytest.mark.parametrize("B,I,N,n", [(70, 300, 1000, 6), (33, 301, 1001, 5), (5, 6272, 2000, 6)])
def test_gather_staged_kernels_vs_oracle(dev, B, I, N, n):
    """`get_mapping` at sizes that take the shared-memory staged gather kernels (wide rows, with and without
    16-byte alignment of the rows): the forward is an exact copy, the backward a segmented sum."""
    from difflut_b200.layers.fused_ops import ConnectionPlan, GatherFunction

    gen = torch.Generator().manual_seed(B + N)
    idx = torch.randint(0, I, (N, n), generator=gen)
    idx[:, 0] = torch.arange(N) % I  # every feature is read at least once when N >= I
    plan = ConnectionPlan(idx, I, 1, dev)
    x = torch.rand(B, I, generator=gen)
    xg = x.to(dev).requires_grad_(True)
    out = GatherFunction.apply(xg, plan)
    assert torch.equal(out.cpu(), O.gather_mapping(x, idx))
    g = torch.randn(B, N, n, generator=gen)
    out.backward(g.to(dev))
    close_normwise(xg.grad.cpu(), O.gather_mapping_backward(g, idx, I), "staged gather backward", tol=2e-6)


# ------------------------------------------------------------------------------ tensor-core GEMM
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 320), (300, 500, 200), (1000, 777, 4096)])
def test_gemm_bf16_tn_matches_fp32_matmul(dev, M, N, K):
    """C = A B^T with bf16 operands, fp32 accumulation: equal to an fp32 matmul of the same bf16 values
    up to summation order (1e-5 relative to the row scale)."""
    from difflut_b200 import _native

    gen = torch.Generator().manual_seed(M + N + K)
    A = torch.randn(M, K, generator=gen).to(dev).to(torch.bfloat16)
    B = torch.randn(N, K, generator=gen).to(dev).to(torch.bfloat16)
    C = torch.full((M, N), float("nan"), device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    _native.call("dl_gemm_bf16_tn", A, B, C, M, N, K, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "a bounded wait inside the kernel ran out"
    ref = A.float() @ B.float().t()
    torch.testing.assert_close(C, ref, rtol=1e-4, atol=1e-4 * float(K) ** 0.5)


def test_gemm_with_packing_epilogue_equals_gemm_then_pack(dev):
    """dl_gemm_bf16_tn_bits thresholds and packs its accumulators in the epilogue: the same bits as
    dl_gemm_bf16_tn followed by dl_pack_t_to_t, on a shape with ragged tiles in both directions and values
    centred on the threshold."""
    from difflut_b200 import _native

    gen = torch.Generator().manual_seed(2)
    M, N, K = 333, 640, 264
    A = (torch.randn(M, K, generator=gen) * 0.05).to(dev).to(torch.bfloat16)
    B = torch.randn(N, K, generator=gen).to(dev).to(torch.bfloat16)
    status = torch.zeros(1, device=dev, dtype=torch.int32)
    C = torch.empty(M, N, device=dev)
    _native.call("dl_gemm_bf16_tn", A, B, C, M, N, K, status)
    want = torch.empty(M, N // 32, device=dev, dtype=torch.int32)
    _native.call("dl_pack_t_to_t", C, want, M, N, N, N, 0.1)
    got = torch.full((M, N // 32), -1, device=dev, dtype=torch.int32)
    _native.call("dl_gemm_bf16_tn_bits", A, B, got, M, N, K, N // 32, 0.1, status)
    assert int(status.item()) == 0
    assert torch.equal(got, want)
    assert 0.2 < float((C >= 0.1).float().mean()) < 0.8  # the threshold cuts through the values


def test_soft_select_matches_fp32_reference(dev):
    from difflut_b200.layers.soft_select import soft_select

    gen = torch.Generator().manual_seed(0)
    B, I, M = 200, 300, 90
    x = torch.rand(B, I, generator=gen).to(dev).requires_grad_(True)
    W = (torch.randn(M, I, generator=gen) * 0.5).to(dev).requires_grad_(True)
    gy = torch.randn(B, M, generator=gen).to(dev)
    for tau in (1.0, 0.3):
        xr = x.detach().clone().requires_grad_(True)
        Wr = W.detach().clone().requires_grad_(True)
        ref = torch.matmul(xr, torch.softmax(Wr / tau, dim=-1).t())
        ref.backward(gy)
        x.grad = W.grad = None
        out = soft_select(x, W, tau)  # three-way split: 16 mantissa bits in the forward
        torch.testing.assert_close(out, ref.detach(), rtol=2e-5, atol=2e-5)
        out.backward(gy)
        torch.testing.assert_close(x.grad, xr.grad, rtol=1e-2, atol=1e-2 * float(xr.grad.abs().max()))
        torch.testing.assert_close(W.grad, Wr.grad, rtol=1e-2, atol=1e-2 * float(Wr.grad.abs().max()))
        plain = soft_select(x.detach(), W.detach(), tau, splits=1)
        torch.testing.assert_close(plain, ref.detach(), rtol=1e-2, atol=1e-2)
    xb = (torch.rand(64, I, generator=gen) > 0.5).float().to(dev)  # binary inputs: two pieces are exact enough
    out2 = soft_select(xb, W.detach(), 1.0, splits=2)
    torch.testing.assert_close(out2, xb @ torch.softmax(W.detach(), -1).t(), rtol=2e-5, atol=2e-5)


def test_input_gradient_for_a_disjoint_map_equals_the_general_kernel(dev):
    """dl_dwn_bwd_input_disjoint_t (one warp per node and 1024 samples, for maps in which every feature has one
    reader) against dl_dwn_bwd_input_t on the identity map: the same bits in fp32, and its bf16 output is the
    fp32 result rounded to nearest.  Ragged last slab (B = 1408 = 11 chunks)."""
    from difflut_b200 import _native
    from difflut_b200.layers.fused_ops import ConnectionPlan

    gen = torch.Generator().manual_seed(21)
    B, N, n = 1408, 333, 6
    I = N * n
    Bp = _native.padded_batch(B)
    plan = ConnectionPlan(torch.arange(I).view(N, n), I, 1, dev)
    tab = torch.randn(N, 64, generator=gen).to(dev)
    efd = torch.empty(N, n, 32, device=dev)
    _native.call("dl_dwn_prepare", tab, efd, None, N, n, 0.1, 1 / 3)
    addr = torch.randint(0, 64, (N, Bp), generator=gen, dtype=torch.uint8).to(dev)
    g_t = torch.randn(N, Bp, generator=gen).to(dev)
    want = torch.empty(I, Bp, device=dev)
    _native.call("dl_dwn_bwd_input_t", addr, g_t, 1, 1.0, efd, plan.inv_ptr_virtual, plan.inv_ent8_virtual, want, I, n, Bp)
    got = torch.full((I, Bp), float("nan"), device=dev)
    _native.call("dl_dwn_bwd_input_disjoint_t", addr, g_t, 1, 1.0, efd, plan.map_virtual, got, 0, N, n, Bp)
    assert torch.equal(got, want)
    got16 = torch.empty(I, Bp, device=dev, dtype=torch.bfloat16)
    _native.call("dl_dwn_bwd_input_disjoint_t", addr, g_t, 1, 1.0, efd, plan.map_virtual, got16, 1, N, n, Bp)
    assert torch.equal(got16, want.to(torch.bfloat16))


def test_gather_backward_with_interleaved_entry_table(dev):
    """dl_gather_rows_bwd_ell (gradient rows staged in shared memory, inverse map interleaved by feature) against
    dl_gather_rows_bwd (CSR): the same bits, and both match the scatter-add of
    difflut/layers/random_layer.py:258-304 computed with index_add in float64.  7001 features: two passes of
    the kernel, the second one ragged; 36000 columns: two column tiles."""
    from difflut_b200 import _native
    from difflut_b200.layers.fused_ops import ConnectionPlan, GatherFunction
    from difflut_b200.layers.random_layer import draw_random_mapping

    gen = torch.Generator().manual_seed(9)
    B, I, N, n = 301, 7001, 6000, 6
    plan = ConnectionPlan(draw_random_mapping(I, N, n, 4, True), I, 1, dev)
    g = torch.randn(B, N * n, generator=gen).to(dev)
    want = torch.full((B, I), float("nan"), device=dev)
    _native.call("dl_gather_rows_bwd", g, plan.inv_ptr_nodes, plan.inv_ent_nodes, want, B, I, N, n)
    ell, max_deg = plan.ell_nodes()
    got = torch.full((B, I), float("nan"), device=dev)
    _native.call("dl_gather_rows_bwd_ell", g, ell, max_deg, got, B, I, N, n)
    assert torch.equal(got, want)
    ref = torch.zeros(B, I, dtype=torch.float64).index_add_(1, plan.map_nodes.cpu().reshape(-1).long(), g.cpu().double())
    torch.testing.assert_close(got.cpu().double(), ref, rtol=1e-5, atol=1e-5)
    # and through autograd (get_mapping's backward picks the interleaved form for rows this wide)
    x = torch.rand(B, I, generator=gen).to(dev).requires_grad_(True)
    GatherFunction.apply(x, plan).backward(g.view(B, N, n))
    assert torch.equal(x.grad, want)


def test_soft_select_centred_single_pass(dev):
    """The centred single-pass form of the soft selection (`splits="centered"`): inside the 1e-2 bar of the
    tensor-core contraction for any weights, and for a near-uniform selection (weights N(0, 0.01), binary
    inputs: the regime of the LearnableLayer benchmark, where the result sits near the nodes' 0.5 threshold)
    within a small factor of the two-piece split's distance to a float64 reference and far closer than plain
    bf16.  Gradients are
    those of the other modes.  Sizes with and without K padding."""
    from difflut_b200.layers.soft_select import soft_select, soft_select_t

    gen = torch.Generator().manual_seed(3)
    for B, I, M in ((256, 1024, 192), (200, 300, 90)):
        xb = (torch.rand(B, I, generator=gen) > 0.5).float()
        W = torch.randn(M, I, generator=gen) * 0.01
        ref = xb.double() @ torch.softmax(W.double(), -1).t()
        err = {}
        for mode in (1, 2, "centered"):
            out = soft_select(xb.to(dev), W.to(dev), 1.0, splits=mode)
            err[mode] = float((out.cpu().double() - ref).abs().max())
        assert err["centered"] <= 1e-5, err            # values are about 0.5 (measured 3e-6; the split 9e-7)
        assert err["centered"] <= 8 * err[2], err
        assert err["centered"] * 20 <= err[1], err     # plain bf16 is more than an order of magnitude worse (2e-4)
        if B % 128 == 0:
            out_t = soft_select_t(xb.to(dev), W.to(dev), 1.0, splits="centered")
            assert torch.equal(out_t.t().contiguous(), soft_select(xb.to(dev), W.to(dev), 1.0, splits="centered"))
    # general inputs and sharp weights: the 1e-2 bar, forward and backward
    B, I, M = 200, 300, 90
    x = torch.rand(B, I, generator=gen).to(dev).requires_grad_(True)
    W = (torch.randn(M, I, generator=gen) * 2.0).to(dev).requires_grad_(True)
    gy = torch.randn(B, M, generator=gen).to(dev)
    xr, Wr = x.detach().clone().requires_grad_(True), W.detach().clone().requires_grad_(True)
    ref = torch.matmul(xr, torch.softmax(Wr / 0.5, dim=-1).t())
    ref.backward(gy)
    out = soft_select(x, W, 0.5, splits="centered")
    torch.testing.assert_close(out, ref.detach(), rtol=1e-2, atol=1e-2)
    out.backward(gy)
    torch.testing.assert_close(x.grad, xr.grad, rtol=1e-2, atol=1e-2 * float(xr.grad.abs().max()))
    torch.testing.assert_close(W.grad, Wr.grad, rtol=1e-2, atol=1e-2 * float(Wr.grad.abs().max()))


def test_wide_materialised_path_equals_fused_layer(dev):
    """(B, N, n) mapped inputs with N >= 64 go through the feature-major kernels under the identity map:
    same outputs and gradients as the fused layer forward, and as the oracle."""
    from difflut_b200.layers import RandomLayer
    from difflut_b200.nodes import DWNNode, NodeConfig

    gen = torch.Generator().manual_seed(11)
    B, I, N = 150, 70, 96
    layer = RandomLayer(I, N, DWNNode, NodeConfig(input_dim=6, output_dim=2), seed=5).to(dev).train()
    tab = torch.randn(N, 2, 64, generator=gen)
    with torch.no_grad():
        layer.luts.copy_(tab.to(dev))
    x = torch.rand(B, I, generator=gen)
    gy = torch.randn(B, N * 2, generator=gen).to(dev)
    xa = x.to(dev).requires_grad_(True)
    ya = layer(xa)
    ya.backward(gy)
    ga, gta = xa.grad.clone(), layer.luts.grad.clone()
    layer.luts.grad = None
    xb = x.to(dev).requires_grad_(True)
    yb = layer._run_nodes(layer.get_mapping(xb))
    assert torch.equal(ya, yb)
    yb.backward(gy)
    torch.testing.assert_close(xb.grad, ga, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(layer.luts.grad, gta, rtol=1e-5, atol=1e-6)
    xm = O.gather_mapping(x, layer._mapping_indices.cpu())
    gxm, gl = O.dwn_backward(xm, tab, gy.cpu().reshape(B, N, 2), layer.alpha, layer.beta)
    torch.testing.assert_close(gta.cpu(), gl, rtol=1e-5, atol=1e-6)
    close_normwise(ga.cpu(), O.gather_mapping_backward(gxm, layer._mapping_indices.cpu(), I), "ga.cpu()")


def test_dwn_stack_equals_sequential_layers(dev):
    """DWNStack(layers) = nn.Sequential(*layers): same outputs and gradients (rows in), also with the
    encoder folded in, in eval mode, and for DWNStable layers."""
    from difflut_b200.encoder import ThermometerEncoder
    from difflut_b200.layers import DWNStack, RandomLayer
    from difflut_b200.nodes import DWNNode, DWNStableNode, NodeConfig

    gen = torch.Generator().manual_seed(5)
    B, F, Tb = 1500, 10, 4
    x = torch.rand(B, F, generator=gen)
    enc = ThermometerEncoder(num_bits=Tb).fit(x).to(dev)
    for node in (DWNNode, DWNStableNode):
        layers, I = [], F * Tb
        for li, N in enumerate((90, 48, 17)):
            l = RandomLayer(I, N, node, NodeConfig(input_dim=6, output_dim=1), seed=li).to(dev)
            with torch.no_grad():
                for p in l.parameters():
                    if p.dim() == 3:
                        p.copy_(torch.randn(p.shape, generator=gen).to(dev))
            layers.append(l)
            I = N
        seq = torch.nn.Sequential(*layers).train()
        stack = DWNStack(layers).train()
        rows = enc(x.to(dev))
        gy = torch.randn(B, 17, generator=gen).to(dev)
        xa = rows.clone().requires_grad_(True)
        ya = seq(xa)
        ya.backward(gy)
        ref = [p.grad.clone() for p in seq.parameters() if p.dim() == 3]
        gxa = xa.grad.clone()
        for p in seq.parameters():
            p.grad = None
        xb = rows.clone().requires_grad_(True)
        yb = stack(xb)
        assert torch.equal(ya, yb)
        yb.backward(gy)
        close_normwise(xb.grad, gxa, "xb.grad")
        for r, p in zip(ref, [p for p in stack.parameters() if p.dim() == 3]):
            close_normwise(p.grad, r, "p.grad")
            p.grad = None
        # encoder folded in: raw features in, same outputs and table gradients
        fused = DWNStack(layers, encoder=enc).train()
        yc = fused(x.to(dev))
        assert torch.equal(yc, ya)
        yc.backward(gy)
        for r, p in zip(ref, [p for p in fused.parameters() if p.dim() == 3]):
            close_normwise(p.grad, r, "p.grad")
        # GroupSum folded in: logits and gradients of GroupSum(Sequential(...)); 17 nodes in 4 classes is ragged
        from difflut_b200.utils import GroupSum

        head = GroupSum(k=4, tau=3.0, use_randperm=False)
        glog = torch.randn(B, 4, generator=gen).to(dev)
        for p in seq.parameters():
            p.grad = None
        xh = rows.clone().requires_grad_(True)
        seq.train()
        ref_logits = head(seq(xh))
        ref_logits.backward(glog)
        ref_h = [p.grad.clone() for p in seq.parameters() if p.dim() == 3]
        for p in seq.parameters():
            p.grad = None
        with_head = DWNStack(layers, groupsum=head).train()
        xi = rows.clone().requires_grad_(True)
        logits = with_head(xi)
        torch.testing.assert_close(logits, ref_logits, rtol=1e-5, atol=1e-5)
        logits.backward(glog)
        close_normwise(xi.grad, xh.grad, "xi.grad")
        for r, p in zip(ref_h, [p for p in with_head.parameters() if p.dim() == 3]):
            close_normwise(p.grad, r, "p.grad")
            p.grad = None
        assert torch.equal(with_head.eval()(rows), head(seq.eval()(rows)))
        # encoder and GroupSum both folded in: raw features in (packed straight into the interleaved layout), logits out
        both = DWNStack(layers, encoder=enc, groupsum=head).train()
        lg2 = both(x.to(dev))
        torch.testing.assert_close(lg2, ref_logits, rtol=1e-5, atol=1e-5)
        lg2.backward(glog)
        for r, p in zip(ref_h, [p for p in both.parameters() if p.dim() == 3]):
            close_normwise(p.grad, r, "p.grad")
            p.grad = None
        assert torch.equal(both.eval()(x.to(dev)), head(seq.eval()(rows)))
        seq.train()
        assert torch.equal(stack.eval()(rows), seq.eval()(rows))
        assert torch.equal(fused.eval()(x.to(dev)), seq(rows))
        assert set(stack.state_dict()) == {"layers." + k for k in seq.state_dict()}
    with pytest.raises(ValueError):
        DWNStack([])


def test_prob_config2_full_size_node_subset_vs_oracle(dev):
    """Config 2 at full size (B=1024, 4096 -> 8000 probabilistic nodes, n=6, GroupSum 10): forward values,
    input gradient contributions and table gradients of a random subset of nodes against the oracle
    (the oracle on all 8000 nodes would hold 2 GB of weights per intermediate)."""
    from difflut_b200.layers import RandomLayer
    from difflut_b200.nodes import NodeConfig, ProbabilisticNode

    gen = torch.Generator().manual_seed(2)
    B, I, N = 1024, 4096, 8000
    x = torch.rand(B, I, generator=gen).clamp(1e-4, 1 - 1e-4)
    layer = RandomLayer(I, N, ProbabilisticNode, NodeConfig(input_dim=6, output_dim=1), seed=0).to(dev).train()
    raw = torch.randn(N, 64, 1, generator=gen)
    with torch.no_grad():
        layer.raw_weights.copy_(raw.to(dev))
    y = layer(x.to(dev))
    gy = torch.randn(B, N, generator=gen)
    y.backward(gy.to(dev))
    pick = torch.randperm(N, generator=gen)[:150]
    idx = layer._mapping_indices.cpu()[pick]
    raw_sub = raw[pick].clone().requires_grad_(True)
    y_ref = O.prob_forward(O.gather_mapping(x, idx), raw_sub).reshape(B, -1)
    torch.testing.assert_close(y.cpu()[:, pick], y_ref, rtol=1e-5, atol=1e-6)
    y_ref.backward(gy[:, pick])
    close_normwise(layer.raw_weights.grad.cpu()[pick], raw_sub.grad, "layer.raw_weights.grad.cpu()[pick]")
    # fused GroupSum: logits = class sums of the same outputs
    logits = layer.forward_groupsum(x.to(dev), 10, 1.0)
    torch.testing.assert_close(logits.cpu(), O.groupsum(y.detach().cpu(), 10, 1.0), rtol=1e-5, atol=1e-3)


def test_learnable_config3_width_node_subset_vs_oracle(dev):
    """Config 3 widths (4096 inputs, 16000 nodes x 6 selections) at batch 256: the soft selection of a random
    subset of nodes against an fp32 softmax + matmul, and their DWN outputs against the oracle."""
    from difflut_b200.layers import LearnableLayer
    from difflut_b200.nodes import DWNNode, NodeConfig

    gen = torch.Generator().manual_seed(4)
    B, I, N = 256, 4096, 16000
    x = torch.bernoulli(torch.full((B, I), 0.5), generator=gen)
    layer = LearnableLayer(I, N, DWNNode, NodeConfig(input_dim=6, output_dim=1)).to(dev).train()
    with torch.no_grad():
        layer.mapping.W.copy_((torch.randn(N * 6, I, generator=gen) * 1.5).to(dev))
    y = layer(x.to(dev))  # feature-major path (batch is a multiple of 128)
    pick = torch.randperm(N, generator=gen)[:200]
    rows = (pick[:, None] * 6 + torch.arange(6)[None, :]).reshape(-1)
    W_sub = layer.mapping.W.detach().cpu()[rows]
    m_ref = O.learnable_soft_mapping(x, W_sub, layer.tau).view(B, len(pick), 6)
    y_ref = O.dwn_forward(m_ref, layer.luts.detach().cpu()[pick]).reshape(B, -1)
    safe = ((m_ref - 0.5).abs() > 1e-3).all(dim=2)  # selections that no rounding can move across 0.5
    assert float(safe.float().mean()) > 0.5  # the comparison below is not vacuous
    assert torch.equal(y.cpu()[:, pick][safe], y_ref[safe])
    m = layer.get_mapping(x.to(dev)).cpu()[:, pick, :]
    torch.testing.assert_close(m, m_ref, rtol=1e-3, atol=1e-4)
