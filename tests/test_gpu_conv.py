"""GPU parity of the convolutional LUT layer (all through the C ABI): patch kernels against the
oracle's unfold / fold, the layer against fixtures produced by the reference, merged levels against
the reference's sub-layer loop."""

import warnings

import numpy as np
import pytest
import torch

from oracle import difflut_oracle as O

pytestmark = pytest.mark.gpu
warnings.simplefilter("ignore")


def T(a):
    return torch.from_numpy(np.asarray(a))


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda:0")


GEOMS = [
    # B, C, H, W, kh, kw, sh, sw, ph, pw
    (2, 2, 6, 6, 3, 3, 1, 1, 0, 0),
    (3, 1, 9, 7, 3, 2, 2, 1, 1, 0),
    (1, 3, 28, 28, 5, 5, 1, 1, 2, 2),
    (5, 2, 11, 13, 4, 4, 3, 2, 0, 3),
]


@pytest.mark.parametrize("geom", GEOMS)
def test_patch_kernels_match_unfold_and_fold(dev, geom):
    from difflut_b200 import _native
    from difflut_b200.layers.fused_ops import PatchFunction, PatchGeometry

    B, C, H, W, kh, kw, sh, sw, ph, pw = geom
    gen = torch.Generator().manual_seed(sum(geom))
    x = torch.rand(B, C, H, W, generator=gen)
    ref = O.conv_unfold(x, (kh, kw), (sh, sw), (ph, pw))
    pg = PatchGeometry(x.shape, (kh, kw), (sh, sw), (ph, pw))
    assert (pg.S, pg.F) == tuple(ref.shape)
    xg = x.to(dev).requires_grad_(True)
    patches = PatchFunction.apply(xg, pg)
    assert torch.equal(patches.cpu(), ref)  # pure data movement: exact
    gp = torch.randn(ref.shape, generator=gen)
    patches.backward(gp.to(dev))
    gx_ref = O.conv_fold(gp, x.shape, (kh, kw), (sh, sw), (ph, pw))
    torch.testing.assert_close(xg.grad.cpu(), gx_ref, rtol=1e-6, atol=1e-6)
    # bit-packed feature-major patches, padding samples zero
    Bp = _native.padded_batch(pg.S)
    bits = torch.full((pg.F, Bp // 32), -1, device=dev, dtype=torch.int32)
    _native.call("dl_unfold_pack_t", x.to(dev), bits, *pg.args(), 0.5, Bp)
    want = np.zeros((pg.F, Bp), dtype=np.uint8)
    want[:, :pg.S] = (ref >= 0.5).numpy().T
    assert np.array_equal(bits.cpu().numpy().view(np.uint32), O.pack_bits_feature_major(T(want.T.copy())))
    # feature-major adjoint
    gt = torch.zeros(pg.F, Bp, device=dev)
    gt[:, :pg.S] = gp.t().to(dev)
    gx = torch.empty(B, C, H, W, device=dev)
    _native.call("dl_fold_t", gt, gx, *pg.args(), Bp)
    torch.testing.assert_close(gx.cpu(), gx_ref, rtol=1e-6, atol=1e-6)


def _build(g, tag, C, node, dev):
    from difflut_b200.layers import ConvolutionalLayer, ConvolutionConfig, RandomLayer
    from difflut_b200.nodes import NodeConfig

    k, stride, pad, trees, depth, n, chunk, grouped = (int(v) for v in g[f"{tag}_cfg"])
    conv = ConvolutionalLayer(
        ConvolutionConfig(tree_depth=depth, in_channels=C, out_channels=trees, receptive_field=k, stride=stride,
                          padding=pad, chunk_size=chunk, seed=7),
        node, NodeConfig(input_dim=n, output_dim=1), RandomLayer, n_inputs_per_node=n,
        grouped_connections=bool(grouped), ensure_full_coverage=bool(grouped)).to(dev)
    pname = "raw_weights" if "prob" in tag else "luts"
    with torch.no_grad():
        for l, level in enumerate(conv._level_layers()):
            par = T(g[f"{tag}_par{l}"]).to(dev)
            at = 0
            for sub in level:
                p = getattr(sub, pname)
                p.copy_(par[at:at + p.shape[0]].reshape(p.shape))
                at += p.shape[0]
    return conv, depth, pname


def _level_grads(conv, pname):
    return [torch.cat([getattr(s, pname).grad for s in level]) for level in conv._level_layers()]


@pytest.mark.parametrize("tag,C", [("dwn_d2", 2), ("dwn_s2p1_grouped", 3)])
def test_conv_dwn_matches_reference(golden, dev, tag, C):
    from difflut_b200.nodes import DWNNode

    g = golden("conv_layer")
    conv, depth, pname = _build(g, tag, C, DWNNode, dev)
    x = T(g[f"{tag}_x"])
    xg = x.to(dev).requires_grad_(True)
    conv.train()
    y = conv(xg)
    assert torch.equal(y.cpu(), T(g[f"{tag}_y"]))  # table values: exact
    y.backward(T(g[f"{tag}_gy"]).to(dev))
    torch.testing.assert_close(xg.grad.cpu(), T(g[f"{tag}_gx"]), rtol=1e-5, atol=1e-6)
    for l, got in enumerate(_level_grads(conv, pname)):
        torch.testing.assert_close(got.cpu().reshape(g[f"{tag}_gpar{l}"].shape), T(g[f"{tag}_gpar{l}"]),
                                   rtol=1e-5, atol=1e-6)
    conv.eval()
    ye = conv((x >= 0.5).float().to(dev))
    assert np.array_equal(ye.cpu().numpy().astype(np.uint8), g[f"{tag}_y_eval"])
    # the reference's own schedule (loop over sub-layers on materialised patches) gives the same numbers
    from difflut_b200.layers.fused_ops import PatchFunction, PatchGeometry

    conv.train()
    for p in conv.parameters():
        p.grad = None
    xg2 = x.to(dev).requires_grad_(True)
    pg = PatchGeometry(x.shape, conv.receptive_field, conv.stride, conv.padding)
    rows = conv._forward_loop(PatchFunction.apply(xg2, pg))
    y2 = rows.view(pg.B, pg.P, -1).transpose(1, 2).reshape(y.shape)
    assert torch.equal(y2, y)
    y2.backward(T(g[f"{tag}_gy"]).to(dev))
    torch.testing.assert_close(xg2.grad.cpu(), T(g[f"{tag}_gx"]), rtol=1e-5, atol=1e-6)
    # bit-flip augmentation takes the materialised-patch route and still trains
    conv.flip_probability = 0.3
    y3 = conv(x.to(dev))
    assert y3.shape == y.shape and torch.isfinite(y3).all()


def test_conv_prob_matches_reference(golden, dev):
    from difflut_b200.nodes import ProbabilisticNode

    g = golden("conv_layer")
    tag = "prob_d2"
    conv, depth, pname = _build(g, tag, 2, ProbabilisticNode, dev)
    xg = T(g[f"{tag}_x"]).to(dev).requires_grad_(True)
    y = conv.train()(xg)
    torch.testing.assert_close(y.cpu(), T(g[f"{tag}_y"]), rtol=1e-5, atol=1e-6)
    y.backward(T(g[f"{tag}_gy"]).to(dev))
    torch.testing.assert_close(xg.grad.cpu(), T(g[f"{tag}_gx"]), rtol=1e-5, atol=1e-6)
    for l, got in enumerate(_level_grads(conv, pname)):
        torch.testing.assert_close(got.cpu().reshape(g[f"{tag}_gpar{l}"].shape), T(g[f"{tag}_gpar{l}"]),
                                   rtol=1e-5, atol=1e-6)
    ye = conv.eval()((T(g[f"{tag}_x"]) >= 0.5).float().to(dev))
    assert np.array_equal(ye.cpu().numpy().astype(np.uint8), g[f"{tag}_y_eval"])


@pytest.mark.parametrize("kind", ["dwn_stable", "hybrid"])
def test_conv_other_stacked_nodes_vs_sub_layer_loop(dev, kind):
    """Merged levels of DWNStable / Hybrid trees equal the loop over the (separately verified) sub-layers."""
    from difflut_b200.layers import ConvolutionalLayer, ConvolutionConfig, RandomLayer
    from difflut_b200.layers.fused_ops import PatchFunction, PatchGeometry
    from difflut_b200.nodes import DWNStableNode, HybridNode, NodeConfig

    node = DWNStableNode if kind == "dwn_stable" else HybridNode
    torch.manual_seed(3)
    conv = ConvolutionalLayer(ConvolutionConfig(tree_depth=2, in_channels=3, out_channels=5, receptive_field=3,
                                                stride=1, padding=1, chunk_size=2),
                              node, NodeConfig(input_dim=3, output_dim=1), RandomLayer, n_inputs_per_node=3).to(dev)
    with torch.no_grad():
        for p in conv.parameters():
            if p.dim() == 3:
                p.copy_(torch.randn_like(p))
    x = torch.rand(4, 3, 8, 8, device=dev)
    gy = torch.randn(4, 5, 8, 8, device=dev)
    xa = x.clone().requires_grad_(True)
    ya = conv.train()(xa)
    ya.backward(gy)
    grads_a = [p.grad.clone() for p in conv.parameters() if p.dim() == 3]
    for p in conv.parameters():
        p.grad = None
    xb = x.clone().requires_grad_(True)
    pg = PatchGeometry(x.shape, conv.receptive_field, conv.stride, conv.padding)
    rows = conv._forward_loop(PatchFunction.apply(xb, pg))
    yb = rows.view(pg.B, pg.P, -1).transpose(1, 2).reshape(ya.shape)
    assert torch.equal(ya, yb)
    yb.backward(gy)
    torch.testing.assert_close(xa.grad, xb.grad, rtol=1e-5, atol=1e-6)
    for ga, p in zip(grads_a, [p for p in conv.parameters() if p.dim() == 3]):
        torch.testing.assert_close(ga, p.grad, rtol=1e-5, atol=1e-6)
    conv.eval()
    xb01 = (x >= 0.5).float()
    ye = conv(xb01)
    rows_e = conv._forward_loop(PatchFunction.apply(xb01, pg))
    assert torch.equal(ye, rows_e.view(pg.B, pg.P, -1).transpose(1, 2).reshape(ye.shape))


def test_conv_full_size_properties(dev):
    """28x28 single-channel images, 3-bit thermometer planes, 5x5 receptive field, 16 trees of depth 2,
    batch 64: determinism, eval = thresholded training output, gradient reaches every table."""
    from difflut_b200.layers import ConvolutionalLayer, ConvolutionConfig, RandomLayer
    from difflut_b200.nodes import DWNNode, NodeConfig

    conv = ConvolutionalLayer(ConvolutionConfig(tree_depth=2, in_channels=3, out_channels=16, receptive_field=5,
                                                chunk_size=8),
                              DWNNode, NodeConfig(input_dim=6, output_dim=1), RandomLayer).to(dev)
    gen = torch.Generator().manual_seed(0)
    x = (torch.rand(64, 3, 28, 28, generator=gen) > 0.5).float().to(dev)
    y1 = conv.train()(x)
    y2 = conv(x)
    assert y1.shape == (64, 16, 24, 24) and torch.equal(y1, y2)
    assert torch.equal(conv.eval()(x), (y1 >= 0.5).float())
    conv.train()
    y1.sum().backward()
    for p in conv.parameters():
        assert p.grad is not None and float(p.grad.abs().sum()) > 0
    total = sum(float(p.grad.sum()) for p in conv.trees[0][1].parameters())
    assert total == pytest.approx(64 * 24 * 24, rel=1e-6)  # the root node's histogram counts every patch once


def test_flip_kernels_and_fused_conv_flip(dev):
    """Bit-flip augmentation: Bernoulli rate, determinism in the seed, identical decisions on fp32 and on
    packed bits, identity gradient; a convolution with DWN trees flips packed patch bits (no patches)."""
    from difflut_b200 import _native
    from difflut_b200.layers import ConvolutionalLayer, ConvolutionConfig, LayerConfig, RandomLayer
    from difflut_b200.layers.base_layer import _FlipFunction
    from difflut_b200.nodes import DWNNode, NodeConfig

    F, B = 37, 1000
    gen = torch.Generator().manual_seed(1)
    xt = (torch.rand(F, B, generator=gen) > 0.5).float().to(dev)  # feature-major {0,1}
    out = torch.empty_like(xt)
    _native.call("dl_flip_rows", xt, out, xt.numel(), 0.25, 1234)
    flipped = out != xt
    assert abs(float(flipped.float().mean()) - 0.25) < 0.01
    assert torch.equal(out[flipped], 1.0 - xt[flipped])
    out2 = torch.empty_like(xt)
    _native.call("dl_flip_rows", xt, out2, xt.numel(), 0.25, 1234)
    assert torch.equal(out, out2)
    _native.call("dl_flip_rows", xt, out2, xt.numel(), 0.25, 1235)
    assert not torch.equal(out, out2)
    # the packed variant flips the same elements
    Bp = _native.padded_batch(B)
    bits = torch.from_numpy(O.pack_bits_feature_major(
        torch.cat([xt.t().cpu(), torch.zeros(Bp - B, F)])).view(np.int32)).to(dev)
    _native.call("dl_bits_flip_t", bits, F, B, Bp, 0.25, 1234)
    want = O.pack_bits_feature_major(torch.cat([out.t().cpu(), torch.zeros(Bp - B, F)]))
    assert np.array_equal(bits.cpu().numpy().view(np.uint32), want)
    # identity gradient
    xr = torch.rand(50, 20, device=dev, requires_grad=True)
    y = _FlipFunction.apply(xr, 0.5, 7)
    y.backward(torch.ones_like(y))
    assert torch.equal(xr.grad, torch.ones_like(xr))
    # convolution: flips change the output, are reproducible under torch.manual_seed, gradients flow
    conv = ConvolutionalLayer(ConvolutionConfig(tree_depth=1, in_channels=2, out_channels=4, receptive_field=3),
                              DWNNode, NodeConfig(input_dim=6, output_dim=1), RandomLayer,
                              layer_config=LayerConfig(flip_probability=0.3)).to(dev).train()
    x = (torch.rand(8, 2, 10, 10, generator=gen) > 0.5).float().to(dev).requires_grad_(True)
    torch.manual_seed(5)
    y1 = conv(x)
    torch.manual_seed(5)
    y2 = conv(x)
    assert torch.equal(y1, y2)
    y3 = conv(x)
    assert not torch.equal(y1, y3)
    conv.flip_probability = 0.0
    y0 = conv(x)
    assert not torch.equal(y0, y1)
    y1.sum().backward()
    assert x.grad is not None and float(x.grad.abs().sum()) > 0
    assert torch.equal(conv.eval()(x), conv(x))  # no flips in eval


@pytest.mark.parametrize("mode", ["layerwise", "batchwise"])
@pytest.mark.parametrize("subtract", [False, True])
def test_gradient_rescale_matches_reference(golden, dev, mode, subtract):
    """dl_grad_rescale against outputs of the reference's _apply_gradient_stabilization
    (difflut/layers/base_layer.py:266-339) and, on larger shapes, against the oracle's restatement of it."""
    from difflut_b200.layers import LayerConfig, RandomLayer
    from difflut_b200.nodes import DWNNode, NodeConfig

    fx = golden("layer_options")
    target, eps = (float(v) for v in fx["rescale_params"])
    layer = RandomLayer(12, 4, DWNNode, NodeConfig(input_dim=3, output_dim=1),
                        layer_config=LayerConfig(grad_stabilization=mode, grad_target_std=target,
                                                 grad_subtract_mean=subtract, grad_epsilon=eps)).train()
    for name in ("small", "wide"):
        got = layer._apply_gradient_stabilization(T(fx[f"g_{name}"]).to(dev))
        torch.testing.assert_close(got.cpu(), T(fx[f"rescaled_{mode}_{int(subtract)}_{name}"]), rtol=1e-5, atol=1e-7)
    gen = torch.Generator().manual_seed(3)
    for shape in ((300, 1000), (64, 4097)):
        g = torch.randn(shape, generator=gen) * 3.0 + 0.7
        ref = O.grad_rescale(g, mode, target, subtract, eps)
        got = layer._apply_gradient_stabilization(g.to(dev))
        torch.testing.assert_close(got.cpu(), ref, rtol=1e-5, atol=1e-6)
    layer.eval()
    assert layer._apply_gradient_stabilization(g.to(dev)) is not None


def test_exact_count_flip_below_five_percent(dev):
    """Below p = 0.05 the reference flips exactly int(numel * p) distinct positions, the head of a random
    permutation drawn on the tensor's device (difflut/layers/base_layer.py:226-262): the layer draws the same
    permutation from torch's CUDA generator, so the flipped positions can be re-derived from the seed."""
    from difflut_b200 import _native
    from difflut_b200.layers import LayerConfig, RandomLayer
    from difflut_b200.nodes import DWNNode, NodeConfig

    gen = torch.Generator().manual_seed(5)
    x = torch.rand(300, 77, generator=gen).to(dev)
    p = 0.03
    layer = RandomLayer(77, 4, DWNNode, NodeConfig(input_dim=3, output_dim=1),
                        layer_config=LayerConfig(flip_probability=p)).to(dev).train()
    torch.manual_seed(123)
    xg = x.clone().requires_grad_(True)
    out = layer._apply_bit_flip(xg)
    torch.manual_seed(123)
    want = torch.randperm(x.numel(), device=dev)[: int(x.numel() * p)]
    assert torch.equal(out.detach().cpu(), O.flip_apply(x.cpu(), want.cpu()))
    assert int((out.detach() != x).sum()) == int(x.numel() * p)
    out.sum().backward()
    assert torch.equal(xg.grad, torch.ones_like(x))  # the flip carries no gradient
    # too few elements for a single flip: the input comes back untouched
    tiny = torch.rand(2, 7, device=dev)
    assert layer._apply_bit_flip(tiny) is tiny
    # packed variant: the same positions of the row-major (B, F) matrix, applied to feature-major bits
    B, F = 300, 77
    Bp = _native.padded_batch(B)
    bits = torch.empty(F, Bp // 32, dtype=torch.int32, device=dev)
    _native.call("dl_pack_rows_to_t", x, bits, B, F, Bp, 0.5)
    _native.call("dl_bits_flip_at_t", bits, want, want.numel(), F, B, Bp)
    ref_bits = torch.empty_like(bits)
    _native.call("dl_pack_rows_to_t", out.detach().contiguous(), ref_bits, B, F, Bp, 0.5)
    assert torch.equal(bits, ref_bits)
