"""Generate the golden fixtures in this directory from the UNMODIFIED reference.

Run where the reference checkout is available:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py [--ref /path/to/difflut/checkout]

It imports the reference package (pure PyTorch, CPU path — the optional CUDA extensions are
absent, which selects exactly the PyTorch implementation that is the parity target), runs
it on seeded inputs and writes small `.npz` files.  The fixtures, not the reference, travel
with the repository; the tests never import the reference.
"""

import argparse
import hashlib
import os
import sys
import warnings

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _np(t):
    return t.detach().cpu().numpy()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("DIFFLUT_REFERENCE", "reference"),
                    help="path of the unmodified difflut checkout (or set DIFFLUT_REFERENCE)")
    args = ap.parse_args()
    sys.path.insert(0, args.ref)
    warnings.filterwarnings("ignore")
    import difflut  # noqa: F401  (registers components)
    from difflut.encoder import ThermometerEncoder
    from difflut.layers import LearnableLayer, RandomLayer
    from difflut.nodes import DWNNode, ProbabilisticNode
    from difflut.nodes.node_config import NodeConfig
    from difflut.nodes.utils.initializers import residual_init
    from difflut.utils.modules import GroupSum

    torch.set_num_threads(4)

    # ---------------------------------------------------------------- thermometer
    out = {}
    for T in (1, 3, 8):
        g = torch.Generator().manual_seed(100 + T)
        x = torch.rand(70, 21, generator=g)
        x[3, 5] = x[:, 5].min()  # exact-equality edge: x == min is below every threshold
        enc = ThermometerEncoder(num_bits=T).fit(x)
        xt = torch.rand(37, 21, generator=g) * 1.2 - 0.1  # some values outside the fitted range
        xt[0] = _as(enc.thresholds[:, 0])  # exact equality with a threshold -> strict '>' gives 0
        out[f"x_fit_T{T}"] = _np(x)
        out[f"x_T{T}"] = _np(xt)
        out[f"thr_T{T}"] = _np(enc.thresholds)
        out[f"bits_T{T}"] = _np(enc.encode(xt)).astype(np.uint8)
    from difflut.encoder import DistributiveThermometerEncoder, GaussianThermometerEncoder

    g = torch.Generator().manual_seed(77)
    xv = torch.randn(90, 13, generator=g) * 2 + 1
    xq = torch.randn(25, 13, generator=g) * 2 + 1
    for tag, cls in (("gauss", GaussianThermometerEncoder), ("distr", DistributiveThermometerEncoder)):
        enc = cls(num_bits=4).fit(xv)
        out[f"{tag}_thr"] = _np(enc.thresholds)
        out[f"{tag}_bits"] = _np(enc.encode(xq)).astype(np.uint8)
    out["variant_x_fit"], out["variant_x"] = _np(xv), _np(xq)
    np.savez_compressed(os.path.join(HERE, "thermometer.npz"), **out)

    # ---------------------------------------------------------------- index maps
    out = {}
    cases = [
        ("c1", 2352, 2000, 6, 0, False),
        ("cov_rem", 50, 23, 6, 7, True),  # cycles + remainder
        ("cov_exact", 48, 16, 6, 3, True),  # exact cycles
        ("small_in", 4, 5, 6, 1, False),  # n > input_size -> with replacement
        ("n4", 100, 30, 4, 42, True),
    ]
    for name, I, N, n, seed, cov in cases:
        layer = RandomLayer(I, N, DWNNode, NodeConfig(input_dim=n, output_dim=1), seed=seed,
                            ensure_full_input_coverage=cov)
        out[name] = _np(layer._mapping_indices)
        out[name + "_args"] = np.array([I, N, n, seed, int(cov)])
    # full-size maps of the 3-layer network: store digests only
    for name, I, N, seed in (("c4_l1", 6272, 16000, 0), ("c4_l2", 16000, 8000, 1), ("c4_l3", 8000, 4000, 2)):
        state = torch.get_rng_state()
        torch.manual_seed(seed)
        total = N * 6
        cycles, rest = divmod(total, I)
        parts = [torch.randperm(I) for _ in range(cycles)]
        if rest:
            parts.append(torch.multinomial(torch.ones(I), num_samples=rest, replacement=False))
        idx = torch.cat(parts).reshape(N, 6).to(torch.int16)
        torch.set_rng_state(state)
        # the lines above are what RandomLayer._init_mapping runs; verify on the real class once
        if name == "c4_l3":
            real = RandomLayer(I, N, DWNNode, NodeConfig(input_dim=6, output_dim=1), seed=seed)
            assert torch.equal(real._mapping_indices, idx)
        out[name + "_sha256"] = np.frombuffer(hashlib.sha256(_np(idx).tobytes()).digest(), dtype=np.uint8)
        out[name + "_head"] = _np(idx[:4])
    np.savez_compressed(os.path.join(HERE, "index_maps.npz"), **out)

    # ---------------------------------------------------------------- DWN layer fwd+bwd
    out = {}
    for tag, B, I, N, n, O, seed in (("n6", 24, 40, 20, 6, 1, 0), ("n4o2", 10, 16, 6, 4, 2, 5), ("n2", 9, 8, 5, 2, 1, 2)):
        g = torch.Generator().manual_seed(seed)
        x = torch.rand(B, I, generator=g, requires_grad=True)
        layer = RandomLayer(I, N, DWNNode, NodeConfig(input_dim=n, output_dim=O), seed=seed,
                            ensure_full_input_coverage=False)
        tables = torch.randn(N, O, 2**n, generator=g)
        with torch.no_grad():
            for j, node in enumerate(layer.nodes):
                node.luts.copy_(tables[j])
        layer.train()
        y = layer(x)
        gy = torch.randn(y.shape, generator=g)
        y.backward(gy)
        out[f"{tag}_x"] = _np(x)
        out[f"{tag}_map"] = _np(layer._mapping_indices)
        out[f"{tag}_tables"] = _np(tables)
        out[f"{tag}_y"] = _np(y)
        out[f"{tag}_gy"] = _np(gy)
        out[f"{tag}_gx"] = _np(x.grad)
        out[f"{tag}_gtables"] = _np(torch.stack([nd.luts.grad for nd in layer.nodes]))
        out[f"{tag}_alpha_beta"] = np.array([layer.nodes[0].alpha.item(), layer.nodes[0].beta.item()], dtype=np.float64)
        layer.eval()
        xb = (x.detach() >= 0.5).float()
        out[f"{tag}_y_eval"] = _np(layer(xb)).astype(np.uint8)
    # residual-init known answer: eval output equals input bit 0 on all 64 patterns
    node = DWNNode(input_dim=6, output_dim=1, init_fn=residual_init, init_kwargs={"node_type": "dwn", "param_name": "luts", "noise_factor": 0.0, "logit_clarity": 5.0})
    out["residual_tables"] = _np(node.luts)
    np.savez_compressed(os.path.join(HERE, "dwn_layer.npz"), **out)

    # ---------------------------------------------------------------- probabilistic layer + GroupSum + CE
    out = {}
    g = torch.Generator().manual_seed(0)
    B, I, N, n, k = 32, 64, 40, 6, 10
    x = torch.rand(B, I, generator=g).clamp(1e-6, 1 - 1e-6).requires_grad_(True)
    layer = RandomLayer(I, N, ProbabilisticNode, NodeConfig(input_dim=n, output_dim=1), seed=0)
    raw = torch.randn(N, 2**n, 1, generator=g)
    with torch.no_grad():
        for j, node in enumerate(layer.nodes):
            node.raw_weights.copy_(raw[j])
    labels = torch.randint(0, k, (B,), generator=g)
    layer.train()
    y = layer(x)
    logits = GroupSum(k=k, tau=1.0, use_randperm=False)(y)
    loss = torch.nn.functional.cross_entropy(logits, labels)
    loss.backward()
    out.update(x=_np(x), map=_np(layer._mapping_indices), raw=_np(raw), labels=_np(labels), y=_np(y),
               logits=_np(logits), loss=_np(loss), gx=_np(x.grad),
               graw=_np(torch.stack([nd.raw_weights.grad for nd in layer.nodes])))
    layer.eval()
    xb = (x.detach() >= 0.5).float()
    out["y_eval"] = _np(layer(xb)).astype(np.uint8)
    # second case: temperature 0.5, out_dim 2, n=3
    g = torch.Generator().manual_seed(1)
    B2, I2, N2, n2, O2 = 12, 10, 7, 3, 2
    x2 = torch.rand(B2, I2, generator=g, requires_grad=True)
    layer2 = RandomLayer(I2, N2, ProbabilisticNode,
                         NodeConfig(input_dim=n2, output_dim=O2, extra_params={"temperature": 0.5}), seed=4)
    raw2 = torch.randn(N2, 2**n2, O2, generator=g)
    with torch.no_grad():
        for j, node in enumerate(layer2.nodes):
            node.raw_weights.copy_(raw2[j])
    layer2.train()
    y2 = layer2(x2)
    gy2 = torch.randn(y2.shape, generator=g)
    y2.backward(gy2)
    out.update(t_x=_np(x2), t_map=_np(layer2._mapping_indices), t_raw=_np(raw2), t_y=_np(y2), t_gy=_np(gy2),
               t_gx=_np(x2.grad), t_graw=_np(torch.stack([nd.raw_weights.grad for nd in layer2.nodes])))
    np.savez_compressed(os.path.join(HERE, "prob_layer.npz"), **out)

    # ---------------------------------------------------------------- learnable layer + DWN
    out = {}
    g = torch.Generator().manual_seed(0)
    B, I, N, n = 16, 32, 8, 6
    x = torch.bernoulli(torch.full((B, I), 0.5), generator=g).requires_grad_(True)
    layer = LearnableLayer(I, N, DWNNode, NodeConfig(input_dim=n, output_dim=1))
    W = torch.randn(N * n, I, generator=g) * 0.5
    tables = torch.randn(N, 1, 2**n, generator=g)
    with torch.no_grad():
        layer.mapping.W.copy_(W)
        for j, node in enumerate(layer.nodes):
            node.luts.copy_(tables[j])
    layer.train()
    m = layer.get_mapping(x)
    y = layer(x)
    gy = torch.randn(y.shape, generator=g)
    y.backward(gy)
    out.update(x=_np(x), W=_np(W), tables=_np(tables), m=_np(m), y=_np(y), gy=_np(gy), gx=_np(x.grad),
               gW=_np(layer.mapping.W.grad), gtables=_np(torch.stack([nd.luts.grad for nd in layer.nodes])),
               tau=np.array([layer.tau]))
    layer.eval()
    out["y_eval"] = _np(layer(x.detach())).astype(np.uint8)
    out["hard_idx"] = _np(layer.get_mapping_matrix())
    layer.update_tau(500)
    out["tau_500"] = np.array([layer.tau])
    np.savez_compressed(os.path.join(HERE, "learnable_layer.npz"), **out)

    # ---------------------------------------------------------------- 3-layer DWN classifier, 2 Adam steps
    out = {}
    g = torch.Generator().manual_seed(0)
    B, Fdim, T, k, tau = 48, 20, 4, 10, 3.0
    sizes = [60, 40, 20]
    x = torch.rand(B, Fdim, generator=g)
    enc = ThermometerEncoder(num_bits=T).fit(x)
    layers, I = [], Fdim * T
    tabs = []
    for li, N in enumerate(sizes):
        layers.append(RandomLayer(I, N, DWNNode, NodeConfig(input_dim=6, output_dim=1), seed=li))
        tabs.append(torch.randn(N, 1, 64, generator=g))
        with torch.no_grad():
            for j, node in enumerate(layers[-1].nodes):
                node.luts.copy_(tabs[-1][j])
        I = N
    labels = torch.randint(0, k, (B,), generator=g)
    gs = GroupSum(k=k, tau=tau, use_randperm=False)
    model = torch.nn.Sequential(*layers)
    opt = torch.optim.Adam(model.parameters(), lr=1e-2)
    out.update(x=_np(x), thr=_np(enc.thresholds), labels=_np(labels), sizes=np.array(sizes), k_tau=np.array([k, tau]))
    for li in range(3):
        out[f"map{li}"] = _np(layers[li]._mapping_indices)
        out[f"tables{li}"] = _np(tabs[li])
    model.train()
    for step in range(2):
        opt.zero_grad()
        bits = enc(x)
        logits = gs(model(bits))
        loss = torch.nn.functional.cross_entropy(logits, labels)
        loss.backward()
        out[f"logits_step{step}"] = _np(logits)
        out[f"loss_step{step}"] = _np(loss)
        for li in range(3):
            out[f"gtables{li}_step{step}"] = _np(torch.stack([nd.luts.grad for nd in layers[li].nodes]))
        opt.step()
        for li in range(3):
            out[f"tables{li}_after{step}"] = _np(torch.stack([nd.luts.data for nd in layers[li].nodes]))
    model.eval()
    with torch.no_grad():
        counts = gs(model(enc(x))) * tau
    out["eval_counts"] = _np(counts.round()).astype(np.int32)
    np.savez_compressed(os.path.join(HERE, "dwn_net3.npz"), **out)

    # ---------------------------------------------------------------- gradient-stabilised DWN layer fwd+bwd
    from difflut.nodes import DWNStableNode

    out = {}
    for tag, B, I, N, n, O, seed, scale in (("n6", 20, 40, 18, 6, 1, 3, 1.25), ("n4o2", 10, 16, 6, 4, 2, 6, 0.7),
                                            ("n3", 9, 8, 5, 3, 1, 8, 2.0)):
        g = torch.Generator().manual_seed(seed)
        x = torch.rand(B, I, generator=g, requires_grad=True)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            layer = RandomLayer(I, N, DWNStableNode,
                                NodeConfig(input_dim=n, output_dim=O, extra_params={"gradient_scale": scale}),
                                seed=seed, ensure_full_input_coverage=False)
        raw = torch.randn(N, O, 2**n, generator=g)
        with torch.no_grad():
            for j, node in enumerate(layer.nodes):
                node.raw_luts.copy_(raw[j])
        layer.train()
        y = layer(x)
        gy = torch.randn(y.shape, generator=g)
        y.backward(gy)
        out[f"{tag}_x"] = _np(x)
        out[f"{tag}_map"] = _np(layer._mapping_indices)
        out[f"{tag}_raw"] = _np(raw)
        out[f"{tag}_scale"] = np.array([scale], dtype=np.float64)
        out[f"{tag}_y"] = _np(y)
        out[f"{tag}_gy"] = _np(gy)
        out[f"{tag}_gx"] = _np(x.grad)
        out[f"{tag}_graw"] = _np(torch.stack([nd.raw_luts.grad for nd in layer.nodes]))
        layer.eval()
        xb = (x.detach() >= 0.5).float()
        out[f"{tag}_y_eval"] = _np(layer(xb)).astype(np.uint8)
    np.savez_compressed(os.path.join(HERE, "dwn_stable_layer.npz"), **out)

    # ---------------------------------------------------------------- hybrid layer fwd+bwd
    from difflut.nodes import HybridNode

    out = {}
    for tag, B, I, N, n, O, seed in (("n6", 20, 40, 18, 6, 1, 4), ("n4o2", 10, 16, 6, 4, 2, 7), ("n2", 9, 8, 5, 2, 1, 9)):
        g = torch.Generator().manual_seed(seed)
        x = torch.rand(B, I, generator=g)
        x[0, : I // 2] = (x[0, : I // 2] >= 0.5).float()  # exactly binary inputs: the input gradient is zero there
        x.requires_grad_(True)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            layer = RandomLayer(I, N, HybridNode, NodeConfig(input_dim=n, output_dim=O), seed=seed,
                                ensure_full_input_coverage=False)
        raw = torch.randn(N, O, 2**n, generator=g)
        with torch.no_grad():
            for j, node in enumerate(layer.nodes):
                node.raw_luts.copy_(raw[j])
        layer.train()
        y = layer(x)
        gy = torch.randn(y.shape, generator=g)
        y.backward(gy)
        out[f"{tag}_x"] = _np(x)
        out[f"{tag}_map"] = _np(layer._mapping_indices)
        out[f"{tag}_raw"] = _np(raw)
        out[f"{tag}_y"] = _np(y)
        out[f"{tag}_gy"] = _np(gy)
        out[f"{tag}_gx"] = _np(x.grad)
        out[f"{tag}_graw"] = _np(torch.stack([nd.raw_luts.grad for nd in layer.nodes]))
        layer.eval()
        xb = (x.detach() >= 0.5).float()
        out[f"{tag}_y_eval"] = _np(layer(xb)).astype(np.uint8)
    np.savez_compressed(os.path.join(HERE, "hybrid_layer.npz"), **out)

    # ---------------------------------------------------------------- convolutional layer fwd+bwd
    from difflut.layers import ConvolutionalLayer, ConvolutionConfig, GroupedInputConfig
    from difflut.nodes import ProbabilisticNode as _Prob

    out = {}
    cases = (
        # tag, node, B, C, H, W, k, stride, pad, trees, depth, n, chunk, grouped, binary input
        ("dwn_d2", DWNNode, 2, 2, 6, 6, 3, 1, 0, 3, 2, 3, 2, False, False),
        ("dwn_s2p1_grouped", DWNNode, 2, 3, 7, 6, 3, 2, 1, 4, 1, 2, 32, True, True),
        ("prob_d2", _Prob, 2, 2, 5, 5, 2, 1, 0, 3, 2, 2, 2, False, False),
    )
    for tag, node_cls, B, C, H, W, k, stride, pad, trees, depth, n, chunk, grouped, binary in cases:
        g = torch.Generator().manual_seed(len(tag))
        x = torch.rand(B, C, H, W, generator=g)
        if binary:
            x = (x >= 0.5).float()
        x.requires_grad_(True)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            conv = ConvolutionalLayer(
                ConvolutionConfig(tree_depth=depth, in_channels=C, out_channels=trees, receptive_field=k,
                                  stride=stride, padding=pad, chunk_size=chunk, seed=7),
                node_cls, NodeConfig(input_dim=n, output_dim=1), RandomLayer, n_inputs_per_node=n,
                grouped_connections=grouped, ensure_full_coverage=grouped)
        levels = [list(conv.first_layer_chunks)] + [[tree[l] for tree in conv.trees] for l in range(depth)]
        pname = "luts" if node_cls is DWNNode else "raw_weights"
        with torch.no_grad():
            for level in levels:
                for layer in level:
                    for node in layer.nodes:
                        getattr(node, pname).copy_(torch.randn(getattr(node, pname).shape, generator=g))
        conv.train()
        y = conv(x)
        gy = torch.randn(y.shape, generator=g)
        y.backward(gy)
        out[f"{tag}_x"] = _np(x)
        out[f"{tag}_y"] = _np(y)
        out[f"{tag}_gy"] = _np(gy)
        out[f"{tag}_gx"] = _np(x.grad)
        out[f"{tag}_cfg"] = np.array([k, stride, pad, trees, depth, n, chunk, int(grouped)], dtype=np.int64)
        for li, level in enumerate(levels):
            out[f"{tag}_map{li}"] = _np(torch.cat([layer._mapping_indices.long() for layer in level]))
            out[f"{tag}_par{li}"] = _np(torch.stack([getattr(nd, pname) for layer in level for nd in layer.nodes]))
            out[f"{tag}_gpar{li}"] = _np(torch.stack([getattr(nd, pname).grad for layer in level for nd in layer.nodes]))
        conv.eval()
        xb = (x.detach() >= 0.5).float()
        out[f"{tag}_y_eval"] = _np(conv(xb)).astype(np.uint8)
    for tag, cover in (("cover", True), ("free", False)):
        gi = GroupedInputConfig(n_groups=3, input_size=27, output_trees=5, luts_per_tree=6, bits_per_node=4,
                                seed=11, ensure_full_coverage=cover)
        out[f"grouped_{tag}"] = _np(gi.mapping_indices)
    np.savez_compressed(os.path.join(HERE, "conv_layer.npz"), **out)

    # ---------------------------------------------------------------- GroupSum known answers
    out = {}
    g = torch.Generator().manual_seed(9)
    xg = torch.randn(5, 23, generator=g)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        out["x"] = _np(xg)
        out["k4_tau2"] = _np(GroupSum(k=4, tau=2.0, use_randperm=False)(xg))  # padded: 23 -> 24
        out["k1_tau1"] = _np(GroupSum(k=1, tau=1.0, use_randperm=False)(xg))
    np.savez_compressed(os.path.join(HERE, "groupsum.npz"), **out)

    # ---------------------------------------------------------------- layer training options (LUTLayerMixin)
    # gradient rescaling (base_layer.py:266-339) on fixed gradients, and the two bit-flip rules
    # (base_layer.py:149-264) under a fixed CPU generator seed
    from difflut.layers import LayerConfig

    out = {}
    g = torch.Generator().manual_seed(21)
    grads = {"small": torch.randn(5, 7, generator=g) * 3.0 + 0.7, "wide": torch.randn(12, 515, generator=g) * 0.02 - 0.01}
    for name, gr in grads.items():
        out[f"g_{name}"] = _np(gr)
    out["rescale_params"] = np.array([2.0, 1e-6])  # target_std, epsilon
    for mode in ("layerwise", "batchwise"):
        for subtract in (False, True):
            layer = RandomLayer(12, 4, DWNNode, NodeConfig(input_dim=3, output_dim=1),
                                layer_config=LayerConfig(grad_stabilization=mode, grad_target_std=2.0,
                                                         grad_subtract_mean=subtract, grad_epsilon=1e-6)).train()
            for name, gr in grads.items():
                out[f"rescaled_{mode}_{int(subtract)}_{name}"] = _np(layer._apply_gradient_stabilization(gr.clone()))
    xf = torch.rand(40, 50, generator=g)
    out["flip_x"] = _np(xf)
    for tag, p in (("sparse", 0.03), ("dense", 0.3)):
        layer = RandomLayer(50, 4, DWNNode, NodeConfig(input_dim=3, output_dim=1),
                            layer_config=LayerConfig(flip_probability=p)).train()
        torch.manual_seed(77)
        out[f"flip_{tag}_out"] = _np(layer._apply_bit_flip(xf.clone()))
        out[f"flip_{tag}_p"] = np.array([p])
    np.savez_compressed(os.path.join(HERE, "layer_options.npz"), **out)
    print("golden fixtures written to", HERE)


def _as(t):
    return t.detach().clone()


if __name__ == "__main__":
    main()
