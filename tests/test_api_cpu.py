"""Host-side behaviour of the reference-compatible API (no GPU): registry, configs, validation,
index maps, stacked layers with node views, reference-format state dicts."""

import hashlib
import warnings

import numpy as np
import pytest
import torch

warnings.simplefilter("ignore")

import difflut_b200 as difflut  # noqa: E402
from difflut_b200.encoder import ThermometerEncoder  # noqa: E402
from difflut_b200.layers import LayerConfig, LearnableLayer, RandomLayer  # noqa: E402
from difflut_b200.nodes import DWNNode, NodeConfig, ProbabilisticNode  # noqa: E402
from difflut_b200.utils import GroupSum  # noqa: E402
from difflut_b200.utils.warnings import DefaultValueWarning  # noqa: E402


def test_registry_names_and_errors():
    R = difflut.REGISTRY
    assert R.get_node("dwn") is DWNNode and R.get_node("probabilistic") is ProbabilisticNode
    assert R.get_layer("random") is RandomLayer and R.get_layer("learnable") is LearnableLayer
    assert R.get_encoder("thermometer") is ThermometerEncoder
    with pytest.raises(ValueError, match="not found"):
        R.get_node("nope")
    with pytest.raises(ValueError):
        R.get_initializer("nope")
    assert set(R.list_all()) == {"nodes", "layers", "convolutional_layers", "encoders", "initializers", "regularizers"}


def test_registry_decorators_and_suffix_aliases():
    R = difflut.registry.Registry()

    @R.register_initializer()
    def my_init(param, **kw):
        param.fill_(1.0)

    @R.register_regularizer("L2_regularizer")
    def l2(node):
        return node.luts.pow(2).sum()

    assert R.get_initializer("my") is my_init and R.get_initializer("MY_INIT") is my_init
    assert R.get_regularizer("l2") is l2
    with pytest.warns(UserWarning):
        R.register_node("x")(int)
        R.register_node("x")(float)
    assert R.build_node("x") == 0.0


def test_node_config_to_dict():
    cfg = NodeConfig(input_dim=6, output_dim=1, extra_params={"alpha": 0.1})
    assert cfg.to_dict() == {"input_dim": 6, "output_dim": 1, "alpha": 0.1}
    c2 = cfg.copy()
    c2.extra_params["alpha"] = 0.2
    assert cfg.extra_params["alpha"] == 0.1


def test_layer_config_validation():
    with pytest.raises(ValueError):
        LayerConfig(flip_probability=1.5)
    with pytest.raises(ValueError):
        LayerConfig(grad_stabilization="bogus")
    with pytest.raises(TypeError):
        RandomLayer(10, 4, DWNNode, NodeConfig(input_dim=2, output_dim=1), layer_config={"flip_probability": 0.1})
    assert "default" in repr(LayerConfig())


def test_validation_errors_match_reference_types():
    with pytest.raises(ValueError):
        RandomLayer(0, 4, DWNNode, NodeConfig(input_dim=2, output_dim=1))
    with pytest.raises(ValueError):
        RandomLayer(10, -1, DWNNode, NodeConfig(input_dim=2, output_dim=1))
    with pytest.raises(ValueError):
        DWNNode(input_dim=0, output_dim=1)
    with pytest.raises(TypeError):
        DWNNode(input_dim=2, output_dim=1, init_fn="not callable")
    with pytest.raises(ValueError):
        GroupSum(k=0, tau=1.0, use_randperm=False)
    with pytest.raises(ValueError):
        GroupSum(k=2, tau=-1.0, use_randperm=False)
    layer = RandomLayer(10, 4, DWNNode, NodeConfig(input_dim=2, output_dim=1))
    with pytest.raises(ValueError):
        layer(torch.zeros(3, 11))
    with pytest.raises(ValueError):
        layer(torch.zeros(3, 10, 1))
    with pytest.raises(ValueError):
        layer(torch.zeros(0, 10))
    with pytest.raises(RuntimeError, match="CUDA"):
        layer(torch.zeros(3, 10))  # valid shape, but there is no CPU path
    with pytest.raises(RuntimeError):
        ThermometerEncoder(num_bits=2).encode(torch.zeros(2, 2))


def test_default_value_warnings():
    with pytest.warns(DefaultValueWarning):
        DWNNode(input_dim=3, output_dim=1)  # alpha / beta defaults
    with pytest.warns(DefaultValueWarning):
        GroupSum()


def test_index_maps_equal_reference(golden):
    g = golden("index_maps")
    for name in ("c1", "cov_rem", "cov_exact", "small_in", "n4"):
        I, N, n, seed, cov = (int(v) for v in g[name + "_args"])
        from difflut_b200.layers.random_layer import draw_random_mapping

        before = torch.get_rng_state()
        draw_random_mapping(I, N, n, seed, bool(cov))
        assert torch.equal(before, torch.get_rng_state()), "drawing the map must not disturb the global RNG"
        layer = RandomLayer(I, N, DWNNode, NodeConfig(input_dim=n, output_dim=1), seed=seed,
                            ensure_full_input_coverage=bool(cov))
        assert np.array_equal(layer._mapping_indices.numpy(), g[name])
        assert layer.get_mapping_matrix().dtype == torch.int64
    for name, I, N, seed in (("c4_l1", 6272, 16000, 0), ("c4_l2", 16000, 8000, 1), ("c4_l3", 8000, 4000, 2)):
        layer = RandomLayer(I, N, DWNNode, NodeConfig(input_dim=6, output_dim=1), seed=seed)
        digest = np.frombuffer(hashlib.sha256(layer._mapping_indices.numpy().tobytes()).digest(), dtype=np.uint8)
        assert np.array_equal(digest, g[name + "_sha256"])
    given = torch.arange(12).reshape(3, 4)
    layer = RandomLayer(20, 3, DWNNode, NodeConfig(input_dim=4, output_dim=1), mapping_indices=given)
    assert torch.equal(layer._mapping_indices.long(), given) and layer._mapping_indices.dtype == torch.int16


def test_stacked_layer_structure_and_node_views():
    calls = []

    def init_fn(param, **kw):
        calls.append((tuple(param.shape), kw.get("input_dim")))
        param.fill_(0.25)

    layer = RandomLayer(40, 7, DWNNode, NodeConfig(input_dim=4, output_dim=2, init_fn=init_fn), seed=1)
    assert layer.n == 4 and layer.output_dim_per_node == 2 and layer.output_size == 7
    assert len(calls) == 7 and calls[0] == ((2, 16), 4)  # per node, reference-shaped, input_dim injected
    assert layer.luts.shape == (7, 2, 16) and bool((layer.luts == 0.25).all())
    assert len(layer.nodes) == 7
    node = layer.nodes[3]
    assert isinstance(node, DWNNode) and node.luts.shape == (2, 16) and node.num_inputs == 4 and node.output_dim == 2
    with torch.no_grad():
        node.luts.fill_(2.0)  # a view: the layer sees the edit
    assert bool((layer.luts[3] == 2.0).all()) and bool((layer.luts[2] == 0.25).all())
    assert [nd.input_dim for nd in layer.nodes][:2] == [4, 4] and len(layer.nodes[-2:]) == 2
    names = [n for n, _ in layer.named_parameters()]
    assert names == ["luts"]
    assert float(layer.regularization()) == 0.0
    reg_layer = RandomLayer(40, 3, DWNNode, NodeConfig(input_dim=4, output_dim=1,
                            regularizers={"l2": [lambda nd: nd.luts.pow(2).sum(), 0.5, {}]}), seed=1)
    assert float(reg_layer.regularization()) == pytest.approx(0.5 * float(reg_layer.luts.pow(2).sum()), rel=1e-5)
    p = RandomLayer(40, 5, ProbabilisticNode, NodeConfig(input_dim=3, output_dim=2, extra_params={"temperature": 0.5}))
    assert p.raw_weights.shape == (5, 8, 2) and p.nodes[0].raw_weights.shape == (8, 2)
    assert float(p.nodes[0].temperature) == 0.5 and p.nodes[0].binary_combinations.shape == (8, 3)


def test_state_dict_uses_reference_keys_and_round_trips():
    layer = RandomLayer(30, 4, DWNNode, NodeConfig(input_dim=3, output_dim=1), seed=2)
    sd = layer.state_dict()
    assert set(sd) == {"_mapping_indices"} | {f"nodes.{i}.{k}" for i in range(4) for k in ("luts", "alpha", "beta")}
    assert sd["nodes.2.luts"].shape == (1, 8) and sd["_mapping_indices"].dtype == torch.int16
    other = RandomLayer(30, 4, DWNNode, NodeConfig(input_dim=3, output_dim=1), seed=9)
    other.load_state_dict(sd)
    assert torch.equal(other.luts, layer.luts) and torch.equal(other._mapping_indices, layer._mapping_indices)
    # the stacked layout loads too
    third = RandomLayer(30, 4, DWNNode, NodeConfig(input_dim=3, output_dim=1), seed=9)
    third.load_state_dict({"_mapping_indices": layer._mapping_indices, "luts": layer.luts.detach()})
    assert torch.equal(third.luts, layer.luts)
    p = RandomLayer(30, 2, ProbabilisticNode, NodeConfig(input_dim=3, output_dim=1), seed=2)
    psd = p.state_dict()
    assert {"nodes.0.raw_weights", "nodes.1.temperature", "nodes.0.binary_combinations"} <= set(psd)
    q = RandomLayer(30, 2, ProbabilisticNode, NodeConfig(input_dim=3, output_dim=1), seed=2)
    q.load_state_dict(psd)
    assert torch.equal(q.raw_weights, p.raw_weights)


def test_learnable_layer_host_logic():
    layer = LearnableLayer(16, 3, DWNNode, NodeConfig(input_dim=2, output_dim=1), tau=0.5, tau_start=1.0,
                           tau_min=0.01, tau_decay_iters=100.0, use_cuda_soft=False)
    assert layer.tau == 1.0 and layer.mapping.W.shape == (6, 16)  # tau argument is ignored, as in the reference
    layer.update_tau(100)
    assert layer.tau == pytest.approx(0.1) and layer.mapping.tau == layer.tau
    layer.update_tau(10_000)
    assert layer.tau == 0.01
    assert layer.get_mapping_matrix().shape == (3, 2)
    layer.eval()
    idx = layer.mapping.hard_indices()
    assert torch.equal(idx.long(), torch.argmax(layer.mapping.W, -1))
    layer.train()
    assert layer.mapping._cache_valid is False


def test_thermometer_fit_host_side(golden):
    g = golden("thermometer")
    enc = ThermometerEncoder(num_bits=3)
    assert not enc.is_fitted
    assert enc.fit(torch.from_numpy(g["x_fit_T3"])) is enc and enc.is_fitted
    assert torch.equal(enc.thresholds, torch.from_numpy(g["thr_T3"]))
    assert "thresholds" not in enc.state_dict()
    assert torch.equal(enc.get_thresholds(torch.from_numpy(g["x_fit_T3"])), enc.thresholds)
    assert repr(enc) == "ThermometerEncoder(num_bits=3, flatten=True)"


def test_mixin_helpers_on_cpu():
    layer = RandomLayer(8, 2, DWNNode, NodeConfig(input_dim=2, output_dim=1),
                        layer_config=LayerConfig(flip_probability=0.5, grad_stabilization="layerwise"))
    x = torch.zeros(64, 8)
    flipped = layer._apply_bit_flip(x)
    assert 0 < float(flipped.mean()) < 1 and set(flipped.unique().tolist()) <= {0.0, 1.0}
    g = torch.randn(16, 2) * 10
    out = layer._apply_gradient_stabilization(g)
    assert float(out.pow(2).mean()) == pytest.approx(1.0, rel=1e-3)
    layer.eval()
    assert layer._apply_bit_flip(x) is x


def test_thermometer_fit_variants_match_reference(golden):
    from difflut_b200.encoder import DistributiveThermometerEncoder, GaussianThermometerEncoder

    g = golden("thermometer")
    x = torch.from_numpy(g["variant_x_fit"])
    for tag, cls in (("gauss", GaussianThermometerEncoder), ("distr", DistributiveThermometerEncoder)):
        enc = cls(num_bits=4).fit(x)
        assert torch.equal(enc.thresholds, torch.from_numpy(g[f"{tag}_thr"]))
    assert difflut.REGISTRY.get_encoder("gaussian_thermometer") is GaussianThermometerEncoder
    assert difflut.REGISTRY.get_encoder("distributive_thermometer") is DistributiveThermometerEncoder


def test_new_node_types_registered_and_stacked():
    from difflut_b200.nodes import DWNStableNode, HybridNode

    R = difflut.REGISTRY
    assert R.get_node("dwn_stable") is DWNStableNode and R.get_node("hybrid") is HybridNode
    stable = RandomLayer(12, 5, DWNStableNode, NodeConfig(input_dim=3, output_dim=2,
                                                          extra_params={"gradient_scale": 0.8}), seed=1)
    assert stable.raw_luts.shape == (5, 2, 8) and stable.gradient_scale.shape == (5,)
    assert float(stable.gradient_scale[3]) == pytest.approx(0.8)
    assert stable.nodes[2].raw_luts.shape == (2, 8)
    sd = stable.state_dict()
    assert {"nodes.4.raw_luts", "nodes.4.gradient_scale", "_mapping_indices"} <= set(sd)
    assert "raw_luts" not in sd and "gradient_scale" not in sd
    other = RandomLayer(12, 5, DWNStableNode, NodeConfig(input_dim=3, output_dim=2), seed=1)
    other.load_state_dict(sd)
    assert torch.equal(other.raw_luts, stable.raw_luts) and torch.equal(other.gradient_scale, stable.gradient_scale)
    hybrid = RandomLayer(12, 5, HybridNode, NodeConfig(input_dim=3, output_dim=1), seed=1)
    assert hybrid.raw_luts.shape == (5, 1, 8)
    assert hybrid.nodes[0].binary_combinations.tolist()[3] == [1.0, 1.0, 0.0]
    assert "nodes.0.binary_combinations" in hybrid.state_dict()
    for cls in (DWNStableNode, HybridNode):
        with pytest.raises(ValueError):
            cls(input_dim=17, output_dim=1)
        assert cls(input_dim=9, output_dim=2).raw_luts.shape == (2, 512)  # wider than the layer kernels' 6 inputs
        node = cls(input_dim=4, output_dim=1)
        assert node.raw_luts.shape == (1, 16) and float(node.raw_luts.abs().max()) < 1.0  # 0.1 * randn


def test_convolutional_layer_structure_matches_reference(golden):
    from difflut_b200.layers import ConvolutionalLayer, ConvolutionConfig, GroupedInputConfig

    g = golden("conv_layer")
    assert difflut.REGISTRY.get_convolutional_layer("convolutional") is ConvolutionalLayer
    for tag, C in (("dwn_d2", 2), ("dwn_s2p1_grouped", 3), ("prob_d2", 2)):
        k, stride, pad, trees, depth, n, chunk, grouped = (int(v) for v in g[f"{tag}_cfg"])
        node = ProbabilisticNode if tag.startswith("prob") else DWNNode
        conv = ConvolutionalLayer(
            ConvolutionConfig(tree_depth=depth, in_channels=C, out_channels=trees, receptive_field=k,
                              stride=stride, padding=pad, chunk_size=chunk, seed=7),
            node, NodeConfig(input_dim=n, output_dim=1), RandomLayer, n_inputs_per_node=n,
            grouped_connections=bool(grouped), ensure_full_coverage=bool(grouped))
        assert conv.hidden_layers == [n ** (depth - i) for i in range(depth + 1)]
        assert len(conv.first_layer_chunks) == -(-trees // min(chunk, trees)) and len(conv.trees) == trees
        levels = conv._level_layers()
        for l, level in enumerate(levels):  # the sub-layers' maps are the reference's, bit for bit
            got = torch.cat([s._mapping_indices.long() for s in level])
            assert np.array_equal(got.numpy(), g[f"{tag}_map{l}"]), (tag, l)
        assert conv._mergeable()
        plans = conv._plans(torch.device("cpu"))
        assert [p.input_size for p in plans] == [C * k * k] + [h * trees for h in conv.hidden_layers[:-1]]
        assert int(plans[1].map_nodes[-1].min()) >= (trees - 1) * conv.hidden_layers[0]  # last tree's own block
        keys = set(conv.state_dict())
        pname = "raw_weights" if node is ProbabilisticNode else "luts"
        assert f"first_layer_chunks.0.nodes.0.{pname}" in keys and f"trees.{trees - 1}.0.nodes.0.{pname}" in keys
    for tag, cover in (("cover", True), ("free", False)):
        state = torch.get_rng_state()
        gi = GroupedInputConfig(n_groups=3, input_size=27, output_trees=5, luts_per_tree=6, bits_per_node=4,
                                seed=11, ensure_full_coverage=cover)
        assert torch.equal(torch.get_rng_state(), state)
        assert np.array_equal(gi.mapping_indices.numpy(), g[f"grouped_{tag}"])
        assert np.array_equal(gi.get_mapping_indices(1, 3).numpy(), g[f"grouped_{tag}"][6:18])
    with pytest.raises(ValueError):
        GroupedInputConfig(0, 27, 5, 6, 4, 11)
    with pytest.raises(AssertionError):
        ConvolutionConfig(in_channels=None, out_channels=4)
    with pytest.raises(ValueError):  # wrong rank
        conv(torch.zeros(2, 5))


def test_dwn_stack_validation():
    from difflut_b200.layers import DWNStack

    cfg = NodeConfig(input_dim=6, output_dim=1)
    a = RandomLayer(24, 10, DWNNode, cfg, seed=1)
    b = RandomLayer(10, 4, DWNNode, cfg, seed=2)
    stack = DWNStack([a, b])
    assert list(stack.state_dict()) == ["layers." + k for k in torch.nn.Sequential(a, b).state_dict()]
    assert [p.data_ptr() for p in stack.parameters()] == [a.luts.data_ptr(), b.luts.data_ptr()]  # same parameters
    with pytest.raises(ValueError):
        DWNStack([])
    with pytest.raises(ValueError, match="does not match"):
        DWNStack([b, a])
    with pytest.raises(ValueError):
        DWNStack([RandomLayer(24, 10, ProbabilisticNode, cfg, seed=1)])
    with pytest.raises(ValueError):
        DWNStack([RandomLayer(24, 10, DWNNode, NodeConfig(input_dim=6, output_dim=2), seed=1)])
    with pytest.raises(ValueError, match="randperm"):
        DWNStack([a, b], groupsum=GroupSum(k=2, tau=1.0, use_randperm=True))
    with pytest.raises(RuntimeError):
        stack(torch.zeros(3, 24))  # CPU tensors are rejected, there is no CPU path
    # options that only the per-layer API applies are refused, not silently dropped
    with pytest.raises(ValueError, match="flip_probability"):
        DWNStack([RandomLayer(24, 10, DWNNode, cfg, seed=1, flip_probability=0.1), b])
    with pytest.raises(ValueError, match="grad_stabilization"):
        DWNStack([a, RandomLayer(10, 4, DWNNode, cfg, seed=2, grad_stabilization="layerwise")])


def test_dwn_network_refuses_layer_options_it_would_drop():
    from difflut_b200.encoder import ThermometerEncoder
    from difflut_b200.network import DWNNetwork

    cfg = NodeConfig(input_dim=6, output_dim=1)
    enc = ThermometerEncoder(num_bits=2).fit(torch.rand(16, 12))
    gs = GroupSum(k=2, tau=1.0, use_randperm=False)
    for kw in ({"flip_probability": 0.2}, {"grad_stabilization": "batchwise"}):
        with pytest.raises(ValueError, match="flip_probability / grad_stabilization"):
            DWNNetwork(enc, [RandomLayer(24, 10, DWNNode, cfg, seed=1, **kw)], gs)


def test_layer_option_host_paths_match_reference(golden):
    """The mixin's host-side branches (CPU tensors) reproduce the reference's outputs: both flip rules under the
    same generator seed, bit for bit, and the gradient rescaling."""
    from difflut_b200.layers import LayerConfig

    g = golden("layer_options")
    x = torch.from_numpy(g["flip_x"])
    cfg = NodeConfig(input_dim=3, output_dim=1)
    for tag in ("sparse", "dense"):
        layer = RandomLayer(50, 4, DWNNode, cfg, layer_config=LayerConfig(flip_probability=float(g[f"flip_{tag}_p"][0]))).train()
        torch.manual_seed(77)
        assert torch.equal(layer._apply_bit_flip(x.clone()), torch.from_numpy(g[f"flip_{tag}_out"])), tag
    for mode in ("layerwise", "batchwise"):
        for subtract in (0, 1):
            layer = RandomLayer(12, 4, DWNNode, cfg,
                                layer_config=LayerConfig(grad_stabilization=mode, grad_target_std=2.0,
                                                         grad_subtract_mean=bool(subtract), grad_epsilon=1e-6)).train()
            for name in ("small", "wide"):
                got = layer._apply_gradient_stabilization(torch.from_numpy(g[f"g_{name}"]))
                torch.testing.assert_close(got, torch.from_numpy(g[f"rescaled_{mode}_{subtract}_{name}"]), rtol=1e-6, atol=1e-7)


def test_connection_plan_inverse_maps_agree():
    """ConnectionPlan's two forms of the inverse map (CSR, and the table interleaved by feature that
    dl_gather_rows_bwd_ell reads) list the same columns for every feature, in ascending order, and every
    listed column really maps to that feature (difflut/layers/random_layer.py:258-304 scatters by the same map)."""
    import torch

    from difflut_b200.layers.fused_ops import ConnectionPlan
    from difflut_b200.layers.random_layer import draw_random_mapping

    I, N, n = 50, 40, 6
    mapping = draw_random_mapping(I, N, n, 3, True)
    plan = ConnectionPlan(mapping, I, 1, torch.device("cpu"))
    ell, max_deg = plan.ell_nodes()
    ptr, ent = plan.inv_ptr_nodes.long(), plan.inv_ent_nodes
    assert ell.shape == (max_deg, I) and int((ell >= 0).sum()) == N * n
    flat = mapping.reshape(-1)
    for f in range(I):
        seg = ent[ptr[f]:ptr[f + 1]].tolist()
        col = [int(v) for v in ell[:, f].tolist() if v >= 0]
        assert seg == col == sorted(seg)
        assert all(int(flat[c]) == f for c in seg)
        assert (ell[len(seg):, f] == -1).all()

