"""Pins the CPU oracle to fixtures produced by the unmodified reference (tests/golden/make_golden.py)."""

import hashlib
import warnings

import numpy as np
import pytest
import torch

from oracle import difflut_oracle as O
from parity_util import close_normwise


def T(a):
    return torch.from_numpy(np.asarray(a))


def test_thermometer_bits_exact(golden):
    g = golden("thermometer")
    for nb in (1, 3, 8):
        thr = O.thermometer_thresholds(T(g[f"x_fit_T{nb}"]), nb)
        assert torch.equal(thr, T(g[f"thr_T{nb}"]))
        bits = O.thermometer_encode(T(g[f"x_T{nb}"]), thr)
        assert np.array_equal(bits.numpy().astype(np.uint8), g[f"bits_T{nb}"])
        # equality with the threshold must encode as 0 (strict '>')
        assert bits[0].reshape(-1, nb)[:, 0].sum() == 0


def test_index_maps_exact(golden):
    g = golden("index_maps")
    for name in ("c1", "cov_rem", "cov_exact", "small_in", "n4"):
        I, N, n, seed, cov = (int(v) for v in g[name + "_args"])
        before = torch.get_rng_state()
        idx = O.random_mapping(I, N, n, seed, bool(cov))
        assert torch.equal(before, torch.get_rng_state()), "global RNG state must be restored"
        assert idx.dtype == torch.int16
        assert np.array_equal(idx.numpy(), g[name])
    for name, I, N, seed in (("c4_l1", 6272, 16000, 0), ("c4_l2", 16000, 8000, 1), ("c4_l3", 8000, 4000, 2)):
        idx = O.random_mapping(I, N, 6, seed, True)
        digest = np.frombuffer(hashlib.sha256(idx.numpy().tobytes()).digest(), dtype=np.uint8)
        assert np.array_equal(digest, g[name + "_sha256"])
        assert np.array_equal(idx[:4].numpy(), g[name + "_head"])
    assert O.random_mapping(40000, 10, 6, 0).dtype == torch.int32


def test_dwn_layer_matches_reference(golden):
    g = golden("dwn_layer")
    for tag in ("n6", "n4o2", "n2"):
        x, idx, tab = T(g[f"{tag}_x"]), T(g[f"{tag}_map"]), T(g[f"{tag}_tables"])
        alpha, beta = g[f"{tag}_alpha_beta"]
        xm = O.gather_mapping(x, idx)
        y = O.dwn_forward(xm, tab)
        B = x.shape[0]
        assert torch.equal(y.reshape(B, -1), T(g[f"{tag}_y"]))  # table values: exact
        gy = T(g[f"{tag}_gy"]).reshape(y.shape)
        gxm, gl = O.dwn_backward(xm, tab, gy, alpha, beta)
        gx = O.gather_mapping_backward(gxm, idx, x.shape[1])
        torch.testing.assert_close(gx, T(g[f"{tag}_gx"]), rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(gl, T(g[f"{tag}_gtables"]), rtol=1e-5, atol=1e-6)
        ye = O.dwn_forward_eval(O.gather_mapping((x >= 0.5).float(), idx), tab)
        assert np.array_equal(ye.reshape(B, -1).numpy().astype(np.uint8), g[f"{tag}_y_eval"])


def test_dwn_stable_layer_matches_reference(golden):
    g = golden("dwn_stable_layer")
    for tag in ("n6", "n4o2", "n3"):
        x, idx, raw = T(g[f"{tag}_x"]), T(g[f"{tag}_map"]), T(g[f"{tag}_raw"])
        scale = float(g[f"{tag}_scale"][0])
        tab = torch.sigmoid(raw)
        xm = O.gather_mapping(x, idx)
        y = O.dwn_forward(xm, tab)
        B = x.shape[0]
        # sigmoid of the stacked tensor may differ from the per-node sigmoid by one ulp (vector vs scalar tail)
        torch.testing.assert_close(y.reshape(B, -1), T(g[f"{tag}_y"]), rtol=0, atol=1e-7)
        gy = T(g[f"{tag}_gy"]).reshape(y.shape)
        gxm, gl = O.dwn_stable_backward(xm, tab, gy, scale)
        gx = O.gather_mapping_backward(gxm, idx, x.shape[1])
        torch.testing.assert_close(gx, T(g[f"{tag}_gx"]), rtol=1e-5, atol=1e-6)
        graw = gl * tab * (1.0 - tab)  # chain rule through the sigmoid parameterisation
        torch.testing.assert_close(graw, T(g[f"{tag}_graw"]), rtol=1e-5, atol=1e-6)
        ye = O.dwn_forward_eval(O.gather_mapping((x >= 0.5).float(), idx), tab)
        assert np.array_equal(ye.reshape(B, -1).numpy().astype(np.uint8), g[f"{tag}_y_eval"])
    # per-node scales equal the scalar form when all nodes share one value
    a = O.stable_transform(tab, 0.7)
    b = O.stable_transform(tab, torch.full((tab.shape[0],), 0.7))
    torch.testing.assert_close(a, b)


def test_hybrid_layer_matches_reference(golden):
    g = golden("hybrid_layer")
    for tag in ("n6", "n4o2", "n2"):
        x, idx, raw = T(g[f"{tag}_x"]), T(g[f"{tag}_map"]), T(g[f"{tag}_raw"])
        tab = torch.sigmoid(raw)
        xm = O.gather_mapping(x, idx)
        y = O.dwn_forward(xm, tab)
        B = x.shape[0]
        torch.testing.assert_close(y.reshape(B, -1), T(g[f"{tag}_y"]), rtol=0, atol=1e-7)
        gy = T(g[f"{tag}_gy"]).reshape(y.shape)
        gxm, gl = O.hybrid_backward(xm, tab, gy)
        gx = O.gather_mapping_backward(gxm, idx, x.shape[1])
        gx_ref = T(g[f"{tag}_gx"])
        torch.testing.assert_close(gx, gx_ref, rtol=1e-5, atol=1e-6)
        assert torch.count_nonzero(gx_ref[0, : x.shape[1] // 2]) == 0  # binary inputs get no gradient
        torch.testing.assert_close(gl * tab * (1.0 - tab), T(g[f"{tag}_graw"]), rtol=1e-5, atol=1e-6)
        ye = O.dwn_forward_eval(O.gather_mapping((x >= 0.5).float(), idx), tab)
        assert np.array_equal(ye.reshape(B, -1).numpy().astype(np.uint8), g[f"{tag}_y_eval"])


def _conv_case(g, tag):
    k, stride, pad, trees, depth, n, chunk, grouped = (int(v) for v in g[f"{tag}_cfg"])
    hidden = [n ** (depth - i) for i in range(depth + 1)]
    maps = O.conv_level_maps([T(g[f"{tag}_map{l}"]) for l in range(depth + 1)], hidden, trees)
    pars = [T(g[f"{tag}_par{l}"]) for l in range(depth + 1)]
    return k, stride, pad, trees, depth, n, chunk, bool(grouped), hidden, maps, pars


@pytest.mark.parametrize("tag", ["dwn_d2", "dwn_s2p1_grouped"])
def test_conv_dwn_matches_reference(golden, tag):
    g = golden("conv_layer")
    k, stride, pad, trees, depth, n, _, _, hidden, maps, tables = _conv_case(g, tag)
    x = T(g[f"{tag}_x"])
    y_ref = T(g[f"{tag}_y"])
    B, _, OH, OW = y_ref.shape
    rows, acts = O.conv_dwn_forward(x, k, stride, pad, maps, tables)
    assert torch.equal(O.conv_output(rows, B, OH, OW), y_ref)
    gy = T(g[f"{tag}_gy"])
    grows = gy.reshape(B, trees, OH * OW).transpose(1, 2).reshape(B * OH * OW, trees)
    alpha, beta = 0.5 * 0.75 ** (n - 1), 0.25 / 0.75
    gx, gts = O.conv_dwn_backward(acts, maps, tables, grows, alpha, beta, x.shape, k, stride, pad)
    torch.testing.assert_close(gx, T(g[f"{tag}_gx"]), rtol=1e-5, atol=1e-6)
    for l in range(depth + 1):
        torch.testing.assert_close(gts[l], T(g[f"{tag}_gpar{l}"]), rtol=1e-5, atol=1e-6)
    rows_e, _ = O.conv_dwn_forward((x >= 0.5).float(), k, stride, pad, maps, tables, eval_mode=True)
    assert np.array_equal(O.conv_output(rows_e, B, OH, OW).numpy().astype(np.uint8), g[f"{tag}_y_eval"])


def test_conv_prob_matches_reference(golden):
    g = golden("conv_layer")
    tag = "prob_d2"
    k, stride, pad, trees, depth, n, _, _, hidden, maps, raws = _conv_case(g, tag)
    x = T(g[f"{tag}_x"]).requires_grad_(True)
    raws = [r.clone().requires_grad_(True) for r in raws]
    y_ref = T(g[f"{tag}_y"])
    B, _, OH, OW = y_ref.shape
    h = O.conv_unfold(x, k, stride, pad)
    for m, r in zip(maps, raws):
        h = O.prob_forward(O.gather_mapping(h, m), r).reshape(h.shape[0], -1)
    y = O.conv_output(h, B, OH, OW)
    torch.testing.assert_close(y, y_ref, rtol=1e-5, atol=1e-6)
    y.backward(T(g[f"{tag}_gy"]))
    torch.testing.assert_close(x.grad, T(g[f"{tag}_gx"]), rtol=1e-5, atol=1e-6)
    for l in range(depth + 1):
        torch.testing.assert_close(raws[l].grad, T(g[f"{tag}_gpar{l}"]), rtol=1e-5, atol=1e-6)


def test_grouped_mapping_exact(golden):
    g = golden("conv_layer")
    for tag, cover in (("cover", True), ("free", False)):
        state = torch.get_rng_state()
        m = O.grouped_mapping(3, 27, 5, 6, 4, 11, cover)
        assert torch.equal(torch.get_rng_state(), state)
        assert np.array_equal(m.numpy(), g[f"grouped_{tag}"])
        assert bool(((m // 9) == (m[:, :1] // 9)).all())  # a node reads one group only


def test_dwn_residual_tables_pass_bit0(golden):
    tab = T(golden("dwn_layer")["residual_tables"]).reshape(1, 1, 64)
    a = torch.arange(64)
    xm = ((a[:, None] >> torch.arange(6)) & 1).float().reshape(64, 1, 6)
    out = O.dwn_forward_eval(xm, tab).reshape(64)
    assert torch.equal(out, xm[:, 0, 0])


def test_prob_layer_matches_reference(golden):
    g = golden("prob_layer")
    x = T(g["x"]).requires_grad_(True)
    raw = T(g["raw"]).requires_grad_(True)
    idx = T(g["map"])
    y = O.prob_forward(O.gather_mapping(x, idx), raw, 1.0).reshape(x.shape[0], -1)
    torch.testing.assert_close(y, T(g["y"]), rtol=1e-5, atol=1e-6)
    logits = O.groupsum(y, 10, 1.0)
    torch.testing.assert_close(logits, T(g["logits"]), rtol=1e-5, atol=1e-5)
    loss = torch.nn.functional.cross_entropy(logits, T(g["labels"]))
    loss.backward()
    torch.testing.assert_close(loss.detach(), T(g["loss"]), rtol=1e-6, atol=1e-6)
    close_normwise(x.grad, T(g["gx"]), "x.grad")
    close_normwise(raw.grad, T(g["graw"]), "raw.grad")
    ye = O.prob_forward_eval(O.gather_mapping((x.detach() >= 0.5).float(), idx), raw.detach(), 1.0)
    assert np.array_equal(ye.reshape(x.shape[0], -1).numpy().astype(np.uint8), g["y_eval"])
    # temperature 0.5, n=3, two outputs per node
    x2 = T(g["t_x"]).requires_grad_(True)
    raw2 = T(g["t_raw"]).requires_grad_(True)
    y2 = O.prob_forward(O.gather_mapping(x2, T(g["t_map"])), raw2, 0.5).reshape(x2.shape[0], -1)
    torch.testing.assert_close(y2, T(g["t_y"]), rtol=1e-5, atol=1e-6)
    y2.backward(T(g["t_gy"]))
    close_normwise(x2.grad, T(g["t_gx"]), "x2.grad")
    close_normwise(raw2.grad, T(g["t_graw"]), "raw2.grad")


def test_learnable_layer_matches_reference(golden):
    g = golden("learnable_layer")
    x = T(g["x"]).requires_grad_(True)
    W = T(g["W"]).requires_grad_(True)
    tab = T(g["tables"])
    tau = float(g["tau"][0])
    m = O.learnable_soft_mapping(x, W, tau)
    torch.testing.assert_close(m.reshape(g["m"].shape), T(g["m"]), rtol=1e-6, atol=1e-7)
    N = tab.shape[0]
    xm = m.reshape(x.shape[0], N, 6)
    y = O.dwn_forward(xm.detach(), tab).reshape(x.shape[0], -1)
    assert torch.equal(y, T(g["y"]))
    alpha, beta = 0.5 * 0.75**5, 0.25 / 0.75
    gxm, gl = O.dwn_backward(xm.detach(), tab, T(g["gy"]).reshape(x.shape[0], N, 1), alpha, beta)
    torch.testing.assert_close(gl, T(g["gtables"]), rtol=1e-5, atol=1e-6)
    m.backward(gxm.reshape(m.shape))
    close_normwise(x.grad, T(g["gx"]), "x.grad")
    close_normwise(W.grad, T(g["gW"]), "W.grad")
    idx = torch.argmax(W.detach(), -1).reshape(N, 6)
    assert np.array_equal(idx.numpy(), g["hard_idx"])
    ye = O.dwn_forward_eval(O.learnable_hard_mapping(x.detach(), W.detach()).reshape(-1, N, 6), tab)
    assert np.array_equal(ye.reshape(x.shape[0], -1).numpy().astype(np.uint8), g["y_eval"])
    assert abs(O.learnable_tau(500, 1.0, 0.0001, 1000.0) - float(g["tau_500"][0])) < 1e-12


def test_groupsum_known_answers(golden):
    g = golden("groupsum")
    x = T(g["x"])
    torch.testing.assert_close(O.groupsum(x, 4, 2.0), T(g["k4_tau2"]), rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(O.groupsum(x, 1, 1.0), T(g["k1_tau1"]), rtol=1e-6, atol=1e-6)
    ones = torch.ones(3, 12)
    assert torch.equal(O.groupsum(ones, 4, 1.0), torch.full((3, 4), 3.0))


def test_dwn_net3_two_adam_steps(golden):
    g = golden("dwn_net3")
    x, labels = T(g["x"]), T(g["labels"])
    k, tau = int(g["k_tau"][0]), float(g["k_tau"][1])
    thr = O.thermometer_thresholds(x, 4)
    assert torch.equal(thr, T(g["thr"]))
    bits = O.thermometer_encode(x, thr)
    maps = [T(g[f"map{i}"]) for i in range(3)]
    tabs = [T(g[f"tables{i}"]) for i in range(3)]
    alpha, beta = 0.5 * 0.75**5, 0.25 / 0.75
    ms = [torch.zeros_like(t) for t in tabs]
    vs = [torch.zeros_like(t) for t in tabs]
    for step in range(2):
        logits, acts = O.dwn_network_forward(bits, maps, tabs, k, tau)
        torch.testing.assert_close(logits, T(g[f"logits_step{step}"]), rtol=1e-5, atol=1e-5)
        lg = logits.clone().requires_grad_(True)
        loss = torch.nn.functional.cross_entropy(lg, labels)
        loss.backward()
        torch.testing.assert_close(loss.detach(), T(g[f"loss_step{step}"]), rtol=1e-5, atol=1e-6)
        grads = O.dwn_network_backward(acts, maps, tabs, lg.grad, k, tau, alpha, beta)
        for i in range(3):
            close_normwise(grads[i], T(g[f"gtables{i}_step{step}"]), "grads[i]")
            tabs[i], ms[i], vs[i] = O.adam_step(tabs[i], grads[i], ms[i], vs[i], step + 1, 1e-2)
            torch.testing.assert_close(tabs[i], T(g[f"tables{i}_after{step}"]), rtol=1e-5, atol=2e-6)
    counts = O.dwn_network_hard_counts(bits, maps, tabs, k)
    assert np.array_equal(counts.numpy(), g["eval_counts"])


def test_pack_layouts():
    bits = (torch.rand(70, 45, generator=torch.Generator().manual_seed(0)) > 0.5).float()
    fm = O.pack_bits_feature_major(bits)
    assert fm.shape == (45, 3)
    for b, f in ((0, 0), (33, 7), (69, 44)):
        assert (fm[f, b // 32] >> (b % 32)) & 1 == int(bits[b, f])
    rm = O.pack_bits_row_major(bits)
    assert rm.shape == (70, 2)
    for b, f in ((0, 0), (33, 7), (69, 44)):
        assert (rm[b, f // 32] >> (f % 32)) & 1 == int(bits[b, f])


def test_oracle_adjoint_and_linearity_properties():
    """Size-independent properties of the checker itself: the gather backward is the adjoint of the gather,
    fold is the adjoint of unfold, GroupSum is linear, the two transforms are linear in the table."""
    gen = torch.Generator().manual_seed(123)
    x = torch.randn(7, 20, generator=gen, dtype=torch.float64)
    idx = torch.randint(0, 20, (9, 4), generator=gen)
    g = torch.randn(7, 9, 4, generator=gen, dtype=torch.float64)
    lhs = (O.gather_mapping(x, idx) * g).sum()
    rhs = (x * O.gather_mapping_backward(g, idx, 20).double()).sum()
    assert abs(float(lhs - rhs)) < 1e-4 * (1 + abs(float(lhs)))
    img = torch.randn(2, 3, 7, 6, generator=gen)
    for kernel, stride, pad in (((3, 3), (1, 1), (0, 0)), ((3, 2), (2, 1), (1, 0)), ((4, 4), (3, 2), (0, 3))):
        p = O.conv_unfold(img, kernel, stride, pad)
        gp = torch.randn(p.shape, generator=gen)
        a = (p * gp).sum()
        b = (img * O.conv_fold(gp, img.shape, kernel, stride, pad)).sum()
        assert abs(float(a - b)) < 1e-3 * (1 + abs(float(a)))
    y = torch.randn(5, 23, generator=gen)
    z = torch.randn(5, 23, generator=gen)
    torch.testing.assert_close(O.groupsum(y + 2 * z, 4, 3.0), O.groupsum(y, 4, 3.0) + 2 * O.groupsum(z, 4, 3.0),
                               rtol=1e-5, atol=1e-5)
    t1 = torch.rand(3, 2, 16, generator=gen, dtype=torch.float64)
    t2 = torch.rand(3, 2, 16, generator=gen, dtype=torch.float64)
    torch.testing.assert_close(O.efd_transform(t1 + t2, 0.3, 0.4), O.efd_transform(t1, 0.3, 0.4) + O.efd_transform(t2, 0.3, 0.4))
    torch.testing.assert_close(O.stable_transform(t1 + t2, 1.25), O.stable_transform(t1, 1.25) + O.stable_transform(t2, 1.25))
    # the transform does not depend on the value of the differentiated bit of the address
    T = O.efd_transform(t1, 0.3, 0.4)  # (N, O, L, n)
    for i in range(4):
        a = torch.arange(16)
        assert torch.equal(T[:, :, a, i], T[:, :, a ^ (1 << i), i])
    # packing round trip
    bits = (torch.rand(70, 9, generator=gen) > 0.5).float()
    packed = O.pack_bits_feature_major(bits)
    unpacked = ((packed[:, :, None] >> np.arange(32, dtype=np.uint32)[None, None, :]) & 1).reshape(9, -1)[:, :70].T
    assert np.array_equal(unpacked, bits.numpy().astype(np.uint32))


def test_layer_options_match_reference(golden):
    """Gradient rescaling and the two bit-flip rules against outputs of the reference's LUTLayerMixin."""
    g = golden("layer_options")
    target, eps = (float(v) for v in g["rescale_params"])
    for mode in ("layerwise", "batchwise"):
        for subtract in (0, 1):
            for name in ("small", "wide"):
                got = O.grad_rescale(T(g[f"g_{name}"]), mode, target, bool(subtract), eps)
                torch.testing.assert_close(got, T(g[f"rescaled_{mode}_{subtract}_{name}"]), rtol=1e-6, atol=1e-7)
    x = T(g["flip_x"])
    torch.manual_seed(77)
    pos = O.flip_positions_sparse(x.numel(), float(g["flip_sparse_p"][0]))
    assert pos.numel() == int(x.numel() * 0.03)
    assert torch.equal(O.flip_apply(x, pos), T(g["flip_sparse_out"]))
    # dense rule: about p of the entries flip, and a flipped entry holds exactly 1 - x
    dense = T(g["flip_dense_out"])
    changed = dense != x
    assert 0.2 < float(changed.float().mean()) < 0.4
    assert torch.equal(dense[changed], (x + (1.0 - 2.0 * x))[changed])
