"""CPU oracle for the DiffLUT LUT-network hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, as vectorised torch-CPU / numpy code, the arithmetic of the
reference's PyTorch path (aplesner/difflut v1.4.4).  It exists so the CUDA path can be
checked against it; nothing in the shipped package imports it.  Only the test-suite,
the smoke check and the CPU-baseline leg of the benchmark may call it.

Parity status: PINNED.  `tests/golden/make_golden.py` imports the unmodified reference,
runs it on seeded inputs and stores inputs + outputs as small fixtures; the oracle
is asserted equal to those fixtures in `tests/test_oracle_golden.py` (bit-exact for
bits / addresses / index maps / hard outputs, 1e-6 for fp32 values and gradients).

Every function cites the reference file:line it follows.  Conventions (all from the
reference): thermometer bit = `x > thr` (strict); DWN address bit = `x >= 0.5`; address
is LSB-first (input slot i -> bit i); DWN tables are (out_dim, 2^n); probabilistic
tables are (2^n, out_dim); GroupSum class c sums the contiguous block c of nodes.
Stacked layouts used here: DWN tables (N, O, 2^n); probabilistic raw (N, 2^n, O).
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import numpy as np
import torch
import torch.nn.functional as F

# ----------------------------------------------------------------------------------
# Thermometer encoder
# ----------------------------------------------------------------------------------


def thermometer_thresholds(x: torch.Tensor, num_bits: int) -> torch.Tensor:
    """Per-feature thresholds `min + i*(max-min)/(T+1)`, i=1..T -> (F, T).

    Follows difflut/encoder/thermometer.py:38-59 with the same torch op order
    (int64 arange promoted against fp32), which is what makes the bits bit-exact.
    """
    lo = x.min(dim=0)[0]
    hi = x.max(dim=0)[0]
    steps = torch.arange(1, num_bits + 1, device=x.device)
    width = (hi - lo) / (num_bits + 1)
    return lo.unsqueeze(-1) + steps.unsqueeze(0) * width.unsqueeze(-1)


def thermometer_encode(x: torch.Tensor, thresholds: torch.Tensor, flatten: bool = True) -> torch.Tensor:
    """bit[b,f,i] = x[b,f] > thr[f,i]; flattened column = f*T+i.

    Follows difflut/encoder/thermometer.py:89-116.
    """
    enc = (x.unsqueeze(-1) > thresholds).float()
    if flatten:
        enc = enc.reshape(enc.shape[0], -1)
    return enc


def pack_bits_feature_major(bits: torch.Tensor) -> np.ndarray:
    """(B, F) {0,1} -> uint32 (F, ceil(B/32)); bit (b%32) of word b//32 of row f.

    No counterpart in the reference (it has no packed format); this defines the
    packed layout the CUDA kernels are checked against.
    """
    b = bits.detach().cpu().numpy().astype(np.uint8)
    B, Fdim = b.shape
    W = (B + 31) // 32
    pad = np.zeros((W * 32, Fdim), dtype=np.uint8)
    pad[:B] = b
    # little-endian bit order inside each byte, little-endian bytes in each word
    by = np.packbits(pad.T.reshape(Fdim, W, 32), axis=-1, bitorder="little")
    return by.reshape(Fdim, W, 4).view(np.uint32).reshape(Fdim, W)


def pack_bits_row_major(bits: torch.Tensor) -> np.ndarray:
    """(B, F) {0,1} -> uint32 (B, ceil(F/32)); bit (f%32) of word f//32 of row b."""
    b = bits.detach().cpu().numpy().astype(np.uint8)
    B, Fdim = b.shape
    W = (Fdim + 31) // 32
    pad = np.zeros((B, W * 32), dtype=np.uint8)
    pad[:, :Fdim] = b
    by = np.packbits(pad.reshape(B, W, 32), axis=-1, bitorder="little")
    return by.reshape(B, W, 4).view(np.uint32).reshape(B, W)


# ----------------------------------------------------------------------------------
# RandomLayer index map and gather
# ----------------------------------------------------------------------------------


def random_mapping(
    input_size: int,
    output_size: int,
    n: int,
    seed: int,
    ensure_full_input_coverage: bool = True,
) -> torch.Tensor:
    """Seeded (N, n) index map; int16 when input_size < 32768 else int32.

    Follows difflut/layers/random_layer.py:195-256: the global CPU generator is
    saved, seeded, used for randperm / multinomial, and restored.
    """
    state = torch.get_rng_state()
    torch.manual_seed(seed)
    dtype = torch.int16 if input_size < 32768 else torch.int32
    if not ensure_full_input_coverage:
        idx = torch.multinomial(
            torch.ones((output_size, input_size)), num_samples=n, replacement=n > input_size
        ).to(dtype)
    else:
        total = output_size * n
        cycles, rest = divmod(total, input_size)
        parts = [torch.randperm(input_size) for _ in range(cycles)]
        if rest > 0:
            parts.append(torch.multinomial(torch.ones(input_size), num_samples=rest, replacement=False))
        idx = torch.cat(parts).reshape(output_size, n).to(dtype)
    torch.set_rng_state(state)
    return idx


def gather_mapping(x: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    """m[b,j,i] = x[b, idx[j,i]] -> (B, N, n).  difflut/layers/random_layer.py:284-304."""
    return x[:, idx.long()]


def gather_mapping_backward(g: torch.Tensor, idx: torch.Tensor, input_size: int) -> torch.Tensor:
    """Scatter-add of (B, N, n) into (B, input_size); float64 accumulation, fp32 result.

    Adjoint of `gather_mapping` (autograd of torch.gather, random_layer.py:301-302).
    """
    B = g.shape[0]
    out = torch.zeros(B, input_size, dtype=torch.float64)
    out.index_add_(1, idx.long().reshape(-1), g.reshape(B, -1).double())
    return out.float()


# ----------------------------------------------------------------------------------
# DWN node: forward, eval, EFD backward
# ----------------------------------------------------------------------------------


def dwn_addresses(xm: torch.Tensor) -> torch.Tensor:
    """addr[b,j] = sum_i [xm[b,j,i] >= 0.5] << i  (LSB-first).  dwn_node.py:147-153."""
    n = xm.shape[-1]
    bits = (xm >= 0.5).long()
    return (bits << torch.arange(n)).sum(-1)


def dwn_forward(xm: torch.Tensor, luts: torch.Tensor) -> torch.Tensor:
    """out[b,j,o] = luts[j,o,addr[b,j]] (raw table value, no clamp) -> (B, N, O).

    dwn_node.py:138-165; luts stacked (N, O, 2^n).
    """
    addr = dwn_addresses(xm)  # (B, N)
    N, O, L = luts.shape
    gathered = torch.gather(luts.unsqueeze(0).expand(addr.shape[0], N, O, L), 3,
                            addr[:, :, None, None].expand(-1, -1, O, 1))
    return gathered.squeeze(-1)


def dwn_forward_eval(xm: torch.Tensor, luts: torch.Tensor) -> torch.Tensor:
    """Eval path: idx=(x*2^arange).sum().long(); out=(luts[:,idx] >= 0.5).float().

    dwn_node.py:457-483 — float arithmetic on inputs that are already {0,1}.
    """
    n = xm.shape[-1]
    powers = 2 ** torch.arange(n, dtype=torch.float32)
    addr = (xm.float() * powers).sum(-1).long()
    N, O, L = luts.shape
    gathered = torch.gather(luts.unsqueeze(0).expand(addr.shape[0], N, O, L), 3,
                            addr[:, :, None, None].expand(-1, -1, O, 1)).squeeze(-1)
    return (gathered >= 0.5).float()


def efd_transform(luts: torch.Tensor, alpha: float, beta: float) -> torch.Tensor:
    """T[j,o,a,i] = alpha * sum_k sgn(k_i) * luts[j,o,k] * beta^popc((a^k) & ~(1<<i)).

    Direct (non-separable) evaluation of the reference's double loop,
    dwn_node.py:195-227, in float64.  (N, O, 2^n) -> (N, O, 2^n, n) float64.
    """
    N, O, L = luts.shape
    n = int(math.log2(L))
    a = torch.arange(L)
    k = torch.arange(L)
    out = torch.empty(N, O, L, n, dtype=torch.float64)
    l64 = luts.double()
    for i in range(n):
        mask = (L - 1) & ~(1 << i)
        x = (a[:, None] ^ k[None, :]) & mask
        ham = torch.zeros_like(x)
        for bit in range(n):
            ham += (x >> bit) & 1
        sign = torch.where(((k >> i) & 1) == 0, -1.0, 1.0).double()
        M = (float(beta) ** ham.double()) * sign[None, :]  # (a, k)
        out[..., i] = float(alpha) * torch.einsum("ak,jok->joa", M, l64)
    return out


def dwn_backward(
    xm: torch.Tensor, luts: torch.Tensor, g: torch.Tensor, alpha: float, beta: float,
    need_input_grad: bool = True, transform: Optional[torch.Tensor] = None,
) -> Tuple[Optional[torch.Tensor], torch.Tensor]:
    """EFD backward: (gxm (B,N,n) fp32, gluts (N,O,2^n) fp32).

    dwn_node.py:167-229.  gluts[j,o,addr_b] += g[b,j,o];  gxm[b,j,i] = sum_o g[b,j,o]*T[j,o,addr,i].
    The reference accumulates input grads in Python floats (float64) and stores fp32;
    table grads are accumulated in fp32 sample by sample — here in float64 then
    rounded (difference is below the 1e-5 parity bar and checked against the fixture).
    """
    addr = dwn_addresses(xm)  # (B,N)
    B, N = addr.shape
    _, O, L = luts.shape
    n = xm.shape[-1]
    gxm = None
    if need_input_grad:  # callers that only want the table gradient (first layer) skip this half
        T = transform if transform is not None else efd_transform(luts, alpha, beta)  # (N,O,L,n)
        Tsel = T[torch.arange(N)[None, :].expand(B, N), :, addr]  # (B,N,O,n)
        gxm = (g.double().unsqueeze(-1) * Tsel).sum(2).float()
    gl = torch.zeros(N, O, L, dtype=torch.float64)
    flat = (torch.arange(N)[None, :, None] * O + torch.arange(O)[None, None, :]) * L + addr[:, :, None]
    gl.view(-1).index_add_(0, flat.reshape(-1), g.double().reshape(-1))
    return gxm, gl.float()


def stable_transform(luts: torch.Tensor, scale) -> torch.Tensor:
    """T[j,o,a,i] = scale_j * sum_k sgn(k_i) * luts[j,o,k] / (popc((a^k) & ~(1<<i)) + 1).

    Gradient-stabilised variant, dwn_stable_node.py:170-202, in float64.  `scale` is a float or a
    per-node tensor (N,).  (N, O, 2^n) -> (N, O, 2^n, n) float64.
    """
    N, O, L = luts.shape
    n = int(math.log2(L))
    a = torch.arange(L)
    k = torch.arange(L)
    out = torch.empty(N, O, L, n, dtype=torch.float64)
    l64 = luts.double()
    sc = torch.as_tensor(scale, dtype=torch.float64).reshape(-1, 1, 1) if torch.is_tensor(scale) else float(scale)
    for i in range(n):
        mask = (L - 1) & ~(1 << i)
        x = (a[:, None] ^ k[None, :]) & mask
        ham = torch.zeros_like(x)
        for bit in range(n):
            ham += (x >> bit) & 1
        sign = torch.where(((k >> i) & 1) == 0, -1.0, 1.0).double()
        M = sign[None, :] / (ham.double() + 1.0)  # (a, k)
        out[..., i] = sc * torch.einsum("ak,jok->joa", M, l64)
    return out


def dwn_stable_backward(
    xm: torch.Tensor, luts: torch.Tensor, g: torch.Tensor, scale
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Gradient-stabilised backward: (gxm (B,N,n) fp32, gluts (N,O,2^n) fp32) w.r.t. the sigmoid-ed tables.

    dwn_stable_node.py:145-205.  gluts[j,o,addr_b] += scale_j * g[b,j,o];
    gxm[b,j,i] = sum_o g[b,j,o] * T[j,o,addr,i] with T of `stable_transform`.
    """
    addr = dwn_addresses(xm)
    B, N = addr.shape
    _, O, L = luts.shape
    T = stable_transform(luts, scale)
    Tsel = T[torch.arange(N)[None, :].expand(B, N), :, addr]  # (B,N,O,n)
    gxm = (g.double().unsqueeze(-1) * Tsel).sum(2).float()
    gl = torch.zeros(N, O, L, dtype=torch.float64)
    flat = (torch.arange(N)[None, :, None] * O + torch.arange(O)[None, None, :]) * L + addr[:, :, None]
    gl.view(-1).index_add_(0, flat.reshape(-1), g.double().reshape(-1))
    sc = torch.as_tensor(scale, dtype=torch.float64).reshape(-1, 1, 1) if torch.is_tensor(scale) else float(scale)
    return gxm, (gl * sc).float()


def hybrid_backward(xm: torch.Tensor, luts: torch.Tensor, g: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Hybrid-node backward: (gxm (B,N,n) fp32, gluts (N,O,2^n) fp32) w.r.t. the sigmoid-ed tables.

    hybrid_node.py:173-224, vectorised over nodes, same fp32 operation order per node:
    P[b,j,a] = prod_i (x_i a_i + (1-x_i)(1-a_i));  gluts[j,o,a] = sum_b P[b,j,a] g[b,j,o];
    gxm[b,j,i] = sum_o g[b,j,o] sum_a P[b,j,a] (a_i - x_i) / (x_i (1-x_i) + 1e-8) luts[j,o,a].
    """
    n = xm.shape[-1]
    pats = prob_patterns(n)  # (L, n)
    xe = xm.unsqueeze(2)  # (B,N,1,n)
    ae = pats[None, None]  # (1,1,L,n)
    probs = torch.prod(xe * ae + (1 - xe) * (1 - ae), dim=3)  # (B,N,L)
    gl = torch.einsum("bjl,bjo->jol", probs, g)
    deriv = (ae - xe) / (xe * (1 - xe) + 1e-8)  # (B,N,L,n)
    pw = probs.unsqueeze(-1) * deriv
    gxm = torch.einsum("bjli,jol,bjo->bji", pw, luts, g)
    return gxm, gl


# ----------------------------------------------------------------------------------
# Probabilistic node
# ----------------------------------------------------------------------------------


def prob_patterns(n: int) -> torch.Tensor:
    """(2^n, n) LSB-first binary patterns.  probabilistic_node.py:227-234."""
    a = torch.arange(2**n)
    return ((a[:, None] >> torch.arange(n)[None, :]) & 1).float()


def prob_weights(raw: torch.Tensor, temperature: float) -> torch.Tensor:
    """sigmoid(raw / max(T, 1e-6)).  probabilistic_node.py:236-239."""
    t = torch.tensor(float(temperature)).clamp(min=1e-6)
    return torch.sigmoid(raw / t)


def prob_forward(xm: torch.Tensor, raw: torch.Tensor, temperature: float = 1.0) -> torch.Tensor:
    """out[b,j,o] = sum_a sigma(raw[j,a,o]/T) * prod_i (a_i ? x_i : 1-x_i) -> (B, N, O).

    probabilistic_node.py:286-300, vectorised over nodes; raw stacked (N, 2^n, O).
    Differentiable with torch autograd (the reference's backward IS autograd).
    """
    n = xm.shape[-1]
    a = prob_patterns(n).to(xm.dtype)  # (L,n)
    w = prob_weights(raw, temperature)  # (N,L,O)
    xe = xm.unsqueeze(2)  # (B,N,1,n)
    terms = xe * a + (1 - xe) * (1 - a)  # (B,N,L,n)
    probs = torch.prod(terms, dim=-1)  # (B,N,L)
    return torch.einsum("bnl,nlo->bno", probs, w)


def prob_forward_eval(xm: torch.Tensor, raw: torch.Tensor, temperature: float = 1.0) -> torch.Tensor:
    """Hard lookup of sigma(raw/T) thresholded at >= 0.5.  probabilistic_node.py:302-328."""
    n = xm.shape[-1]
    powers = 2 ** torch.arange(n, dtype=xm.dtype)
    addr = (xm * powers).sum(-1).long()  # (B,N)
    w = prob_weights(raw, temperature)  # (N,L,O)
    N = raw.shape[0]
    out = w[torch.arange(N)[None, :].expand_as(addr), addr]  # (B,N,O)
    return (out >= 0.5).float()


# ----------------------------------------------------------------------------------
# GroupSum, LearnableLayer mapping
# ----------------------------------------------------------------------------------


def groupsum(x: torch.Tensor, k: int, tau: float) -> torch.Tensor:
    """Zero-pad to a multiple of k; view (B,k,g); sum(-1)/tau.  utils/modules.py:141-163."""
    Fdim = x.shape[-1]
    if Fdim % k != 0:
        x = F.pad(x, (0, k - Fdim % k))
    g = x.shape[-1] // k
    return x.view(x.shape[0], k, g).sum(-1) / tau


def learnable_soft_mapping(x: torch.Tensor, W: torch.Tensor, tau: float) -> torch.Tensor:
    """Training: x @ softmax(W/tau, -1).T -> (B, N*n).  learnable_layer.py:253-255."""
    return torch.matmul(x, F.softmax(W / tau, dim=-1).t())


def learnable_hard_mapping(x: torch.Tensor, W: torch.Tensor) -> torch.Tensor:
    """Eval: out[b,o] = x[b, argmax(W[o])] (first max on ties).  learnable_layer.py:216-276."""
    return x[:, torch.argmax(W, dim=-1)]


def learnable_tau(iteration: int, tau_start: float, tau_min: float, tau_decay_iters: float) -> float:
    """tau = max(tau_start * 10^(-it/decay), tau_min).  learnable_layer.py:458-468."""
    return max(tau_start * 10.0 ** (-iteration / tau_decay_iters), tau_min)


# ----------------------------------------------------------------------------------
# Convolutional layer: patches, merged tree levels
# ----------------------------------------------------------------------------------


def conv_unfold(x: torch.Tensor, kernel, stride, padding) -> torch.Tensor:
    """(B, C, H, W) -> (B*P, C*kh*kw) patch rows.  convolutional.py:170-173,199-205 (nn.Unfold is
    torch's own op; the transpose + view follow the reference)."""
    patches = F.unfold(x, kernel_size=kernel, padding=padding, stride=stride)  # (B, F, P)
    return patches.transpose(1, 2).contiguous().view(-1, patches.shape[1])


def conv_fold(gpatches: torch.Tensor, shape, kernel, stride, padding) -> torch.Tensor:
    """Adjoint of conv_unfold: (B*P, F) -> (B, C, H, W)."""
    B, C, H, W = shape
    g = gpatches.view(B, -1, gpatches.shape[1]).transpose(1, 2)
    return F.fold(g, output_size=(H, W), kernel_size=kernel, padding=padding, stride=stride)


def conv_level_maps(maps, hidden_layers, trees: int):
    """Per-level index maps of all trees as one layer.  `maps[l]` holds the sub-layers' maps of level l
    one after the other (tree order); for l >= 1 tree t reads its own block of the level below
    (convolutional.py:225-236), i.e. columns t*hidden[l-1] + index."""
    out = [maps[0].long()]
    for l in range(1, len(maps)):
        m = maps[l].long().view(trees, hidden_layers[l], -1)
        shift = (torch.arange(trees) * hidden_layers[l - 1]).view(trees, 1, 1)
        out.append((m + shift).view(trees * hidden_layers[l], -1))
    return out


def conv_output(rows: torch.Tensor, B: int, OH: int, OW: int) -> torch.Tensor:
    """(B*P, trees) -> (B, trees, OH, OW).  convolutional.py:242-249."""
    return rows.view(B, OH * OW, -1).transpose(1, 2).reshape(B, -1, OH, OW)


def conv_dwn_forward(x, kernel, stride, padding, maps, tables, eval_mode: bool = False):
    """DWN trees on every patch: returns (rows (B*P, trees), activations per level)."""
    h = conv_unfold(x, kernel, stride, padding)
    acts = []
    for m, t in zip(maps, tables):
        acts.append(h)
        xm = gather_mapping(h, m)
        h = (dwn_forward_eval(xm, t) if eval_mode else dwn_forward(xm, t)).reshape(h.shape[0], -1)
    return h, acts


def conv_dwn_backward(acts, maps, tables, grows, alpha: float, beta: float, shape, kernel, stride, padding):
    """Backward of conv_dwn_forward: (gx (B,C,H,W), [gtables per level])."""
    grads = [None] * len(maps)
    g = grows
    for l in range(len(maps) - 1, -1, -1):
        xm = gather_mapping(acts[l], maps[l])
        gxm, grads[l] = dwn_backward(xm, tables[l], g.reshape(g.shape[0], -1, 1), alpha, beta)
        g = gather_mapping_backward(gxm, maps[l], acts[l].shape[1])
    return conv_fold(g, shape, kernel, stride, padding), grads


def grouped_mapping(n_groups: int, input_size: int, output_trees: int, luts_per_tree: int, bits_per_node: int,
                    seed: int, ensure_full_coverage: bool) -> torch.Tensor:
    """Index map whose rows stay inside one input group.  layer_config.py:157-215, same generator calls."""
    total = output_trees * luts_per_tree
    size = input_size // n_groups
    state = torch.get_rng_state()
    torch.manual_seed(seed)
    idx = torch.multinomial(torch.ones((total, size)), num_samples=bits_per_node, replacement=bits_per_node > size)
    if not ensure_full_coverage:
        offs = torch.randint(low=0, high=n_groups, size=(total, 1)) * size
    else:
        full, rem = divmod(total, n_groups)
        parts = [torch.randperm(n_groups) for _ in range(full)]
        if rem > 0:
            parts.append(torch.multinomial(torch.ones((n_groups,)), num_samples=rem, replacement=False))
        offs = torch.cat(parts).unsqueeze(1) * size
    torch.set_rng_state(state)
    return idx + offs


# ----------------------------------------------------------------------------------
# Layer training options (LUTLayerMixin)
# ----------------------------------------------------------------------------------


def grad_rescale(g: torch.Tensor, mode: str, target_std: float, subtract_mean: bool, eps: float) -> torch.Tensor:
    """Gradient stabilisation, difflut/layers/base_layer.py:266-339: optionally subtract the mean, then
    multiply by sqrt(target_std / (mean(g^2) + eps)); statistics over the whole tensor ("layerwise") or per
    row ("batchwise")."""
    w = g.clone()
    dims = None if mode == "layerwise" else 1
    if subtract_mean:
        w = w - (w.mean() if dims is None else w.mean(dim=1, keepdim=True))
    var = w.pow(2).mean() if dims is None else w.pow(2).mean(dim=1, keepdim=True)
    return w * torch.sqrt(torch.tensor(float(target_std)) / (var + eps))


def flip_positions_sparse(numel: int, probability: float) -> torch.Tensor:
    """The positions the reference flips when the probability is below 0.05 (base_layer.py:226-262): the first
    int(numel * p) entries of torch.randperm(numel), drawn from the global generator of the calling device."""
    return torch.randperm(numel)[: int(numel * probability)]


def flip_apply(x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
    """x with 1 - x at `positions` of its flattened view (base_layer.py:249-260)."""
    out = x.clone().reshape(-1)
    out[positions] = 1.0 - out[positions]
    return out.view_as(x)


# ----------------------------------------------------------------------------------
# Whole-network helpers (configs of the benchmark)
# ----------------------------------------------------------------------------------


def dwn_network_forward(bits: torch.Tensor, maps, tables, k: int, tau: float):
    """Training-mode forward of a RandomLayer+DWN stack followed by GroupSum.

    bits (B, I0) fp32; maps[l] (N_l, n); tables[l] (N_l, 1, 2^n).  Returns
    (logits (B,k), list of per-layer inputs (B, I_l)) — composition of
    random_layer.py:306-340, dwn_node.py:138-165 and utils/modules.py:116-163.
    """
    acts = [bits]
    h = bits
    for idx, lut in zip(maps, tables):
        h = dwn_forward(gather_mapping(h, idx), lut).reshape(h.shape[0], -1)
        acts.append(h)
    return groupsum(h, k, tau), acts


def dwn_network_backward(acts, maps, tables, glogits: torch.Tensor, k: int, tau: float,
                         alpha: float, beta: float, transforms=None):
    """Backward of `dwn_network_forward`: list of table grads (N_l,1,2^n), first->last.

    `transforms` may hold `efd_transform(tables[l], alpha, beta)` per layer (a caller that walks the
    batch in chunks computes them once); the first layer's input gradient is not formed."""
    N_last = tables[-1].shape[0]
    gsz = (N_last + k - 1) // k
    g = (glogits / tau).repeat_interleave(gsz, dim=1)[:, :N_last]  # (B, N_L)
    grads = [None] * len(tables)
    for l in range(len(tables) - 1, -1, -1):
        xm = gather_mapping(acts[l], maps[l])
        gxm, gl = dwn_backward(xm, tables[l], g.unsqueeze(-1), alpha, beta, need_input_grad=l > 0,
                               transform=None if transforms is None else transforms[l])
        grads[l] = gl
        if l > 0:
            g = gather_mapping_backward(gxm, maps[l], acts[l].shape[1])
    return grads


def dwn_network_hard_counts(bits: torch.Tensor, maps, tables, k: int) -> torch.Tensor:
    """Eval-mode stack: every layer thresholds its table at >= 0.5; class counts int32.

    Composition of dwn_node.py:457-483 per layer and GroupSum with tau=1.
    """
    h = bits
    for idx, lut in zip(maps, tables):
        h = dwn_forward_eval(gather_mapping(h, idx), lut).reshape(h.shape[0], -1)
    return groupsum(h, k, 1.0).round().to(torch.int32)


def adam_step(p, g, m, v, step: int, lr: float, b1: float = 0.9, b2: float = 0.999, eps: float = 1e-8):
    """One torch.optim.Adam step (no weight decay, no amsgrad), single-tensor form.

    Restates torch/optim/adam.py `_single_tensor_adam` (torch 2.11): m,v EMA, bias
    corrections, denom = sqrt(v)/sqrt(bc2) + eps, p -= lr/bc1 * m/denom.
    """
    m = m.lerp(g, 1 - b1)
    v = v * b2 + (1 - b2) * g * g
    bc1 = 1 - b1**step
    bc2 = 1 - b2**step
    denom = v.sqrt() / math.sqrt(bc2) + eps
    p = p - (lr / bc1) * m / denom
    return p, m, v


def dwn_network_train_reference(x: torch.Tensor, labels: torch.Tensor, thresholds: torch.Tensor, maps, tables,
                                k: int, tau: float, alpha: float, beta: float, chunk_rows: int = 1024):
    """Encoder -> DWN stack -> GroupSum -> mean cross-entropy, forward and backward, walked in row
    chunks so that a full-width network at a batch of several thousand fits in host memory.

    The same composition as `dwn_network_forward` / `dwn_network_backward` around
    `F.cross_entropy(logits, labels)` (mean over ALL rows of x); per-chunk table gradients are added in
    float64 and rounded once.  Returns (logits (B,k) fp32, loss (scalar fp32 tensor), [table grads]).
    """
    B = x.shape[0]
    logits_all, loss_sum = [], 0.0
    grads = [torch.zeros(t.shape, dtype=torch.float64) for t in tables]
    transforms = [None] + [efd_transform(t, alpha, beta) for t in tables[1:]]
    for lo in range(0, B, chunk_rows):
        xs, ys = x[lo:lo + chunk_rows], labels[lo:lo + chunk_rows].long()
        bits = thermometer_encode(xs, thresholds)
        logits, acts = dwn_network_forward(bits, maps, tables, k, tau)
        lg = logits.clone().requires_grad_(True)
        part = F.cross_entropy(lg, ys, reduction="sum")
        part.backward()
        loss_sum += float(part.detach().double())
        for acc, g in zip(grads, dwn_network_backward(acts, maps, tables, lg.grad / B, k, tau, alpha, beta,
                                                    transforms)):
            acc += g.double()
        logits_all.append(logits)
    return torch.cat(logits_all), torch.tensor(loss_sum / B, dtype=torch.float32), [g.float() for g in grads]
