"""Layer-granular autograd functions: gather + node arithmetic in one pass over feature-major data.

The reference runs a Python loop over N node modules on a materialised (B, N, n) tensor
(difflut/layers/random_layer.py:306-340).  Here a layer is one forward kernel and, in backward,
one table-gradient kernel plus one input-gradient kernel; rows <-> feature-major transposes sit
at the API edge only.  `ConnectionPlan` holds the device-side index structures of a layer.
"""

from typing import Optional

import torch

from .. import _native


class ConnectionPlan:
    """Device copies of a fixed (N, n) index map: int32 map per virtual node and its inverse (CSR).

    A node with O outputs appears as O consecutive virtual nodes sharing one map row, so the
    same kernels serve output_dim > 1.  `inv_ptr` (F+1) / `inv_ent` list, per input feature, the
    flat positions v*n+i that read it (sorted, so the backward sums in a fixed order);
    `inv_ent8` holds the same entries packed as (v << 3) | i.
    """

    def __init__(self, mapping: torch.Tensor, input_size: int, out_dim: int, device: torch.device):
        m = mapping.to(device=device, dtype=torch.int64)
        self.N, self.n = int(m.shape[0]), int(m.shape[1])
        self.O = int(out_dim)
        self.input_size = int(input_size)
        if m.numel() and (int(m.min()) < 0 or int(m.max()) >= input_size):
            raise ValueError("mapping indices out of range for input_size")
        self.map_nodes = m.to(torch.int32).contiguous()  # (N, n)
        mv = m.repeat_interleave(self.O, dim=0) if self.O > 1 else m
        self.map_virtual = mv.to(torch.int32).contiguous()  # (N*O, n)
        self.inv_ptr_virtual, self.inv_ent_virtual = self._invert(mv, input_size)
        # the DWN kernels take entries packed as (v << 3) | i instead of v*n + i
        flat = self.inv_ent_virtual.to(torch.int64)
        self.inv_ent8_virtual = (((flat // self.n) << 3) | (flat % self.n)).to(torch.int32).contiguous()
        if self.O > 1:
            self.inv_ptr_nodes, self.inv_ent_nodes = self._invert(m, input_size)
        else:
            self.inv_ptr_nodes, self.inv_ent_nodes = self.inv_ptr_virtual, self.inv_ent_virtual
        self.device = device
        self._ell_nodes = None

    def ell_nodes(self):
        """The inverse map of the nodes as a table interleaved by feature, (max_deg, F) int32: row j holds the
        j-th column (ascending) that each feature collects, -1 where a feature has fewer (built on first use)."""
        if self._ell_nodes is None:
            ptr = self.inv_ptr_nodes.long()
            deg = ptr[1:] - ptr[:-1]
            max_deg = int(deg.max()) if deg.numel() else 0
            F = self.input_size
            ell = torch.full((max(max_deg, 1), F), -1, dtype=torch.int32, device=ptr.device)
            f_of = torch.repeat_interleave(torch.arange(F, device=ptr.device), deg)
            j_of = torch.arange(f_of.numel(), device=ptr.device) - ptr[:-1][f_of]
            ell[j_of, f_of] = self.inv_ent_nodes
            self._ell_nodes = (ell.contiguous(), max_deg)
        return self._ell_nodes

    @staticmethod
    def _invert(m: torch.Tensor, input_size: int):
        flat = m.reshape(-1)
        order = torch.argsort(flat, stable=True)
        counts = torch.bincount(flat, minlength=input_size)
        ptr = torch.zeros(input_size + 1, dtype=torch.int64, device=m.device)
        ptr[1:] = torch.cumsum(counts, 0)
        return ptr.to(torch.int32).contiguous(), order.to(torch.int32).contiguous()


def _rows_to_t(rows: torch.Tensor, Bp: int) -> torch.Tensor:
    B, F = rows.shape
    t = torch.empty(F, Bp, device=rows.device, dtype=torch.float32)
    _native.call("dl_f32_rows_to_t", rows, t, B, F, Bp)
    return t


def _t_to_rows(t: torch.Tensor, B: int) -> torch.Tensor:
    F, Bp = t.shape
    rows = torch.empty(B, F, device=t.device, dtype=torch.float32)
    _native.call("dl_f32_t_to_rows", t, rows, B, F, Bp)
    return rows


def _efd_tables(tables, NO, n, alpha, beta, stable_scale):
    """Per-step backward transform (N*O, n, 32): beta^hamming weights (DWN) or, when `stable_scale` is
    given, 1/(hamming+1) weights times that scale (gradient-stabilised DWN)."""
    import ctypes

    efd = torch.empty(NO, n, 32, device=tables.device, dtype=torch.float32)
    if stable_scale is None:
        _native.call("dl_dwn_prepare", tables, efd, None, NO, n, alpha, beta)
    else:
        w = _native.host_floats([1.0 / (h + 1.0) for h in range(n)])
        scalar = 1.0 if isinstance(stable_scale, torch.Tensor) else float(stable_scale)
        _native.call("dl_dwn_prepare_weighted", tables, efd, None, NO, n, scalar, ctypes.addressof(w))
        if isinstance(stable_scale, torch.Tensor):  # one scale per virtual node
            efd.mul_(stable_scale.reshape(NO, 1, 1))
    return efd


class PatchGeometry:
    """Convolution geometry of an image batch (B, C, H, W): receptive field, stride, zero padding.

    A sample is one patch (b, oy, ox) and a feature one tap (c, ki, kj), in nn.Unfold's order
    (difflut/layers/convolutional.py:170-173,199-205)."""

    def __init__(self, shape, kernel, stride, padding):
        self.B, self.C, self.H, self.W = (int(v) for v in shape)
        self.kh, self.kw = int(kernel[0]), int(kernel[1])
        self.sh, self.sw = int(stride[0]), int(stride[1])
        self.ph, self.pw = int(padding[0]), int(padding[1])
        lib = _native.lib()
        self.OH = int(lib.dl_unfold_positions(self.H, self.kh, self.sh, self.ph))
        self.OW = int(lib.dl_unfold_positions(self.W, self.kw, self.sw, self.pw))
        if self.OH <= 0 or self.OW <= 0:
            raise ValueError(
                f"receptive field {(self.kh, self.kw)} does not fit the padded input {(self.H, self.W)} "
                f"+ 2*{(self.ph, self.pw)}"
            )
        self.P = self.OH * self.OW
        self.S = self.B * self.P  # samples
        self.F = self.C * self.kh * self.kw  # features per sample

    def args(self):
        return (self.B, self.C, self.H, self.W, self.kh, self.kw, self.sh, self.sw, self.ph, self.pw)


class FeatureMajorInput:
    """Marks the input of DWNLayerFunction as fp32 feature-major (I, B) with B a multiple of 128 (what a
    contraction with swapped operands produces); the input gradient comes back in the same layout.

    The marker doubles as a private channel between the two autograd functions of a LearnableLayer: when the
    producer of the input (soft_select_t) sets `want_bf16`, the layer function leaves the input gradient as a
    bf16 (I, B) tensor in `grad_bf16` (the dtype the weight-gradient contraction reads, written once by the
    node kernel instead of fp32 + a conversion pass) and hands autograd a zero-stride placeholder of the right
    shape, which the producer's backward ignores.  Only for disjoint connection plans (`disjoint`).  The same
    channel carries the forward hand-over of packed bits (`want_bits` / `bits_t`)."""

    def __init__(self, disjoint: bool = False, want_bits: bool = False):
        self.disjoint = disjoint
        self.want_bf16 = False
        self.grad_bf16 = None
        # forward direction: the consumer only reads `value >= 0.5`, so the producer may leave the packed bits
        # (I, B / 32) int32 here, written by its contraction's epilogue, and return a zero-stride placeholder
        self.want_bits = want_bits
        self.bits_t = None


class PatchFunction(torch.autograd.Function):
    """x (B, C, H, W) -> patches (B*OH*OW, C*kh*kw) fp32 rows; backward folds the gradient back."""

    @staticmethod
    def forward(ctx, x, geom: PatchGeometry):
        x = x.contiguous().float()
        out = torch.empty(geom.S, geom.F, device=x.device, dtype=torch.float32)
        with torch.cuda.device(x.device):
            _native.call("dl_unfold_rows", x, out, *geom.args())
        ctx.geom = geom
        return out

    @staticmethod
    def backward(ctx, g):
        geom = ctx.geom
        gx = torch.empty(geom.B, geom.C, geom.H, geom.W, device=g.device, dtype=torch.float32)
        with torch.cuda.device(g.device):
            _native.call("dl_fold_rows", g.contiguous().float(), gx, *geom.args())
        return gx, None


class DWNLayerFunction(torch.autograd.Function):
    """RandomLayer(+DWN) training forward/backward: x (B, I) rows, tables (N, O, 2^n) -> (B, N*O).

    Counterpart of EFDFusedFunction (difflut/nodes/dwn_node.py:232-316) with per-node tables.
    With `stable_scale` (a float or a per-virtual-node tensor) the backward is the gradient-stabilised
    variant of difflut/nodes/dwn_stable_node.py:145-205: table gradient times the scale, input gradient
    with 1/(hamming+1) weights times the scale.
    With `geom` the input is an image batch (B, C, H, W) and the layer runs on its patches
    (difflut/layers/convolutional.py:194-205) without materialising them: the patch bits are packed
    straight from the image and the input gradient is folded straight back into it.
    """

    @staticmethod
    def forward(ctx, x, tables, plan: ConnectionPlan, alpha: float, beta: float, stable_scale=None,
                geom: Optional[PatchGeometry] = None):
        tables = tables.contiguous().float()
        feature_major = isinstance(geom, FeatureMajorInput)
        handed_bits = None
        if feature_major and geom.bits_t is not None:
            handed_bits, geom.bits_t = geom.bits_t, None  # x is a placeholder of the right shape: do not touch it
        else:
            x = x.contiguous().float()
        if feature_major:
            I, B = x.shape
            if B % 128 != 0:
                raise ValueError("feature-major input needs a batch that is a multiple of 128")
        elif geom is None:
            B, I = x.shape
        else:
            B, I = geom.S, geom.F
        NO, n = plan.N * plan.O, plan.n
        Bp = _native.padded_batch(B)
        with torch.cuda.device(x.device):
            bits = handed_bits if handed_bits is not None else torch.empty(I, Bp // 32, device=x.device, dtype=torch.int32)
            if handed_bits is not None:
                pass
            elif feature_major:
                _native.call("dl_pack_t_to_t", x, bits, I, B, B, Bp, 0.5)
            elif geom is None:
                _native.call("dl_pack_rows_to_t", x, bits, B, I, Bp, 0.5)
            else:
                _native.call("dl_unfold_pack_t", x, bits, *geom.args(), 0.5, Bp)
            out_t = torch.empty(NO, Bp, device=x.device, dtype=torch.float32)
            _native.call("dl_dwn_fwd_vals_t", bits, plan.map_virtual, tables, out_t, None, NO, n, Bp)
            out = _t_to_rows(out_t, B)
        ctx.save_for_backward(bits, tables)
        ctx.plan, ctx.alpha, ctx.beta, ctx.B, ctx.geom = plan, float(alpha), float(beta), B, geom
        ctx.stable_scale = stable_scale.detach() if isinstance(stable_scale, torch.Tensor) else stable_scale
        return out

    @staticmethod
    def backward(ctx, g):
        bits, tables = ctx.saved_tensors
        plan, B, geom = ctx.plan, ctx.B, ctx.geom
        NO, n, I = plan.N * plan.O, plan.n, plan.input_size
        Bp = bits.shape[1] * 32
        need_x, need_t = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        gx = gt = None
        with torch.cuda.device(g.device):
            g_t = _rows_to_t(g.contiguous().float(), Bp)
            addr = torch.empty(NO, Bp, device=g.device, dtype=torch.uint8) if need_x else None
            gt = torch.empty_like(tables)
            # the table-gradient kernel also produces the addresses the input-gradient kernel reads
            groups = int(_native.lib().dl_dwn_bwd_groups(Bp))
            if groups == 1:
                _native.call("dl_dwn_bwd_tables_t", bits, plan.map_virtual, g_t, 1, 1.0, gt, addr, NO, n, Bp)
            else:
                # large batches: one warp per (1024-sample group, node) and an ordered sum of the groups, so
                # that layers with few nodes still fill the machine
                partial = torch.empty(groups, gt.numel(), device=g.device, dtype=torch.float32)
                _native.call("dl_dwn_bwd_fused_t", None, g_t, 1, 1.0, None, 1, 0, None, None, bits, plan.map_virtual,
                             None, addr, partial, gt.numel(), NO, n, Bp)
                _native.call("dl_sum_groups", partial, gt, gt.numel(), gt.numel(), groups)
            if ctx.stable_scale is not None:
                sc = ctx.stable_scale
                gt = gt * (sc.reshape(gt.shape[0], gt.shape[1], 1) if isinstance(sc, torch.Tensor) else float(sc))
            if need_x:
                efd = _efd_tables(tables, NO, n, ctx.alpha, ctx.beta, ctx.stable_scale)
                if isinstance(geom, FeatureMajorInput) and geom.disjoint:
                    # every feature has one reader: node-major kernel, bf16 rows if the producer asked for them
                    as_bf16 = geom.want_bf16
                    gx_t = torch.empty(I, Bp, device=g.device, dtype=torch.bfloat16 if as_bf16 else torch.float32)
                    _native.call("dl_dwn_bwd_input_disjoint_t", addr, g_t, 1, 1.0, efd, plan.map_virtual, gx_t,
                                 1 if as_bf16 else 0, NO, n, Bp)
                    if as_bf16:
                        geom.grad_bf16 = gx_t
                        return (torch.zeros(1, 1, device=g.device).expand(I, Bp), (gt if need_t else None),
                                None, None, None, None, None)
                    return gx_t, (gt if need_t else None), None, None, None, None, None
                gx_t = torch.empty(I, Bp, device=g.device, dtype=torch.float32)
                _native.call("dl_dwn_bwd_input_t", addr, g_t, 1, 1.0, efd, plan.inv_ptr_virtual,
                             plan.inv_ent8_virtual, gx_t, I, n, Bp)
                if isinstance(geom, FeatureMajorInput):
                    gx = gx_t  # (I, B): B == Bp
                elif geom is None:
                    gx = _t_to_rows(gx_t, B)
                else:
                    gx = torch.empty(geom.B, geom.C, geom.H, geom.W, device=g.device, dtype=torch.float32)
                    _native.call("dl_fold_t", gx_t, gx, *geom.args(), Bp)
        return gx, (gt if need_t else None), None, None, None, None, None


class PackedInput:
    """Marks the first argument of DWNStackFunction as already bit-packed feature-major rows
    (int32 (I, Bp/32), e.g. `ThermometerEncoder.encode_packed_t`) holding `batch` samples."""

    def __init__(self, batch: int, interleaved: bool = False):
        self.B = int(batch)
        self.interleaved = bool(interleaved)  # chunk-interleaved rows (`encode_packed_s`) instead of natural ones


FEW_NODES = 2960  # fewer nodes than resident warps of the fused backward: parallelise over sample groups as well


class StackOptions:
    """How a DWNStackFunction reads its input and what it appends: `source` None (fp32 rows), a
    PatchGeometry (image batch, samples = patches) or a PackedInput (bits already packed); `flip`
    (probability, seed) XORs a Bernoulli mask into the packed input, (probability, 0, positions) flips exactly
    the given positions of the row-major (samples, features) matrix (None: nothing); `head` (k, tau) fuses a following
    GroupSum(k, tau) (difflut/utils/modules.py:116-163) so that the function returns (B, k) logits."""

    def __init__(self, source=None, flip=None, head=None):
        self.source, self.flip, self.head = source, flip, head


class DWNStackFunction(torch.autograd.Function):
    """Consecutive DWN layers (output_dim 1, n <= 6) as one autograd node, bit-packed from end to end.

    A DWN layer only looks at `input >= 0.5`, so between the layers one bit per activation is enough:
    the forward runs the bit-sliced hard-LUT kernel for every level but the last and reads table values
    only there; the backward runs one fused kernel per level (pull the output gradient from the level
    above, form the addresses, accumulate the table gradient) and never goes back to rows in between.
    Same arithmetic as applying DWNLayerFunction level after level (difflut/nodes/dwn_node.py:58-229 per
    node).  `levels` is a list of (plan, alpha, beta, stable_scale); x is (B, I) rows, or with a
    PatchGeometry as `geom` an image batch whose patches are the samples, or with a PackedInput already
    packed bits (no input gradient then); `tables` are the levels' (N, 1, 2^n) tables.
    """

    @staticmethod
    def forward(ctx, x, levels, geom, *tables):
        flip = head = None
        if isinstance(geom, StackOptions):
            flip, head, geom = geom.flip, geom.head, geom.source
        tables = [t.contiguous().float() for t in tables]
        packed = isinstance(geom, PackedInput)
        interleaved_in = packed and geom.interleaved
        if packed:
            B, I = geom.B, x.shape[0]
            geom = None
        elif geom is None:
            x = x.contiguous().float()
            B, I = x.shape
        else:
            x = x.contiguous().float()
            B, I = geom.S, geom.F
        Bp = _native.padded_batch(B)
        Wp = Bp // 32
        dev = x.device
        # with a fused GroupSum every consumer of the activations has a variant for the chunk-interleaved
        # layout, which saves a fifth of the backward's instructions
        swz = head is not None
        Ws = int(_native.lib().dl_swizzled_words(Bp)) if swz else Wp
        if interleaved_in and (not swz or (flip is not None and flip[0] > 0.0)):
            raise ValueError("interleaved packed input needs a fused GroupSum head and no bit flip")
        with torch.cuda.device(dev):
            if packed:
                want = Ws if interleaved_in else Wp
                if x.dtype != torch.int32 or tuple(x.shape) != (I, want) or not x.is_contiguous():
                    raise ValueError(f"packed input must be contiguous int32 ({I}, {want})")
                bits = [x]
            else:
                bits = [torch.empty(I, Wp, device=dev, dtype=torch.int32)]
                if geom is None:
                    _native.call("dl_pack_rows_to_t", x, bits[0], B, I, Bp, 0.5)
                else:
                    _native.call("dl_unfold_pack_t", x, bits[0], *geom.args(), 0.5, Bp)
            if flip is not None and flip[0] > 0.0:
                if packed:
                    bits[0] = bits[0].clone()
                if len(flip) > 2:  # exact count: flip[2] holds the positions in the row-major (B, I) matrix
                    if flip[2] is not None:
                        _native.call("dl_bits_flip_at_t", bits[0], flip[2], flip[2].numel(), I, B, Bp)
                else:
                    _native.call("dl_bits_flip_t", bits[0], I, B, Bp, flip[0], flip[1])
            if swz and not interleaved_in:
                natural = bits[0]
                bits[0] = torch.empty(I, Ws, device=dev, dtype=torch.int32)
                _native.call("dl_bits_swizzle_t", natural, bits[0], I, Bp)
            for (plan, _, _, _), tab in zip(levels[:-1], tables[:-1]):
                masks = torch.empty(plan.N, device=dev, dtype=torch.int64)
                _native.call("dl_dwn_prepare", tab, None, masks, plan.N, plan.n, 0.0, 0.0)
                nxt = torch.empty(plan.N, Ws, device=dev, dtype=torch.int32)
                # bit-sliced: indifferent to where a sample sits in a row, only the row length matters
                _native.call("dl_dwn_fwd_bits_t", bits[-1], plan.map_nodes, masks, nxt, plan.N, plan.n, Ws * 32)
                bits.append(nxt)
            last = levels[-1][0]
            if head is None:
                out_t = torch.empty(last.N, Bp, device=dev, dtype=torch.float32)
                _native.call("dl_dwn_fwd_vals_t", bits[-1], last.map_nodes, tables[-1], out_t, None, last.N, last.n, Bp)
            else:
                k, tau = int(head[0]), float(head[1])
                splits = int(_native.lib().dl_dwn_groupsum_splits(last.N, k))
                partial = torch.empty(k * splits, Bp, device=dev, dtype=torch.float32)
                out_t = torch.empty(k, Bp, device=dev, dtype=torch.float32)
                _native.call("dl_dwn_fwd_groupsum_s", bits[-1], last.map_nodes, tables[-1], partial, out_t, last.N,
                             last.n, k, tau, Bp)
            out = _t_to_rows(out_t, B)
        ctx.save_for_backward(*bits, *tables)
        ctx.levels, ctx.geom, ctx.B, ctx.head, ctx.Bp = levels, geom, B, head, Bp
        return out

    @staticmethod
    def backward(ctx, g):
        levels, geom, B = ctx.levels, ctx.geom, ctx.B
        L = len(levels)
        bits, tables = ctx.saved_tensors[:L], ctx.saved_tensors[L:]
        Bp = ctx.Bp
        fused = "dl_dwn_bwd_fused_s" if ctx.head is not None else "dl_dwn_bwd_fused_t"
        dev = g.device
        need_x = ctx.needs_input_grad[0]
        sizes = [lv[0].N * (1 << lv[0].n) for lv in levels]
        offs = [0]
        for sz in sizes:
            offs.append(offs[-1] + sz)
        total = offs[-1]
        # gradient of the last level's outputs: g itself, or with a fused GroupSum the k class gradients,
        # read as g_t[node / group size] / tau without materialising their broadcast
        gdiv, gscale = 1, 1.0
        if ctx.head is not None:
            k, tau = int(ctx.head[0]), float(ctx.head[1])
            gdiv, gscale = (levels[-1][0].N + k - 1) // k, 1.0 / tau
        with torch.cuda.device(dev):
            g_t = _rows_to_t(g.contiguous().float(), Bp)
            flat = torch.empty(total, device=dev, dtype=torch.float32)  # all levels' table gradients
            efd = [None] * L
            for l in range(L):
                if l > 0 or need_x:
                    plan, alpha, beta, scale = levels[l]
                    efd[l] = _efd_tables(tables[l], plan.N, plan.n, alpha, beta, scale)
            addr = [None] * L
            gact = [None] * L
            gact[L - 1] = g_t
            groups = int(_native.lib().dl_dwn_bwd_groups(Bp))
            for l in range(L - 1, -1, -1):
                plan = levels[l][0]
                below = l > 0 or need_x  # somebody reads this level's addresses and output gradient
                if below:
                    addr[l] = torch.empty(plan.N, Bp, device=dev, dtype=torch.uint8)
                # a level with many nodes adds its sample groups into the gradient in place; one with few nodes
                # writes one slab per group, so that the groups can run side by side, and sums them afterwards
                slabs = groups > 1 and plan.N < FEW_NODES
                if slabs:
                    dst = torch.empty(groups, sizes[l], device=dev, dtype=torch.float32)
                    stride = sizes[l]
                else:
                    dst, stride = flat[offs[l]:], 0
                if l == L - 1:
                    _native.call(fused, None, g_t, gdiv, gscale, None, 1, 0, None, None, bits[l],
                                 plan.map_nodes, None, addr[l], dst, stride, plan.N, plan.n, Bp)
                else:
                    up = levels[l + 1][0]
                    if below:
                        gact[l] = torch.empty(plan.N, Bp, device=dev, dtype=torch.float32)
                    top = l + 1 == L - 1
                    _native.call(fused, addr[l + 1], gact[l + 1], gdiv if top else 1,
                                 gscale if top else 1.0, efd[l + 1], up.n, up.N, up.inv_ptr_virtual, up.inv_ent8_virtual,
                                 bits[l], plan.map_nodes, gact[l], addr[l], dst, stride, plan.N, plan.n, Bp)
                if slabs:
                    _native.call("dl_sum_groups", dst, flat[offs[l]:], sizes[l], sizes[l], groups)
                    if l + 1 < L - 1:
                        gact[l + 1] = None  # the gradient of the level above is no longer needed
            gx = None
            if need_x:
                plan = levels[0][0]
                I = plan.input_size
                gx_t = torch.empty(I, Bp, device=dev, dtype=torch.float32)
                _native.call("dl_dwn_bwd_input_t", addr[0], gact[0], gdiv if L == 1 else 1, gscale if L == 1 else 1.0,
                             efd[0], plan.inv_ptr_virtual, plan.inv_ent8_virtual, gx_t, I, plan.n, Bp)
                if geom is None:
                    gx = _t_to_rows(gx_t, B)
                else:
                    gx = torch.empty(geom.B, geom.C, geom.H, geom.W, device=dev, dtype=torch.float32)
                    _native.call("dl_fold_t", gx_t, gx, *geom.args(), Bp)
        grads = []
        for l in range(L):
            gt = None
            if ctx.needs_input_grad[3 + l]:
                gt = flat[offs[l]:offs[l + 1]].view(tables[l].shape)
                scale = levels[l][3]
                if scale is not None:
                    gt = gt * (scale.reshape(-1, 1, 1) if isinstance(scale, torch.Tensor) else float(scale))
            grads.append(gt)
        return (gx, None, None, *grads)


def dwn_levels_eval(x: torch.Tensor, levels, geom: Optional[PatchGeometry] = None) -> torch.Tensor:
    """Eval forward of consecutive hard-LUT layers on {0,1} inputs, bit-packed from end to end.

    `levels` is a list of (tables (N, O, 2^n), plan); the output of one level is the input of the next.
    x is (B, I) rows, or with `geom` an image batch whose patches are the samples.  Returns the last
    level's fp32 {0,1} rows (dwn_node.py:457-483 applied layer after layer)."""
    packed = isinstance(geom, PackedInput)
    if packed:
        B, I = geom.B, x.shape[0]
    elif geom is None:
        x = x.contiguous().float()
        B, I = x.shape
    else:
        x = x.contiguous().float()
        B, I = geom.S, geom.F
    Bp = _native.padded_batch(B)
    with torch.cuda.device(x.device):
        if packed:
            if x.dtype != torch.int32 or tuple(x.shape) != (I, Bp // 32) or not x.is_contiguous():
                raise ValueError(f"packed input must be contiguous int32 ({I}, {Bp // 32})")
            bits = x
        else:
            bits = torch.empty(I, Bp // 32, device=x.device, dtype=torch.int32)
            if geom is None:
                _native.call("dl_pack_rows_to_t", x, bits, B, I, Bp, 0.5)
            else:
                _native.call("dl_unfold_pack_t", x, bits, *geom.args(), 0.5, Bp)
        for tables, plan in levels:
            tables = tables.detach().contiguous().float()
            NO, n = plan.N * plan.O, plan.n
            masks = torch.empty(NO, device=x.device, dtype=torch.int64)
            _native.call("dl_dwn_prepare", tables, None, masks, NO, n, 0.0, 0.0)
            out_bits = torch.empty(NO, Bp // 32, device=x.device, dtype=torch.int32)
            _native.call("dl_dwn_fwd_bits_t", bits, plan.map_virtual, masks, out_bits, NO, n, Bp)
            bits = out_bits
        out = torch.empty(B, NO, device=x.device, dtype=torch.float32)
        _native.call("dl_bits_t_to_rows", bits, out, B, NO, Bp)
    return out


def dwn_layer_eval(x: torch.Tensor, tables: torch.Tensor, plan: ConnectionPlan) -> torch.Tensor:
    """Eval forward on {0,1} inputs: bit-sliced hard LUTs, fp32 {0,1} rows out (dwn_node.py:457-483)."""
    return dwn_levels_eval(x, [(tables, plan)])


class ProbLayerFunction(torch.autograd.Function):
    """RandomLayer(+Probabilistic) training forward/backward; optional fused GroupSum.

    x (B, I) rows, raw (N, 2^n, O).  With `k` set the function returns the GroupSum logits
    (B, k) instead of the node outputs, without writing the (B, N*O) tensor.
    """

    @staticmethod
    def forward(ctx, x, raw, plan: ConnectionPlan, temperature: float, k: Optional[int], tau: float):
        x = x.contiguous().float()
        raw = raw.contiguous().float()
        B, I = x.shape
        N, n, O = plan.N, plan.n, plan.O
        Bp = _native.padded_batch(B)
        with torch.cuda.device(x.device):
            x_t = _rows_to_t(x, Bp)
            if k is None:
                out_t = torch.empty(N * O, Bp, device=x.device, dtype=torch.float32)
                _native.call("dl_prob_fwd_t", x_t, plan.map_nodes, raw, temperature, out_t, N, n, O, Bp)
                out = _t_to_rows(out_t, B)
            else:
                S = _native.lib().dl_prob_groupsum_splits(N * O, k)
                partial = torch.empty(k * S, Bp, device=x.device, dtype=torch.float32)
                logits_t = torch.empty(k, Bp, device=x.device, dtype=torch.float32)
                _native.call("dl_prob_fwd_groupsum_t", x_t, plan.map_nodes, raw, temperature, None, partial,
                             logits_t, N, n, O, k, tau, Bp)
                out = _t_to_rows(logits_t, B)
        ctx.save_for_backward(x_t, raw)
        ctx.plan, ctx.temperature, ctx.k, ctx.tau, ctx.B = plan, float(temperature), k, float(tau), B
        return out

    @staticmethod
    def backward(ctx, g):
        x_t, raw = ctx.saved_tensors
        plan, B, k = ctx.plan, ctx.B, ctx.k
        N, n, O, I = plan.N, plan.n, plan.O, plan.input_size
        Bp = x_t.shape[1]
        need_x, need_r = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        gx = None
        with torch.cuda.device(g.device):
            g_t = _rows_to_t(g.contiguous().float(), Bp)
            if k is None:
                gdiv, gscale = 1, 1.0
            else:
                gdiv, gscale = (N * O + k - 1) // k, 1.0 / ctx.tau
            graw = torch.empty_like(raw)
            gxm_t = torch.empty(N * n, Bp, device=g.device, dtype=torch.float32) if need_x else None
            _native.call("dl_prob_bwd_t", x_t, plan.map_nodes, raw, ctx.temperature, g_t, gdiv, gscale, graw,
                         gxm_t, N, n, O, B, Bp)
            if need_x:
                gx_t = torch.empty(I, Bp, device=g.device, dtype=torch.float32)
                _native.call("dl_seg_sum_t", gxm_t, plan.inv_ptr_nodes, plan.inv_ent_nodes, gx_t, I, Bp)
                gx = _t_to_rows(gx_t, B)
        return gx, (graw if need_r else None), None, None, None, None


class HybridLayerFunction(torch.autograd.Function):
    """RandomLayer(+Hybrid) training forward/backward: x (B, I) rows, tables (N, O, 2^n) -> (B, N*O).

    Forward is the DWN look-up on `x >= 0.5`; backward is the probabilistic one on the real-valued x
    (HybridFunctionCPU, difflut/nodes/hybrid_node.py:119-224).
    """

    @staticmethod
    def forward(ctx, x, tables, plan: ConnectionPlan):
        x = x.contiguous().float()
        tables = tables.contiguous().float()
        B, I = x.shape
        NO, n = plan.N * plan.O, plan.n
        Bp = _native.padded_batch(B)
        with torch.cuda.device(x.device):
            x_t = _rows_to_t(x, Bp)
            bits = torch.empty(I, Bp // 32, device=x.device, dtype=torch.int32)
            _native.call("dl_pack_rows_to_t", x, bits, B, I, Bp, 0.5)
            out_t = torch.empty(NO, Bp, device=x.device, dtype=torch.float32)
            _native.call("dl_dwn_fwd_vals_t", bits, plan.map_virtual, tables, out_t, None, NO, n, Bp)
            out = _t_to_rows(out_t, B)
        ctx.save_for_backward(x_t, tables)
        ctx.plan, ctx.B = plan, B
        return out

    @staticmethod
    def backward(ctx, g):
        x_t, tables = ctx.saved_tensors
        plan, B = ctx.plan, ctx.B
        N, n, O, I = plan.N, plan.n, plan.O, plan.input_size
        Bp = x_t.shape[1]
        need_x, need_t = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        gx = None
        with torch.cuda.device(g.device):
            g_t = _rows_to_t(g.contiguous().float(), Bp)
            gt = torch.empty_like(tables)
            gxm_t = torch.empty(N * n, Bp, device=g.device, dtype=torch.float32) if need_x else None
            _native.call("dl_hybrid_bwd_t", x_t, plan.map_nodes, tables, g_t, 1, 1.0, gt, gxm_t, N, n, O, B, Bp)
            if need_x:
                gx_t = torch.empty(I, Bp, device=g.device, dtype=torch.float32)
                _native.call("dl_seg_sum_t", gxm_t, plan.inv_ptr_nodes, plan.inv_ent_nodes, gx_t, I, Bp)
                gx = _t_to_rows(gx_t, B)
        return gx, (gt if need_t else None), None


class GatherFunction(torch.autograd.Function):
    """x (B, I) -> (B, N, n): the materialised mapping `get_mapping` returns.

    Counterpart of MappingFunction (difflut/layers/random_layer.py:34-100); the backward is a
    segmented sum over the inverse map instead of fp32 atomics.
    """

    @staticmethod
    def forward(ctx, x, plan: ConnectionPlan):
        x = x.contiguous().float()
        B, I = x.shape
        out = torch.empty(B, plan.N, plan.n, device=x.device, dtype=torch.float32)
        with torch.cuda.device(x.device):
            _native.call("dl_gather_rows", x, plan.map_nodes, out, B, I, plan.N, plan.n)
        ctx.plan, ctx.B = plan, B
        return out

    @staticmethod
    def backward(ctx, g):
        plan, B = ctx.plan, ctx.B
        g = g.contiguous().float()
        gx = torch.empty(B, plan.input_size, device=g.device, dtype=torch.float32)
        with torch.cuda.device(g.device):
            M = plan.N * plan.n
            if M % 4 == 0 and M >= 16384 and B >= 64:
                # wide gradient rows: shared-memory staged rows and the feature-interleaved entry table
                ell, max_deg = plan.ell_nodes()
                _native.call("dl_gather_rows_bwd_ell", g, ell, max_deg, gx, B, plan.input_size, plan.N, plan.n)
            else:
                _native.call("dl_gather_rows_bwd", g, plan.inv_ptr_nodes, plan.inv_ent_nodes, gx, B,
                             plan.input_size, plan.N, plan.n)
        return gx, None
