"""Fused execution of an encoder -> RandomLayer(DWN) x L -> GroupSum classifier.

The per-layer API (`RandomLayer.forward`) is exact to the reference's tensors: fp32 rows in and
out of every layer.  A DWN layer only looks at `input >= 0.5`, so between layers one bit per
activation is enough; this module runs the same kernels on that representation end to end:

  forward   thermometer compare-and-pack -> bit-sliced hard LUT layers -> last layer fused with
            GroupSum (logits), one kernel per layer, activations bit-packed feature-major;
  backward  cross-entropy, then per layer one table-gradient kernel (lane-private histograms)
            and one input-gradient kernel (segmented pull over the inverse map using the
            per-step EFD transform); gradients are fp32 feature-major;
  update    table gradients of all layers live in ONE flat buffer which is all-reduced (NCCL,
            data parallel over the batch) and consumed by one fused Adam kernel.

The parameters are the layers' own `luts` tensors (re-pointed into the flat buffer), so the
API objects and this executor always see the same tables.  Equivalent reference code: user
model + loop as in examples/demo_probabilistic_random.py:111-178 with DWN nodes.
"""

from typing import Optional, Sequence

import os

import torch
import torch.distributed as dist

from . import _native
from .distributed import allreduce_sum_
from .encoder.thermometer import ThermometerEncoder
from .layers.random_layer import RandomLayer
from .utils.modules import GroupSum


class DWNNetwork:
    def __init__(self, encoder: ThermometerEncoder, layers: Sequence[RandomLayer], groupsum: GroupSum,
                 lr: float = 1e-2, betas=(0.9, 0.999), eps: float = 1e-8,
                 process_group: Optional["dist.ProcessGroup"] = None, distributed: Optional[bool] = None,
                 fused_backward: bool = True, peer_optimizer: Optional[bool] = None, peer_status_every: int = 0):
        if not encoder.is_fitted:
            raise RuntimeError("DWNNetwork needs a fitted encoder")
        if groupsum.use_randperm:
            raise ValueError("DWNNetwork does not support GroupSum(use_randperm=True)")
        for l in layers:
            if l._stacked != "dwn" or l.n > 6 or l.output_dim_per_node != 1:
                raise ValueError("DWNNetwork takes RandomLayer(DWNNode) layers with n <= 6 and output_dim 1")
            if l.flip_probability > 0.0 or l.grad_stabilization != "none":
                # the per-layer API applies these options (layers/base_layer.py); this executor keeps the
                # activations bit-packed between layers and does not, so it refuses instead of ignoring them
                raise ValueError("DWNNetwork does not apply flip_probability / grad_stabilization; "
                                 "use the layer API (or DWNStack without these options) for such layers")
        self.encoder, self.layers, self.groupsum = encoder, list(layers), groupsum
        self.device = self.layers[0].luts.device
        if self.device.type != "cuda":
            raise RuntimeError("DWNNetwork needs its layers on a CUDA device (no CPU fallback)")
        self.lr, self.betas, self.eps = float(lr), (float(betas[0]), float(betas[1])), float(eps)
        self.k, self.tau = int(groupsum.k), float(groupsum.tau)
        self.group = process_group
        self.fused_backward = bool(fused_backward)
        # the fused stack kernels read the activations in the chunk-interleaved bit layout
        self.swizzle = self.fused_backward
        if distributed is None:
            distributed = dist.is_available() and dist.is_initialized() and dist.get_world_size(process_group) > 1
        self.distributed = bool(distributed)
        self.world = dist.get_world_size(process_group) if self.distributed else 1
        self.rank = dist.get_rank(process_group) if self.distributed else 0
        # gradient all-reduce + Adam + parameter broadcast as one kernel over peer memory (one node, NCCL
        # process group, at most 8 ranks); DIFFLUT_PEER_OPTIMIZER=0 keeps the NCCL all-reduce path
        if peer_optimizer is None:
            peer_optimizer = (self.distributed and self.fused_backward and self.world <= 8
                              and dist.get_backend(process_group) == "nccl"
                              and os.environ.get("DIFFLUT_PEER_OPTIMIZER", "1") != "0")
        self.peer_optimizer = bool(peer_optimizer) and self.distributed
        # > 0: train_step reads the peer status word every that many steps (a host synchronisation) and raises
        # when a bounded wait has given up; 0 leaves the polling to the caller (peer_status())
        self.peer_status_every = int(peer_status_every)

        thr = encoder.thresholds.reshape(-1, encoder.num_bits)
        self.thr = thr.to(device=self.device, dtype=torch.float32).contiguous()
        self.F, self.T = int(self.thr.shape[0]), int(encoder.num_bits)
        sizes_in = [self.F * self.T] + [l.output_size for l in self.layers[:-1]]
        for l, i in zip(self.layers, sizes_in):
            if l.input_size != i:
                raise ValueError(f"layer input_size {l.input_size} does not match the {i} features feeding it")
        self.n = [l.n for l in self.layers]
        self.N = [l.output_size for l in self.layers]
        self.I = sizes_in
        self.L = [2 ** n for n in self.n]

        # one flat buffer for all tables / gradients / Adam moments; the layers' parameters view it
        self.counts = [N * L for N, L in zip(self.N, self.L)]
        # with the peer optimiser every layer's slice splits into `world` equal runs of whole 16-byte pieces
        unit = 4 * self.world if self.peer_optimizer else 1
        self.offsets, self.padded = [0], []
        for c in self.counts:
            self.padded.append((c + unit - 1) // unit * unit)
            self.offsets.append(self.offsets[-1] + self.padded[-1])
        total = self.offsets[-1]
        moments = total // self.world if self.peer_optimizer else total
        # one exchange kernel per layer (its own flag channel) unless there are more layers than channels
        # (DIFFLUT_PEER_PER_LAYER=1 starts it per layer under the backward of the layers below: measured slower,
        # every exchange is a rendezvous of all ranks)
        self.peer_fused = os.environ.get("DIFFLUT_PEER_FUSED", "1") != "0"
        self.peer_per_layer = len(self.layers) <= 8 and os.environ.get("DIFFLUT_PEER_PER_LAYER", "0") == "1"
        # the exchange does not wait for the peers' "done": the next step (or any read of the tables) does
        self.peer_defer_done = os.environ.get("DIFFLUT_PEER_DEFER_DONE", "1") != "0"
        self.flat = torch.zeros(total, device=self.device, dtype=torch.float32)
        self.flat_grad = torch.zeros(total, device=self.device, dtype=torch.float32)
        self.exp_avg = torch.zeros(moments, device=self.device, dtype=torch.float32)
        self.exp_avg_sq = torch.zeros(moments, device=self.device, dtype=torch.float32)
        self.adam_state = torch.ones(2, device=self.device, dtype=torch.float64)
        self.tables, self.grads = [], []
        for li, l in enumerate(self.layers):
            sl = slice(self.offsets[li], self.offsets[li] + self.counts[li])
            view = self.flat[sl].view(self.N[li], 1, self.L[li])
            view.copy_(l.luts.data)
            l.luts.data = view
            gview = self.flat_grad[sl].view(self.N[li], 1, self.L[li])
            l.luts.grad = gview
            self.tables.append(view)
            self.grads.append(gview)
        if self.peer_optimizer:
            from .distributed import PeerWindow

            # flag words per rank: an "arrive" and a "done" epoch per channel and peer (the separate barrier
            # kernel of the unfused path uses the first 8); ctrl: status + (epoch, CTA counter) per channel
            self.peer_flags = torch.zeros(8 * 2 * 8, device=self.device, dtype=torch.int32)
            self.peer_ctrl = torch.zeros(1 + 2 * 8, device=self.device, dtype=torch.int32)
            self.peer_ctrl_barrier = torch.zeros(2, device=self.device, dtype=torch.int32)
            torch.cuda.synchronize(self.device)
            self.peer_timeout_ms = 5000
            try:
                # a window either exists on every rank or raises on every rank
                self.win_params = PeerWindow(self.flat, process_group)
                self.win_grads = PeerWindow(self.flat_grad, process_group)
                self.win_flags = PeerWindow(self.peer_flags, process_group)
            except RuntimeError as e:
                import warnings

                warnings.warn(f"DWNNetwork: {e}; exchanging gradients with NCCL all-reduces instead", RuntimeWarning)
                self.peer_optimizer = False
                self.exp_avg = torch.zeros(total, device=self.device, dtype=torch.float32)
                self.exp_avg_sq = torch.zeros(total, device=self.device, dtype=torch.float32)
        self.plans = [l._plan(self.device) for l in self.layers]
        self.alpha = [l.alpha for l in self.layers]
        self.beta = [l.beta for l in self.layers]
        # per-step derived tables of all layers in one buffer each (layers are slices): when every
        # layer has the same n / alpha / beta, one kernel launch prepares the whole network
        nodes_total = sum(self.N)
        self.uniform = len(set(self.n)) == 1 and len(set(self.alpha)) == 1 and len(set(self.beta)) == 1
        self.masks_all = torch.empty(nodes_total, device=self.device, dtype=torch.int64)
        self.efd_all = torch.empty(sum(N * n * 32 for N, n in zip(self.N, self.n)), device=self.device,
                                   dtype=torch.float32)
        self.masks, self.efd, node_off, efd_off = [], [], 0, 0
        for N, n in zip(self.N, self.n):
            self.masks.append(self.masks_all[node_off:node_off + N])
            self.efd.append(self.efd_all[efd_off:efd_off + N * n * 32].view(N, n, 32))
            node_off += N
            efd_off += N * n * 32
        self.gsz = (self.N[-1] + self.k - 1) // self.k
        self.splits = int(_native.lib().dl_dwn_groupsum_splits(self.N[-1], self.k))
        self._B = None
        self._train_B = None
        self._graph = None
        self._graph_B_global = None
        # graphs captured on a caller's own input tensor (no copy into the static buffer), by input address
        self._direct_graphs = {}
        self._direct_seen = {}
        self._x_src = None
        self._y_src = None
        self.max_direct_graphs = 4
        self._side = None
        self._comm = None
        self._peer_channels = set()
        self.step_count = 0
        self.infer_chunk = 1 << 18  # hard inference walks large batches in pieces of this many samples

    # ------------------------------------------------------------------ buffers
    def _ensure_buffers(self, B: int, training: bool = True) -> None:
        """Activation buffers for a batch of B samples; gradient-side buffers only when training."""
        dev = self.device
        if self._B != B:
            Bp = _native.padded_batch(B)
            self.Bp = Bp
            # interleaved rows are whole 1024-sample blocks; the natural-layout kernels (hard inference)
            # use the same buffers with Bp/32 words per row
            Wp = int(_native.lib().dl_swizzled_words(Bp)) if self.swizzle else Bp // 32
            self.Bp_bits = Wp * 32
            self.bits = [torch.empty(self.I[0], Wp, device=dev, dtype=torch.int32)]
            for N in self.N[:-1]:
                self.bits.append(torch.empty(N, Wp, device=dev, dtype=torch.int32))
            self.last_bits = torch.empty(self.N[-1], Wp, device=dev, dtype=torch.int32)
            self.partial = torch.empty(self.k * self.splits, Bp, device=dev, dtype=torch.float32)
            self.logits_t = torch.empty(self.k, Bp, device=dev, dtype=torch.float32)
            self._B = B
            self._train_B = None
            self._graph = None
            self._direct_graphs, self._direct_seen = {}, {}
        if training and self._train_B != B:
            Bp = self.Bp
            # gradient w.r.t. the output of layer li (li < last), produced by layer li+1's backward; the
            # fused backward never materialises it for the first layer
            self.gact = [torch.empty(N, Bp, device=dev, dtype=torch.float32)
                         if (li > 0 or not self.fused_backward) else None for li, N in enumerate(self.N[:-1])]
            self.groups = int(_native.lib().dl_dwn_bwd_groups(Bp))
            self.addr = [None] + [torch.empty(N, Bp, device=dev, dtype=torch.uint8) for N in self.N[1:]]
            self.dlogits_t = torch.empty(self.k, Bp, device=dev, dtype=torch.float32)
            self.loss_rows = torch.empty(Bp, device=dev, dtype=torch.float32)
            self.loss = torch.zeros(1, device=dev, dtype=torch.float32)
            self.x_static = torch.empty(B, self.F, device=dev, dtype=torch.float32)
            self.y_static = torch.empty(B, device=dev, dtype=torch.int32)
            self._train_B = B
            self._graph = None
            self._direct_graphs, self._direct_seen = {}, {}

    # ------------------------------------------------------------------ kernels
    def _prepare_tables(self, need_efd: bool, need_masks: bool = True) -> None:
        """EFD transform tables (for the backward) and >= 0.5 masks (for the hard forward) of this step."""
        if not (need_efd or need_masks):
            return
        if self.uniform:
            _native.call("dl_dwn_prepare", self.flat, self.efd_all if need_efd else None,
                         self.masks_all if need_masks else None, sum(self.N), self.n[0], self.alpha[0], self.beta[0])
            return
        for li in range(len(self.layers)):
            _native.call("dl_dwn_prepare", self.tables[li], self.efd[li] if need_efd else None,
                         self.masks[li] if need_masks else None, self.N[li], self.n[li], self.alpha[li], self.beta[li])

    def _forward(self, x: torch.Tensor, B: int) -> None:
        self._encode(x, B)
        self._forward_layers()

    def _encode(self, x: torch.Tensor, B: int) -> None:
        if self.swizzle:
            _native.call("dl_thermo_pack_s", x, self.thr, self.bits[0], B, self.F, self.T, self.Bp)
        else:
            _native.call("dl_thermo_pack_t", x, self.thr, self.bits[0], B, self.F, self.T, self.Bp)

    def _forward_layers(self, with_loss=None) -> None:
        """Hidden layers (bit-sliced) and the last layer fused with GroupSum; with `with_loss` = (B, B_global)
        the kernel that reduces the class sums also does the cross-entropy (gradient of the logits and
        per-sample losses), one launch fewer on the way to the backward."""
        Bp = self.Bp
        last = len(self.layers) - 1
        for li in range(last):
            # bit-sliced: indifferent to the sample order inside a row, only the row length matters
            _native.call("dl_dwn_fwd_bits_t", self.bits[li], self.plans[li].map_nodes, self.masks[li],
                         self.bits[li + 1], self.N[li], self.n[li], self.Bp_bits)
        if with_loss is not None and self.swizzle and self.k <= 128:
            _native.call("dl_dwn_fwd_groupsum_ce_s", self.bits[last], self.plans[last].map_nodes, self.tables[last],
                         self.partial, self.logits_t, self._labels(), self.dlogits_t, self.loss_rows, self.N[last],
                         self.n[last], self.k, self.tau, with_loss[0], with_loss[1], Bp)
            return
        _native.call("dl_dwn_fwd_groupsum_s" if self.swizzle else "dl_dwn_fwd_groupsum_t", self.bits[last],
                     self.plans[last].map_nodes, self.tables[last], self.partial, self.logits_t, self.N[last],
                     self.n[last], self.k, self.tau, Bp)
        if with_loss is not None:
            _native.call("dl_ce_t", self.logits_t, self._labels(), self.dlogits_t, self.loss_rows, None,
                         with_loss[0], with_loss[1], self.k, Bp)

    def _labels(self) -> torch.Tensor:
        return self.y_static if self._y_src is None else self._y_src

    def _backward(self) -> None:
        if self.fused_backward:
            return self._backward_fused()
        Bp = self.Bp
        last = len(self.layers) - 1
        for li in range(last, -1, -1):
            if li == last:
                g, gdiv, gscale = self.dlogits_t, self.gsz, 1.0 / self.tau
            else:
                g, gdiv, gscale = self.gact[li], 1, 1.0
            _native.call("dl_dwn_bwd_tables_t", self.bits[li], self.plans[li].map_nodes, g, gdiv, gscale,
                         self.grads[li], self.addr[li], self.N[li], self.n[li], Bp)
            if li > 0:
                _native.call("dl_dwn_bwd_input_t", self.addr[li], g, gdiv, gscale, self.efd[li],
                             self.plans[li].inv_ptr_virtual, self.plans[li].inv_ent8_virtual, self.gact[li - 1],
                             self.I[li], self.n[li], Bp)

    def _backward_fused(self) -> None:
        """One kernel per layer (top down).  Each kernel adds the table gradient of one 1024-sample group
        after the other straight into the flat gradient buffer (group stride 0: a node belongs to the same
        warp in every group, so the sum has a fixed order and no scratch slabs are needed).  Under NCCL
        data parallelism each layer's all-reduce is started as soon as its slice is complete, so it travels
        while the layers below are still computed."""
        Bp = self.Bp
        last = len(self.layers) - 1
        fused = "dl_dwn_bwd_fused_s" if self.swizzle else "dl_dwn_bwd_fused_t"
        self._pending = []
        for li in range(last, -1, -1):
            grad_out = self.flat_grad[self.offsets[li]:]
            if li == last:
                _native.call(fused, None, self.dlogits_t, self.gsz, 1.0 / self.tau, None, 1, 0, None, None,
                             self.bits[li], self.plans[li].map_nodes, None, self.addr[li], grad_out, 0,
                             self.N[li], self.n[li], Bp)
            else:
                up = li + 1
                if up == last:
                    g_up, gdiv, gscale = self.dlogits_t, self.gsz, 1.0 / self.tau
                else:
                    g_up, gdiv, gscale = self.gact[up], 1, 1.0
                _native.call(fused, self.addr[up], g_up, gdiv, gscale, self.efd[up], self.n[up], self.N[up],
                             self.plans[up].inv_ptr_virtual, self.plans[up].inv_ent8_virtual, self.bits[li],
                             self.plans[li].map_nodes, self.gact[li] if li > 0 else None,
                             self.addr[li] if li > 0 else None, grad_out, 0, self.N[li], self.n[li], Bp)
            if self.distributed and not self.peer_optimizer:
                # sum of per-rank gradients of the GLOBAL-mean loss (dl_ce_t divides by B_global)
                grad = self.flat_grad[self.offsets[li]:self.offsets[li] + self.counts[li]]
                self._pending.append(allreduce_sum_(grad, self.group, async_op=True))
            elif self.peer_optimizer and self.peer_fused and self.peer_per_layer:
                # this layer's gradient is complete on this rank: its exchange (all ranks arrive -> reduce + Adam
                # on the owner -> store everywhere -> all ranks done) runs on the communication stream under
                # the backward of the layers below; the first layer's exchange also advances the Adam state
                main = torch.cuda.current_stream()
                self._comm_events[li].record(main)
                self._comm.wait_event(self._comm_events[li])
                with torch.cuda.stream(self._comm):
                    # every exchange but the first layer's runs next to a backward kernel
                    self._exchange(self.offsets[li], self.padded[li], channel=li, advance=(li == 0), overlapped=li > 0)

    def _exchange(self, offset: int, count: int, channel: int, advance: bool, overlapped: bool = False) -> None:
        _native.call("dl_p2p_exchange_adam", self.win_grads.ptrs, self.win_params.ptrs, self.win_flags.ptrs,
                     self.exp_avg, self.exp_avg_sq, self.adam_state, self.peer_ctrl, offset, count, channel,
                     1 if advance else 0, 1 if overlapped else 0, 1 if self.peer_defer_done else 0, self.rank,
                     self.world, self.lr, self.betas[0], self.betas[1], self.eps, 1.0, self.peer_timeout_ms)
        self._peer_channels.add(channel)

    def _peer_wait_done(self) -> None:
        """Every rank's parameter stores of the latest exchange have landed here and every rank has finished
        reading this rank's gradients (second half of the exchange's rendezvous, see `peer_defer_done`)."""
        if self.peer_optimizer and self.peer_fused and self.peer_defer_done:
            for ch in sorted(self._peer_channels):
                _native.call("dl_p2p_wait_done", self.win_flags.ptrs, self.peer_ctrl, ch, self.rank, self.world,
                             self.peer_timeout_ms)

    def _step_body(self, B: int, B_global: int) -> None:
        """One step as a small dependency graph over three streams (captured as such into the CUDA graph):
        the table preparation (hard masks for the forward, then the EFD transform for the backward) and
        the loss sum run on a side stream next to the encoder / forward / backward chain, and with the peer
        optimiser each layer's gradient exchange runs on a communication stream under the backward of the
        layers below."""
        main = torch.cuda.current_stream()
        if self._side is None:
            self._side = torch.cuda.Stream(device=self.device)
            self._comm = torch.cuda.Stream(device=self.device)
            self._fork, self._masks_ready, self._efd_ready = torch.cuda.Event(), torch.cuda.Event(), torch.cuda.Event()
            self._ce_done, self._side_done, self._comm_done = torch.cuda.Event(), torch.cuda.Event(), torch.cuda.Event()
            self._comm_events = [torch.cuda.Event() for _ in self.layers]
        self._fork.record(main)
        self._side.wait_event(self._fork)
        with torch.cuda.stream(self._side):
            self._peer_wait_done()  # the previous step's exchange, before the tables are read again
            self._prepare_tables(need_efd=False, need_masks=True)
            self._masks_ready.record(self._side)
            self._prepare_tables(need_efd=True, need_masks=False)
            self._efd_ready.record(self._side)
        self._encode(self.x_static if self._x_src is None else self._x_src, B)
        main.wait_event(self._masks_ready)
        self._forward_layers(with_loss=(B, B_global))
        self._ce_done.record(main)
        with torch.cuda.stream(self._side):
            self._side.wait_event(self._ce_done)
            _native.call("dl_loss_sum", self.loss_rows, self.loss, B_global, self.Bp)
            if not self.peer_optimizer:
                # the optimiser's step counter and bias corrections advance here, off the critical path
                _native.call("dl_adam_advance", self.adam_state, self.betas[0], self.betas[1])
            self._side_done.record(self._side)
        main.wait_event(self._efd_ready)
        fused_exchange = self.peer_optimizer and self.peer_fused and self.peer_per_layer and self.fused_backward
        if fused_exchange:
            self._comm.wait_event(self._fork)
        self._backward()
        count = self.flat.numel()
        if self.peer_optimizer:
            if fused_exchange:
                self._comm_done.record(self._comm)
                main.wait_event(self._comm_done)
            elif self.peer_fused:
                self._exchange(0, count, channel=0, advance=True)
            else:
                # three-kernel form: every rank's gradients are complete -> each rank reduces and updates its
                # slice and stores the new parameters everywhere -> every rank's stores have landed
                barrier = (self.win_flags.ptrs, self.rank, self.world, self.peer_ctrl_barrier, self.peer_timeout_ms)
                _native.call("dl_p2p_barrier", *barrier)
                _native.call("dl_p2p_reduce_adam", self.win_grads.ptrs, self.win_params.ptrs, self.exp_avg,
                             self.exp_avg_sq, self.adam_state, self.peer_ctrl_barrier, count, self.rank, self.world,
                             self.lr, self.betas[0], self.betas[1], self.eps, 1.0)
                _native.call("dl_p2p_barrier", *barrier)
        else:
            # (the update of a layer's tables could start as soon as that layer's gradient is complete, under the
            # backward of the layers below; measured, that is slower: the backward kernels divide their work
            # statically over a grid that fills the GPU, and any CTA that has to start late ends the kernel late)
            if self.distributed:
                if self.fused_backward:
                    for work in self._pending:  # the per-layer all-reduces started during the backward
                        if work is not None:
                            work.wait()
                    self._pending = []
                else:
                    allreduce_sum_(self.flat_grad, self.group)
            main.wait_event(self._side_done)
            _native.call("dl_adam_apply", self.flat, self.flat_grad, self.exp_avg, self.exp_avg_sq, self.adam_state,
                         count, self.lr, self.betas[0], self.betas[1], self.eps, 1.0)
        main.wait_event(self._side_done)

    # ------------------------------------------------------------------ public API
    def peer_status(self) -> int:
        """0, or 1 + the rank a bounded peer wait gave up on (synchronises; call it between steps)."""
        if not self.peer_optimizer:
            return 0
        with torch.cuda.device(self.device):
            self._peer_wait_done()  # after this the tables are complete on this rank
        return int(self.peer_ctrl[0].item()) if self.peer_fused else int(self.peer_ctrl_barrier[1].item())

    def host_pipeline(self, x_pinned: torch.Tensor, labels_pinned: torch.Tensor,
                      loss_pinned: Optional[torch.Tensor] = None, global_batch: Optional[int] = None):
        """A training loop whose batches arrive in pinned host memory: returns an object whose `step()` is ONE
        graph launch that trains on the batch copied to the device during the previous step, copies the batch
        now in the pinned buffers to the other device slot meanwhile, and writes the step's loss to pinned
        memory.  See `HostPipeline`."""
        return HostPipeline(self, x_pinned, labels_pinned, loss_pinned, global_batch)

    def kernel_launches_per_step(self) -> int:
        L = len(self.layers)
        backward = L if self.fused_backward else (L + (L - 1))
        prepare = 2 * (1 if self.uniform else L)
        if not self.peer_optimizer:
            update = 2  # state advance, Adam
        elif self.peer_fused:
            update = L if self.peer_per_layer else 1  # one exchange kernel per layer
            if self.peer_defer_done:
                update += 1  # the deferred second rendezvous, waited for at the next step's start
        else:
            update = 4  # barrier, state advance, reduce+Adam+broadcast, barrier
        head = 3 if (self.swizzle and self.k <= 128) else 4  # last layer, reduce (+ cross-entropy), loss sum
        return prepare + 1 + (L - 1) + head + backward + update

    def train_step(self, x: torch.Tensor, labels: torch.Tensor, use_graph: bool = False,
                   global_batch: Optional[int] = None) -> torch.Tensor:
        """One optimisation step on this rank's shard (x (B, F) fp32, labels (B,) integer in [0, k)).

        Returns the 1-element device tensor holding this rank's share of the global mean loss
        (sum over ranks = global mean).  With `use_graph` the step is captured once per batch
        size into a CUDA graph and replayed.  `global_batch` is the number of rows all ranks hold
        together (the denominator of the mean loss); it defaults to B * world, which is only right
        when every rank holds the same number of rows: pass it when the shards are uneven.

        With the peer optimiser a non-zero `peer_status()` means a rank did not arrive within the
        limit; the tables are invalid from the step in which that happened (later steps change
        nothing), so poll it at every host synchronisation point of the training loop.
        """
        B = int(x.shape[0])
        if not labels.is_cuda and labels.numel() > 0 and (int(labels.min()) < 0 or int(labels.max()) >= self.k):
            raise ValueError(f"labels must lie in [0, {self.k})")
        with torch.cuda.device(self.device):
            self._ensure_buffers(B)
            B_global = B * self.world if global_batch is None else int(global_batch)
            if B_global < B:
                raise ValueError("global_batch is smaller than this rank's batch")
            self.y_static.copy_(labels, non_blocking=True)
            # An input tensor that comes back (a training loop's own device buffer) gets a graph captured on its
            # address from its second appearance on: the encoder then reads it in place.  Any other input is
            # copied into the static buffer the general graph reads.
            key = None
            if (use_graph and x.is_cuda and x.device == self.device and x.dtype == torch.float32
                    and x.is_contiguous() and x.data_ptr() % 16 == 0 and tuple(x.shape) == (B, self.F)):
                key = (x.data_ptr(), B, B_global)
            direct = self._direct_graphs.get(key) if key is not None else None
            if direct is None and key is not None and self._direct_seen.get(key, 0) >= 1 \
                    and len(self._direct_graphs) < self.max_direct_graphs and self._graph is not None:
                self._x_src = x
                try:
                    direct = (self._capture_graph(B, B_global), x)  # the tensor is kept alive with its graph
                finally:
                    self._x_src = None
                self._direct_graphs[key] = direct
            if direct is not None:
                direct[0].replay()
            else:
                if key is not None:
                    if len(self._direct_seen) > 64:
                        self._direct_seen = {}
                    self._direct_seen[key] = self._direct_seen.get(key, 0) + 1
                self.x_static.copy_(x, non_blocking=True)
                if self._graph is not None and self._graph_B_global != B_global:
                    self._graph = None  # the denominator is baked into the captured launches
                if not use_graph:
                    self._step_body(B, B_global)
                else:
                    if self._graph is None:
                        self._capture(B, B_global)
                    self._graph.replay()
        self.step_count += 1
        if self.peer_optimizer and self.peer_status_every > 0 and self.step_count % self.peer_status_every == 0:
            status = self.peer_status()
            if status != 0:
                raise RuntimeError(f"peer exchange: rank {status - 1} did not arrive within {self.peer_timeout_ms} ms; "
                                   "the tables are invalid since the last successful poll")
        return self.loss

    def _capture(self, B: int, B_global: int) -> None:
        # run once eagerly on a side stream (warms NCCL and the allocator), restoring the state after
        snap = (self.flat.clone(), self.exp_avg.clone(), self.exp_avg_sq.clone(), self.adam_state.clone())
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            self._step_body(B, B_global)
            self._peer_wait_done()  # no peer may still be storing into the tables that are restored below
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize(self.device)
        self.flat.copy_(snap[0]); self.exp_avg.copy_(snap[1]); self.exp_avg_sq.copy_(snap[2])
        self.adam_state.copy_(snap[3])
        self._graph = self._capture_graph(B, B_global)
        self._graph_B_global = B_global

    def _capture_graph(self, B: int, B_global: int):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self._step_body(B, B_global)
        return graph

    @torch.no_grad()
    def logits(self, x: torch.Tensor) -> torch.Tensor:
        """Training-mode logits (B, k) fp32 = GroupSum(last layer's raw table values)."""
        B = int(x.shape[0])
        with torch.cuda.device(self.device):
            self._ensure_buffers(B, training=False)
            self._peer_wait_done()
            self._prepare_tables(need_efd=False)
            self._forward(x.contiguous().float(), B)
            out = torch.empty(B, self.k, device=self.device, dtype=torch.float32)
            _native.call("dl_f32_t_to_rows", self.logits_t, out, B, self.k, self.Bp)
        return out

    @torch.no_grad()
    def hard_counts(self, x: Optional[torch.Tensor] = None, packed_rows: Optional[torch.Tensor] = None,
                    out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Eval-mode class counts (B, k) int32 of the binarised network (every table >= 0.5).

        Input is either raw features x (B, F) fp32 or thermometer bits already packed as rows
        (B, ceil(F*T/32)) int32 with bit c%32 of word c//32 = encoded column c.
        """
        src = packed_rows if packed_rows is not None else x.contiguous().float()
        B_total = int(src.shape[0])
        with torch.cuda.device(self.device):
            if out is None:
                out = torch.empty(B_total, self.k, device=self.device, dtype=torch.int32)
            self._peer_wait_done()
            self._prepare_tables(need_efd=False)
            for lo in range(0, B_total, self.infer_chunk):
                hi = min(lo + self.infer_chunk, B_total)
                B = hi - lo
                self._ensure_buffers(B, training=False)
                piece = src[lo:hi]
                if packed_rows is not None:
                    _native.call("dl_bits_rows_to_t", piece, self.bits[0], B, self.I[0], piece.shape[1], self.Bp)
                else:
                    _native.call("dl_thermo_pack_t", piece, self.thr, self.bits[0], B, self.F, self.T, self.Bp)
                cur = self.bits[0]
                for li in range(len(self.layers)):
                    nxt = self.bits[li + 1] if li + 1 < len(self.layers) else self.last_bits
                    _native.call("dl_dwn_fwd_bits_t", cur, self.plans[li].map_nodes, self.masks[li], nxt,
                                 self.N[li], self.n[li], self.Bp)
                    cur = nxt
                _native.call("dl_popcount_groupsum_t", cur, out[lo:hi], self.N[-1], self.k, B, self.Bp)
        return out

    def algorithmic_bytes_per_step(self, B: int) -> int:
        """HBM bytes one training step must move in this (bit-packed) mode: per sample
        encoder 4F + FT/8; hidden layer forward I/8 + N/8, last layer forward I/8 + 4k;
        backward per layer 4N (0 for the last: its gradient is the k logits' gradient) + I/8
        + 4I (0 for the first layer); per step tables read (forward, transform) and gradient
        written, index maps, and Adam's 7 passes over the tables."""
        per_sample = 4 * self.F + self.I[0] / 8
        last = len(self.layers) - 1
        for li in range(len(self.layers)):
            per_sample += self.I[li] / 8 + (4 * self.k if li == last else self.N[li] / 8)
            # backward: read the gradient of this layer's output (the k logit gradients for the last
            # layer; never materialised for the first layer in fused mode), re-read the input bits,
            # write the gradient of the input (not for the first layer)
            if li == last:
                per_sample += 4 * self.k
            elif li > 0 or not self.fused_backward:
                per_sample += 4 * self.N[li]
            per_sample += self.I[li] / 8
            if li > 1 or (li == 1 and not self.fused_backward):
                per_sample += 4 * self.I[li]
        table_bytes = 4 * self.flat.numel()
        per_step = 3 * table_bytes + 7 * table_bytes + sum(2 * 4 * N * n for N, n in zip(self.N, self.n))
        return int(per_sample * B + per_step)



class HostPipeline:
    """Double-buffered training steps fed from pinned host memory, one CUDA graph launch per step.

    `x_pinned` (B, F) fp32 and `labels_pinned` (B,) int32 are the caller's staging buffers.  The constructor
    copies their current content to device slot 0.  Every `step()` replays a graph that (a) trains on the slot
    filled last, (b) on a parallel branch copies the CURRENT content of the pinned buffers into the other slot,
    (c) copies the step's loss into `loss` (pinned, 1 element).  So the caller writes batch k + 1 into the pinned
    buffers, calls `step()` (which trains on batch k and fetches k + 1), and must not overwrite the pinned
    buffers again before that step has finished (synchronise, or read `loss` after an event).  The host's share
    of a step is a single launch, which matters when the device step is short (many GPUs, small per-rank
    batches).  With the peer optimiser `step()` polls the exchange status as `train_step` does.
    """

    def __init__(self, net: DWNNetwork, x_pinned, labels_pinned, loss_pinned=None, global_batch=None):
        if not (x_pinned.is_pinned() and labels_pinned.is_pinned()):
            raise ValueError("host_pipeline needs pinned host tensors")
        if x_pinned.dtype != torch.float32 or labels_pinned.dtype != torch.int32:
            raise ValueError("host_pipeline takes fp32 inputs and int32 labels")
        B = int(x_pinned.shape[0])
        if tuple(x_pinned.shape) != (B, net.F) or tuple(labels_pinned.shape) != (B,):
            raise ValueError("host_pipeline: inputs (B, F) and labels (B,) expected")
        if int(labels_pinned.min()) < 0 or int(labels_pinned.max()) >= net.k:
            raise ValueError(f"labels must lie in [0, {net.k})")
        self.net, self.x_pinned, self.labels_pinned = net, x_pinned, labels_pinned
        self.loss = loss_pinned if loss_pinned is not None else torch.zeros(1).pin_memory()
        self.B = B
        self.B_global = B * net.world if global_batch is None else int(global_batch)
        dev = net.device
        with torch.cuda.device(dev):
            net._ensure_buffers(B)
            if net._graph is None or net._graph_B_global != self.B_global:
                net._capture(B, self.B_global)  # the eager warm-up step (state restored afterwards) and the general graph
            self.slots = [(torch.empty(B, net.F, device=dev, dtype=torch.float32),
                           torch.empty(B, device=dev, dtype=torch.int32)) for _ in range(2)]
            self.copy_stream = torch.cuda.Stream(device=dev)
            self.slots[0][0].copy_(x_pinned, non_blocking=True)
            self.slots[0][1].copy_(labels_pinned, non_blocking=True)
            self.graphs = [self._capture(0), self._capture(1)]
        self.cur = 0

    def _capture(self, s: int):
        net = self.net
        net._x_src, net._y_src = self.slots[s]
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                main = torch.cuda.current_stream()
                self.copy_stream.wait_stream(main)
                with torch.cuda.stream(self.copy_stream):
                    self.slots[s ^ 1][0].copy_(self.x_pinned, non_blocking=True)
                    self.slots[s ^ 1][1].copy_(self.labels_pinned, non_blocking=True)
                net._step_body(self.B, self.B_global)
                self.loss.copy_(net.loss, non_blocking=True)
                main.wait_stream(self.copy_stream)
        finally:
            net._x_src = net._y_src = None
        return graph

    def step(self) -> torch.Tensor:
        net = self.net
        with torch.cuda.device(net.device):
            self.graphs[self.cur].replay()
        self.cur ^= 1
        net.step_count += 1
        if net.peer_optimizer and net.peer_status_every > 0 and net.step_count % net.peer_status_every == 0:
            status = net.peer_status()
            if status != 0:
                raise RuntimeError(f"peer exchange: rank {status - 1} did not arrive within {net.peer_timeout_ms} ms; "
                                   "the tables are invalid since the last successful poll")
        return self.loss
