"""Soft input selection of LearnableLayer: `x @ softmax(W / tau, dim=-1).T` on the tensor cores.

Reference: difflut/layers/learnable_layer.py:253-255 (F.softmax + torch.matmul, fp32).  Here the
row softmax, the forward contraction and the two backward contractions run in the CUDA library:
`dl_softmax_rows_bf16`, `dl_gemm_bf16_tn` (tcgen05 / TMA, bf16 operands, fp32 accumulation) and
`dl_softmax_bwd_rows`.

Precision.  A DWN node thresholds the selected value at 0.5 and with near-uniform selection weights
that value sits close to 0.5, so the FORWARD keeps 16 mantissa bits: every operand is split into a
bf16 head and a bf16 residual and the products head*head + head*residual (+ residual*head) are
summed by concatenating the pieces along K of one GEMM.  `FORWARD_SPLITS` picks the number of
pieces: 1 = plain bf16, 2 = split the softmax only (exact when x is exactly representable in bf16,
e.g. binary inputs), 3 = split both (default).  The backward GEMMs use plain bf16 (1e-2 bar).

`FORWARD_SPLITS = "centered"` is a single-pass alternative for the regime that matters for the threshold:
a softmax row sums to one, so `S = 1/I + D` and `x @ S.T = sum(x)/I + x @ D.T`; bf16 rounds D (error
relative to the deviation from a uniform selection, tiny while the selection is soft and the node inputs
sit near 0.5), and `sum(x)/I` enters the same GEMM exactly through three extra K columns
(`dl_softmax_rows_centered_bf16`, `dl_row_sum_split_bf16`).  Half the forward tensor-core work of 2; x
itself is rounded to bf16 (exact for binary inputs); once the selection is sharp its error is that of plain
bf16, where the selected values are far from the threshold.
"""

import torch

from .. import _native

FORWARD_SPLITS = 3
_CENTER_EXT = 64  # extra K columns of the centred form (three used): one K block, so the row pitch stays a multiple of 128 bytes


def _round_up(v: int, m: int) -> int:
    return (v + m - 1) // m * m


def _check_status(status: torch.Tensor, what: str) -> None:
    code = int(status.item())
    if code != 0:
        raise RuntimeError(f"dl_gemm_bf16_tn ({what}): a bounded wait inside the kernel ran out (status {code:#x})")


def _forward_operands(x, W, tau, splits):
    """bf16 operands of the forward contraction, pieces concatenated along K: A (B, ld) from x and Bm (M, ld) from
    softmax(W / tau).  splits 1..3: A = [x_hi | x_hi | x_lo], Bm = [S_hi | S_lo | S_hi]; 0 (centred):
    A = [x | split(sum(x)/I), 0...], Bm = [S - 1/I | 1, 1, 1, 0...]."""
    B, I = x.shape
    M = W.shape[0]
    Ip = _round_up(I, 8)
    dev, bf = x.device, torch.bfloat16
    # with no K padding every element of both operands is written below: no 3 GB memset for config 3
    alloc = torch.empty if Ip == I else torch.zeros
    if splits == 0:
        Ic = _round_up(I, _CENTER_EXT)  # the extension starts on a K-block boundary
        ld = Ic + _CENTER_EXT
        alloc = torch.empty if Ic == I else torch.zeros
        A = alloc(B, ld, device=dev, dtype=bf)
        Bm = alloc(M, ld, device=dev, dtype=bf)
        _native.call("dl_softmax_rows_centered_bf16", W, tau, Bm, ld, M, I, Ic, _CENTER_EXT)
        _native.call("dl_f32_to_bf16", x, A, None, B, I, ld, 0)
        _native.call("dl_row_sum_split_bf16", A, ld, B, I, Ic, 1.0 / I, _CENTER_EXT)
        return A, Bm, ld
    ld = splits * Ip
    A = alloc(B, ld, device=dev, dtype=bf)
    Bm = alloc(M, ld, device=dev, dtype=bf)
    s_lo = Bm.data_ptr() + 2 * Ip if splits >= 2 else None
    _native.call("dl_softmax_rows_bf16", W, tau, Bm, s_lo, ld, M, I)
    x_lo = A.data_ptr() + 2 * 2 * Ip if splits >= 3 else None
    _native.call("dl_f32_to_bf16", x, A, x_lo, B, I, ld, 0)
    if splits >= 2:
        A[:, Ip:Ip + I].copy_(A[:, :I])
    if splits >= 3:
        Bm[:, 2 * Ip:2 * Ip + I].copy_(Bm[:, :I])
    return A, Bm, ld


class SoftSelectFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, W, tau, splits, check):
        x = x.contiguous().float()
        W = W.contiguous().float()
        B, I = x.shape
        M = W.shape[0]
        Ip = _round_up(I, 8)
        dev = x.device
        bf = torch.bfloat16
        with torch.cuda.device(dev):
            # operands concatenated along K: A = [x_hi | x_hi | x_lo], Bm = [S_hi | S_lo | S_hi]
            A, Bm, ld = _forward_operands(x, W, tau, splits)
            out = torch.empty(B, M, device=dev, dtype=torch.float32)
            status = torch.zeros(1, device=dev, dtype=torch.int32)
            _native.call("dl_gemm_bf16_tn", A, Bm, out, B, M, ld, status)
            if check:
                _check_status(status, "forward")
        ctx.save_for_backward(x, W)
        ctx.tau, ctx.check = float(tau), check
        return out

    @staticmethod
    def backward(ctx, gy):
        x, W = ctx.saved_tensors
        B, I = x.shape
        M = W.shape[0]
        dev = x.device
        bf = torch.bfloat16
        gy = gy.contiguous().float()
        need_x, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        gx = gW = None
        with torch.cuda.device(dev):
            status = torch.zeros(1, device=dev, dtype=torch.int32)
            if need_x:
                # gx (B, I) = gy (B, M) @ S (M, I): operands gy [B, K=M] and S^T [I, K=M]
                Mp = _round_up(M, 8)
                S = torch.empty(M, I, device=dev, dtype=bf)
                _native.call("dl_softmax_rows_bf16", W, ctx.tau, S, None, I, M, I)
                St = torch.zeros(I, Mp, device=dev, dtype=bf)
                _native.call("dl_bf16_transpose", S, St, M, I, I, Mp)
                del S
                gyb = torch.zeros(B, Mp, device=dev, dtype=bf)
                _native.call("dl_f32_to_bf16", gy, gyb, None, B, M, Mp, 0)
                gx = torch.empty(B, I, device=dev, dtype=torch.float32)
                _native.call("dl_gemm_bf16_tn", gyb, St, gx, B, I, Mp, status)
                del St, gyb
            if need_w:
                # gS (M, I) = gy^T (M, B) @ x (B, I): operands gy^T [M, K=B] and x^T [I, K=B]
                Bp = _round_up(B, 8)
                gyt = torch.zeros(M, Bp, device=dev, dtype=bf)
                _native.call("dl_f32_to_bf16", gy, gyt, None, B, M, Bp, 1)
                xt = torch.zeros(I, Bp, device=dev, dtype=bf)
                _native.call("dl_f32_to_bf16", x, xt, None, B, I, Bp, 1)
                gS = torch.empty(M, I, device=dev, dtype=torch.float32)
                _native.call("dl_gemm_bf16_tn", gyt, xt, gS, M, I, Bp, status)
                del gyt, xt
                gW = torch.empty(M, I, device=dev, dtype=torch.float32)
                _native.call("dl_softmax_bwd_rows", W, gS, ctx.tau, gW, M, I)
            if ctx.check:
                _check_status(status, "backward")
        return gx, gW, None, None, None


class SoftSelectTFunction(torch.autograd.Function):
    """The same contraction with the operands swapped: (B, I), (M, I) -> (M, B) feature-major,
    `softmax(W / tau) @ x.T`, which is the layout the DWN layer kernels read and write.  The backward takes
    the gradient in that layout, so the gradient of the node inputs goes into the weight-gradient
    contraction as it leaves the node kernels: no transposes of (B, M) tensors in either direction.
    B must be a multiple of 128."""

    @staticmethod
    def forward(ctx, x, W, tau, splits, check, grad_channel=None):
        x = x.contiguous().float()
        W = W.contiguous().float()
        B, I = x.shape
        M = W.shape[0]
        if B % 128 != 0:
            raise ValueError("soft_select_t needs a batch that is a multiple of 128")
        # a consumer that can write its input gradient as bf16 (M, B) leaves it in the channel (FeatureMajorInput)
        ctx.grad_channel = grad_channel if (grad_channel is not None and grad_channel.disjoint) else None
        if ctx.grad_channel is not None:
            grad_channel.want_bf16 = True
        want_bits = grad_channel is not None and grad_channel.want_bits
        Ip = _round_up(I, 8)
        dev = x.device
        bf = torch.bfloat16
        with torch.cuda.device(dev):
            A, Bm, ld = _forward_operands(x, W, tau, splits)
            status = torch.zeros(1, device=dev, dtype=torch.int32)
            if want_bits:
                # the consumer reads only `value >= 0.5`: packed in the epilogue, nothing else is stored; what
                # autograd sees is a placeholder of the result's shape
                bits = torch.empty(M, B // 32, device=dev, dtype=torch.int32)
                _native.call("dl_gemm_bf16_tn_bits", Bm, A, bits, M, B, ld, B // 32, 0.5, status)
                grad_channel.bits_t = bits
                out_t = torch.zeros(1, 1, device=dev, dtype=torch.float32).expand(M, B)
            else:
                out_t = torch.empty(M, B, device=dev, dtype=torch.float32)
                _native.call("dl_gemm_bf16_tn", Bm, A, out_t, M, B, ld, status)
            if check:
                _check_status(status, "forward")
        ctx.save_for_backward(x, W)
        ctx.tau, ctx.check = float(tau), check
        return out_t

    @staticmethod
    def backward(ctx, gy_t):
        x, W = ctx.saved_tensors
        B, I = x.shape
        M = W.shape[0]
        dev = x.device
        bf = torch.bfloat16
        channel = ctx.grad_channel
        gyb = None
        from_channel = channel is not None and channel.grad_bf16 is not None
        if from_channel:
            gyb, channel.grad_bf16 = channel.grad_bf16, None  # (M, B) bf16 from the consumer; gy_t is a placeholder
        else:
            gy_t = gy_t.contiguous().float()  # (M, B)
        need_x, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        gx = gW = None
        with torch.cuda.device(dev):
            status = torch.zeros(1, device=dev, dtype=torch.int32)
            if need_w:
                # gS (M, I) = gy_t (M, K=B) @ x (B, I): operands gy_t [M, K=B] as it is and x^T [I, K=B]
                if gyb is None:
                    gyb = torch.empty(M, B, device=dev, dtype=bf)
                    _native.call("dl_f32_to_bf16", gy_t, gyb, None, M, B, B, 0)
                xt = torch.zeros(I, B, device=dev, dtype=bf)
                _native.call("dl_f32_to_bf16", x, xt, None, B, I, B, 1)
                gS = torch.empty(M, I, device=dev, dtype=torch.float32)
                _native.call("dl_gemm_bf16_tn", gyb, xt, gS, M, I, B, status)
                del xt
                gW = torch.empty(M, I, device=dev, dtype=torch.float32)
                _native.call("dl_softmax_bwd_rows", W, gS, ctx.tau, gW, M, I)
            if need_x:
                # gx (B, I) = gy (B, M) @ S (M, I): operands gy [B, K=M] (a transpose of gy_t) and S^T [I, K=M]
                Mp = _round_up(M, 8)
                S = torch.empty(M, I, device=dev, dtype=bf)
                _native.call("dl_softmax_rows_bf16", W, ctx.tau, S, None, I, M, I)
                St = torch.zeros(I, Mp, device=dev, dtype=bf)
                _native.call("dl_bf16_transpose", S, St, M, I, I, Mp)
                del S
                gyr = torch.zeros(B, Mp, device=dev, dtype=bf)
                if from_channel:
                    _native.call("dl_bf16_transpose", gyb, gyr, M, B, B, Mp)
                else:
                    _native.call("dl_f32_to_bf16", gy_t, gyr, None, M, B, Mp, 1)
                gx = torch.empty(B, I, device=dev, dtype=torch.float32)
                _native.call("dl_gemm_bf16_tn", gyr, St, gx, B, I, Mp, status)
            if ctx.check:
                _check_status(status, "backward")
        return gx, gW, None, None, None, None


def _splits_code(splits) -> int:
    if splits is None:
        splits = FORWARD_SPLITS
    if splits == "centered":
        return 0
    if splits not in (1, 2, 3):
        raise ValueError('splits must be 1, 2, 3 or "centered"')
    return int(splits)


def soft_select_t(x: torch.Tensor, W: torch.Tensor, tau: float, splits: int = None, check: bool = True,
                  grad_channel=None) -> torch.Tensor:
    """(B, I), (M, I) -> (M, B) feature-major with autograd (B a multiple of 128); see soft_select.
    `grad_channel`: a `fused_ops.FeatureMajorInput` shared with the one consumer of the result, through which
    that consumer may hand its input gradient over as bf16."""
    if not (x.is_cuda and W.is_cuda):
        raise RuntimeError("difflut_b200 layers run on CUDA tensors only (no CPU fallback)")
    splits = _splits_code(splits)
    return SoftSelectTFunction.apply(x, W, float(tau), int(splits), bool(check), grad_channel)


def soft_select(x: torch.Tensor, W: torch.Tensor, tau: float, splits: int = None, check: bool = True) -> torch.Tensor:
    """(B, I), (M, I) -> (B, M) with autograd.  `check` reads the kernels' status word back (one
    host synchronisation per call); pass False inside a captured or latency-critical region."""
    if not (x.is_cuda and W.is_cuda):
        raise RuntimeError("difflut_b200 layers run on CUDA tensors only (no CPU fallback)")
    splits = _splits_code(splits)
    return SoftSelectFunction.apply(x, W, float(tau), int(splits), bool(check))
