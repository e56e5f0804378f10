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
"""

import torch

from .. import _native

FORWARD_SPLITS = 3


def _round_up(v: int, m: int) -> int:
    return (v + m - 1) // m * m


def _check_status(status: torch.Tensor, what: str) -> None:
    code = int(status.item())
    if code != 0:
        raise RuntimeError(f"dl_gemm_bf16_tn ({what}): a bounded wait inside the kernel ran out (status {code:#x})")


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
            # with no K padding every element of both operands is written below: no 3 GB memset for config 3
            alloc = torch.empty if Ip == I else torch.zeros
            A = alloc(B, splits * Ip, device=dev, dtype=bf)
            Bm = alloc(M, splits * Ip, device=dev, dtype=bf)
            ld = splits * Ip
            s_lo = Bm.data_ptr() + 2 * Ip if splits >= 2 else None
            _native.call("dl_softmax_rows_bf16", W, tau, Bm, s_lo, ld, M, I)
            x_lo = A.data_ptr() + 2 * 2 * Ip if splits >= 3 else None
            _native.call("dl_f32_to_bf16", x, A, x_lo, B, I, ld, 0)
            if splits >= 2:
                A[:, Ip:Ip + I].copy_(A[:, :I])
            if splits >= 3:
                Bm[:, 2 * Ip:2 * Ip + I].copy_(Bm[:, :I])
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
    def forward(ctx, x, W, tau, splits, check):
        x = x.contiguous().float()
        W = W.contiguous().float()
        B, I = x.shape
        M = W.shape[0]
        if B % 128 != 0:
            raise ValueError("soft_select_t needs a batch that is a multiple of 128")
        Ip = _round_up(I, 8)
        dev = x.device
        bf = torch.bfloat16
        with torch.cuda.device(dev):
            # with no K padding every element of both operands is written below: no 3 GB memset for config 3
            alloc = torch.empty if Ip == I else torch.zeros
            A = alloc(B, splits * Ip, device=dev, dtype=bf)
            Bm = alloc(M, splits * Ip, device=dev, dtype=bf)
            ld = splits * Ip
            s_lo = Bm.data_ptr() + 2 * Ip if splits >= 2 else None
            _native.call("dl_softmax_rows_bf16", W, tau, Bm, s_lo, ld, M, I)
            x_lo = A.data_ptr() + 2 * 2 * Ip if splits >= 3 else None
            _native.call("dl_f32_to_bf16", x, A, x_lo, B, I, ld, 0)
            if splits >= 2:
                A[:, Ip:Ip + I].copy_(A[:, :I])
            if splits >= 3:
                Bm[:, 2 * Ip:2 * Ip + I].copy_(Bm[:, :I])
            out_t = torch.empty(M, B, device=dev, dtype=torch.float32)
            status = torch.zeros(1, device=dev, dtype=torch.int32)
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
        gy_t = gy_t.contiguous().float()  # (M, B)
        need_x, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        gx = gW = None
        with torch.cuda.device(dev):
            status = torch.zeros(1, device=dev, dtype=torch.int32)
            if need_w:
                # gS (M, I) = gy_t (M, K=B) @ x (B, I): operands gy_t [M, K=B] as it is and x^T [I, K=B]
                gyb = torch.empty(M, B, device=dev, dtype=bf)
                _native.call("dl_f32_to_bf16", gy_t, gyb, None, M, B, B, 0)
                xt = torch.zeros(I, B, device=dev, dtype=bf)
                _native.call("dl_f32_to_bf16", x, xt, None, B, I, B, 1)
                gS = torch.empty(M, I, device=dev, dtype=torch.float32)
                _native.call("dl_gemm_bf16_tn", gyb, xt, gS, M, I, B, status)
                del gyb, xt
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
                _native.call("dl_f32_to_bf16", gy_t, gyr, None, M, B, Mp, 1)
                gx = torch.empty(B, I, device=dev, dtype=torch.float32)
                _native.call("dl_gemm_bf16_tn", gyr, St, gx, B, I, Mp, status)
            if ctx.check:
                _check_status(status, "backward")
        return gx, gW, None, None, None


def soft_select_t(x: torch.Tensor, W: torch.Tensor, tau: float, splits: int = None, check: bool = True) -> torch.Tensor:
    """(B, I), (M, I) -> (M, B) feature-major with autograd (B a multiple of 128); see soft_select."""
    if not (x.is_cuda and W.is_cuda):
        raise RuntimeError("difflut_b200 layers run on CUDA tensors only (no CPU fallback)")
    if splits is None:
        splits = FORWARD_SPLITS
    if splits not in (1, 2, 3):
        raise ValueError("splits must be 1, 2 or 3")
    return SoftSelectTFunction.apply(x, W, float(tau), int(splits), bool(check))


def soft_select(x: torch.Tensor, W: torch.Tensor, tau: float, splits: int = None, check: bool = True) -> torch.Tensor:
    """(B, I), (M, I) -> (B, M) with autograd.  `check` reads the kernels' status word back (one
    host synchronisation per call); pass False inside a captured or latency-critical region."""
    if not (x.is_cuda and W.is_cuda):
        raise RuntimeError("difflut_b200 layers run on CUDA tensors only (no CPU fallback)")
    if splits is None:
        splits = FORWARD_SPLITS
    if splits not in (1, 2, 3):
        raise ValueError("splits must be 1, 2 or 3")
    return SoftSelectFunction.apply(x, W, float(tau), int(splits), bool(check))
