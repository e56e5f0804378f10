"""ctypes binding of the C ABI declared in `include/difflut_b200.h`.

There is no CPU fallback: if the shared library is missing, `lib()` raises.  Every wrapper
passes raw device pointers plus the current CUDA stream and turns a negative return code
into RuntimeError (the reference's bindings raise RuntimeError through TORCH_CHECK,
difflut/nodes/cuda/efd_cuda.cpp:18-40).
"""

import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_lib", "libdifflut_b200.so")

# signature strings: p = pointer, l = int64, i = int, f = float, d = double; the trailing
# stream argument is implicit for every entry marked with a final 's'.
SIGNATURES = {
    "dl_thermo_rows": "ppplll s",
    "dl_thermo_pack_t": "pppllll s",
    "dl_thermo_pack_s": "pppllll s",
    "dl_thermo_pack_rows": "ppplll s",
    "dl_pack_rows_to_t": "pplllf s",
    "dl_pack_t_to_t": "ppllllf s",
    "dl_f32_rows_to_t": "pplll s",
    "dl_f32_t_to_rows": "pplll s",
    "dl_bits_t_to_rows": "pplll s",
    "dl_bits_rows_to_t": "ppllll s",
    "dl_gather_rows": "pppllll s",
    "dl_gather_rows_bwd": "ppppllll s",
    "dl_gather_rows_bwd_ell": "pplpllll s",
    "dl_unfold_rows": "ppllllllllll s",
    "dl_unfold_pack_t": "ppllllllllllfl s",
    "dl_fold_rows": "ppllllllllll s",
    "dl_fold_t": "pplllllllllll s",
    "dl_dwn_prepare": "pppllff s",
    "dl_dwn_prepare_weighted": "pppllfp s",
    "dl_dwn_prepare_full": "ppllff s",
    "dl_dwn_fwd_bits_t": "pppplll s",
    "dl_dwn_fwd_vals_t": "ppppplll s",
    "dl_dwn_bwd_tables_t": "ppplfpplll s",
    "dl_dwn_bwd_input_t": "pplfpppplll s",
    "dl_dwn_bwd_input_disjoint_t": "pplfpppllll s",
    "dl_dwn_bwd_fused_t": "pplfpllpppppppllll s",
    "dl_sum_groups": "pplll s",
    "dl_dwn_mapped_fwd": "ppplllli s",
    "dl_dwn_mapped_bwd": "pppppllll s",
    "dl_dwn_stable_mapped_bwd_input": "ppppfpllll s",
    "dl_hybrid_mapped_bwd": "pppppllll s",
    "dl_prob_fwd_t": "pppfpllll s",
    "dl_prob_fwd_groupsum_t": "pppfpppllllfl s",
    "dl_prob_bwd_t": "pppfplfpplllll s",
    "dl_hybrid_bwd_t": "pppplfpplllll s",
    "dl_seg_sum_t": "ppppll s",
    "dl_gemm_bf16_tn": "ppplllp s",
    "dl_gemm_bf16_tn_bits": "pppllllfp s",
    "dl_softmax_rows_bf16": "pfpplll s",
    "dl_softmax_rows_centered_bf16": "pfplllll s",
    "dl_row_sum_split_bf16": "pllllfl s",
    "dl_softmax_bwd_rows": "ppfpll s",
    "dl_f32_to_bf16": "pppllli s",
    "dl_bf16_transpose": "ppllll s",
    "dl_groupsum_rows": "pplllf s",
    "dl_groupsum_rows_bwd": "pplllf s",
    "dl_groupsum_t": "ppllfl s",
    "dl_dwn_fwd_groupsum_t": "ppppplllfl s",
    "dl_dwn_fwd_groupsum_s": "ppppplllfl s",
    "dl_dwn_fwd_groupsum_ce_s": "pppppppplllflll s",
    "dl_dwn_bwd_fused_s": "pplfpllpppppppllll s",
    "dl_bits_swizzle_t": "ppll s",
    "dl_dwn_fwd_groupsum_noalloc_t": "pppplllfl s",
    "dl_flip_rows": "pplfl s",
    "dl_bits_flip_t": "plllfl s",
    "dl_flip_at": "pppll s",
    "dl_bits_flip_at_t": "ppllll s",
    "dl_grad_rescale": "ppllififp s",
    "dl_p2p_barrier": "pllpl s",
    "dl_p2p_reduce_adam": "pppppplllfffff s",
    "dl_p2p_exchange_adam": "pppppppllllllllfffffl s",
    "dl_p2p_wait_done": "ppllll s",
    "dl_popcount_groupsum_t": "ppllll s",
    "dl_ce_t": "pppppllll s",
    "dl_loss_sum": "ppll s",
    "dl_adam_step": "ppppplfffff s",
    "dl_adam_advance": "pff s",
    "dl_adam_apply": "ppppplfffff s",
    "dl_adam_step_groups": "ppllpppplfffff s",
}

_CT = {"p": ctypes.c_void_p, "l": ctypes.c_int64, "i": ctypes.c_int, "f": ctypes.c_float, "d": ctypes.c_double}

_lib = None


def lib():
    """Load the shared library once; raise (never fall back) when it is absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"difflut_b200: CUDA library not found at {LIB_PATH}. Build it with "
            "`python -m difflut_b200.build` (needs nvcc, targets sm_100a). There is no CPU fallback."
        )
    handle = ctypes.CDLL(LIB_PATH)
    for name, sig in SIGNATURES.items():
        fn = getattr(handle, name)
        sig = sig.replace(" ", "")
        args = [_CT[c] for c in sig if c != "s"]
        if sig.endswith("s"):
            args.append(ctypes.c_void_p)
        fn.argtypes = args
        fn.restype = ctypes.c_int
    handle.dl_version.restype = ctypes.c_int
    handle.dl_error_string.restype = ctypes.c_char_p
    handle.dl_error_string.argtypes = [ctypes.c_int]
    handle.dl_padded_batch.restype = ctypes.c_int64
    handle.dl_padded_batch.argtypes = [ctypes.c_int64]
    handle.dl_dwn_groupsum_splits.restype = ctypes.c_int64
    handle.dl_dwn_groupsum_splits.argtypes = [ctypes.c_int64, ctypes.c_int64]
    handle.dl_dwn_bwd_groups.restype = ctypes.c_int64
    handle.dl_dwn_bwd_groups.argtypes = [ctypes.c_int64]
    handle.dl_prob_groupsum_splits.restype = ctypes.c_int64
    handle.dl_prob_groupsum_splits.argtypes = [ctypes.c_int64, ctypes.c_int64]
    handle.dl_grad_rescale_scratch_doubles.restype = ctypes.c_int64
    handle.dl_grad_rescale_scratch_doubles.argtypes = []
    handle.dl_p2p_enable_peer.restype = ctypes.c_int
    handle.dl_p2p_enable_peer.argtypes = [ctypes.c_int64]
    handle.dl_swizzled_words.restype = ctypes.c_int64
    handle.dl_swizzled_words.argtypes = [ctypes.c_int64]
    handle.dl_unfold_positions.restype = ctypes.c_int64
    handle.dl_unfold_positions.argtypes = [ctypes.c_int64] * 4
    _lib = handle
    return _lib


def available() -> bool:
    return os.path.exists(LIB_PATH)


def padded_batch(B: int) -> int:
    return (int(B) + 127) // 128 * 128


def _ptr(a):
    if a is None:
        return None
    if isinstance(a, torch.Tensor):
        if not a.is_cuda:
            raise RuntimeError("difflut_b200 kernels take CUDA tensors only (no CPU fallback)")
        if not a.is_contiguous():
            raise RuntimeError("difflut_b200 kernels take contiguous tensors")
        return a.data_ptr()
    return int(a)


def host_floats(values):
    """ctypes float array for entry points that take a small HOST array; pass `ctypes.addressof(arr)`
    (keep `arr` alive until the call returns)."""
    return (ctypes.c_float * len(values))(*[float(v) for v in values])


_CALL_PLANS = {}


def _call_plan(name: str):
    """(function, argument kinds, takes a stream) of entry `name`, resolved once."""
    plan = _CALL_PLANS.get(name)
    if plan is None:
        sig = SIGNATURES[name].replace(" ", "")
        plan = (getattr(lib(), name), tuple(c for c in sig if c != "s"), sig.endswith("s"))
        _CALL_PLANS[name] = plan
    return plan


def call(name: str, *args, stream=None):
    """Invoke C-ABI entry `name`; tensors become device pointers, the stream is appended."""
    fn, kinds, has_stream = _call_plan(name)
    if len(kinds) != len(args):
        raise TypeError(f"{name}: expected {len(kinds)} arguments, got {len(args)}")
    conv = [_ptr(a) if kind == "p" else (int(a) if kind in ("l", "i") else float(a)) for kind, a in zip(kinds, args)]
    if has_stream:
        conv.append(torch.cuda.current_stream().cuda_stream if stream is None else stream)
    code = fn(*conv)
    if code != 0:
        raise RuntimeError(f"{name} failed: {lib().dl_error_string(code).decode()} (code {code})")
