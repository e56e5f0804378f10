"""Norm-wise comparison used by the gradient parity tests.

The floating-point bar of this project is 1e-5 relative.  For a gradient tensor that is a long sum
over the batch, individual entries can cancel to almost nothing, so an element-wise relative bound is
meaningless there; the bound that says "this tensor agrees to 1e-5" is norm-wise:

    max |got - ref|  <=  tol * max |ref|          (tol = 1e-5 unless a test states otherwise)

Every call records the error it measured.  The records are printed in pytest's terminal summary and,
when the environment variable DIFFLUT_PARITY_LOG names a file, appended to it as tab-separated text
(test id, tensor, measured error / max|ref|, bound).
"""

import os

import torch

RECORDS = []
_current = {"test": ""}


def set_current_test(nodeid: str) -> None:
    _current["test"] = nodeid


def normwise_error(got: torch.Tensor, ref: torch.Tensor) -> float:
    got = got.detach().double().cpu()
    ref = ref.detach().double().cpu()
    if got.shape != ref.shape:
        raise AssertionError(f"shape mismatch: {tuple(got.shape)} vs {tuple(ref.shape)}")
    if got.numel() == 0:
        return 0.0
    if not bool(torch.isfinite(got).all()):
        return float("inf")
    scale = float(ref.abs().max())
    err = float((got - ref).abs().max())
    if scale == 0.0:
        return 0.0 if err == 0.0 else float("inf")
    return err / scale


def close_normwise(got: torch.Tensor, ref: torch.Tensor, what: str, tol: float = 1e-5) -> float:
    """Assert max|got-ref| <= tol * max|ref| and record the measured ratio."""
    rel = normwise_error(got, ref)
    RECORDS.append((_current["test"], what, rel, tol))
    path = os.environ.get("DIFFLUT_PARITY_LOG")
    if path:
        with open(path, "a") as f:
            f.write(f"{_current['test']}\t{what}\t{rel:.3e}\t{tol:.0e}\n")
    assert rel <= tol, f"{what}: max|got-ref| / max|ref| = {rel:.3e} exceeds {tol:.0e}"
    return rel
