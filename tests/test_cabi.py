"""The C-ABI library loads, exports every symbol the header declares, and the ctypes signature
table agrees with the header's prototypes.  No compute calls (runs without a GPU)."""

import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "difflut_b200.h")


def _prototypes():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    protos = {}
    for m in re.finditer(r"\b(int|int64_t|const char\*)\s+(dl_\w+)\s*\(([^)]*)\)\s*;", text):
        args = [a.strip() for a in m.group(3).split(",") if a.strip() and a.strip() != "void"]
        protos[m.group(2)] = args
    return protos


@pytest.fixture(scope="module")
def library():
    from difflut_b200 import build

    return ctypes.CDLL(build.build())


def test_header_declares_functions():
    protos = _prototypes()
    assert len(protos) >= 30
    for required in ("dl_thermo_pack_t", "dl_dwn_fwd_bits_t", "dl_dwn_bwd_fused_t", "dl_prob_fwd_groupsum_t",
                     "dl_adam_step", "dl_popcount_groupsum_t"):
        assert required in protos


def test_every_declared_symbol_is_exported(library):
    for name in _prototypes():
        assert hasattr(library, name), f"{name} declared in the header but not exported"


def test_ctypes_signatures_match_header():
    from difflut_b200 import _native

    protos = _prototypes()
    kinds = {"p": "*", "l": "int64_t", "i": "int", "f": "float", "d": "double"}
    for name, sig in _native.SIGNATURES.items():
        assert name in protos, f"{name} bound in Python but not declared in the header"
        sig = sig.replace(" ", "")
        args = protos[name]
        want = list(sig[:-1]) + ["stream"] if sig.endswith("s") else list(sig)
        assert len(want) == len(args), f"{name}: {len(want)} bound arguments, header has {len(args)}"
        for code, decl in zip(want, args):
            if code == "stream":
                assert decl.startswith("dl_stream_t")
            elif code == "p":
                assert "*" in decl, f"{name}: '{decl}' bound as pointer"
            else:
                assert "*" not in decl and decl.split()[0] == kinds[code], f"{name}: '{decl}' bound as {kinds[code]}"
    # every compute entry point of the header is bound
    unbound = [n for n in protos if n not in _native.SIGNATURES and n not in (
        "dl_version", "dl_error_string", "dl_padded_batch", "dl_dwn_groupsum_splits", "dl_prob_groupsum_splits",
        "dl_dwn_bwd_groups", "dl_unfold_positions", "dl_swizzled_words", "dl_p2p_enable_peer",
        "dl_grad_rescale_scratch_doubles")]
    assert not unbound, unbound


def test_host_only_helpers(library):
    library.dl_padded_batch.restype = ctypes.c_int64
    library.dl_padded_batch.argtypes = [ctypes.c_int64]
    assert library.dl_padded_batch(1) == 128 and library.dl_padded_batch(128) == 128
    assert library.dl_padded_batch(129) == 256 and library.dl_padded_batch(0) == 0
    library.dl_error_string.restype = ctypes.c_char_p
    assert b"argument" in library.dl_error_string(-1)
    assert library.dl_version() >= 100
    library.dl_dwn_bwd_groups.restype = ctypes.c_int64
    library.dl_dwn_bwd_groups.argtypes = [ctypes.c_int64]
    assert library.dl_dwn_bwd_groups(8192) == 8 and library.dl_dwn_bwd_groups(128) == 1
    library.dl_unfold_positions.restype = ctypes.c_int64
    library.dl_unfold_positions.argtypes = [ctypes.c_int64] * 4
    assert library.dl_unfold_positions(28, 5, 1, 0) == 24 and library.dl_unfold_positions(28, 3, 2, 1) == 14
    assert library.dl_unfold_positions(2, 5, 1, 0) == 0


def test_missing_library_fails_loudly(monkeypatch):
    from difflut_b200 import _native

    monkeypatch.setattr(_native, "_lib", None)
    monkeypatch.setattr(_native, "LIB_PATH", "/nonexistent/libdifflut_b200.so")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _native.lib()
