"""ctypes binding of ``libtcq_b200.so`` (the C ABI declared in ``include/tcq_b200.h``).

The library is built in-tree by ``csrc/Makefile`` (see ``build()``).  There is no
fallback: if the shared object is missing or cannot be loaded, importing the
codec fails with an error that says how to build it.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

_CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
LIB_PATH = os.path.join(_CSRC, "libtcq_b200.so")

ABI_VERSION = 4

# name -> (restype, argtypes); mirrors include/tcq_b200.h one to one
_vp, _i64, _int, _sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_size_t
SIGNATURES = {
    "tcq_abi_version": (_int, []),
    "tcq_strerror": (ctypes.c_char_p, [_int]),
    "tcq_last_cuda_error": (ctypes.c_char_p, []),
    "tcq_workspace_bytes": (_sz, [_i64, _int]),
    "tcq_workspace_min_bytes": (_sz, [_int]),
    "tcq_encode_tb": (_int, [_vp, _i64, _int, _int, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "tcq_encode_tb_static_max_tiles": (_i64, [_int]),
    "tcq_encode_tb_static": (_int, [_vp, _i64, _int, _int, _vp, _vp, _vp, _vp, _vp]),
    "tcq_encode_tb_static_status": (_int, [_vp]),
    "tcq_encode_tb_rows": (_int, [_vp, _vp, _i64, _i64, _int, _int, _vp, _i64, _vp, _vp, _vp, _vp, _sz, _vp]),
    "tcq_viterbi_pass": (_int, [_vp, _i64, _int, _int, _vp, _int, _vp, _vp, _sz, _vp]),
    "tcq_forward_pass": (_int, [_vp, _i64, _int, _int, _vp, _int, _int, _vp, _sz, _vp]),
    "tcq_workspace_status": (_int, [_vp, _sz, _i64, _int, _vp]),
    "tcq_selftest_wait_timeout": (_int, [_vp, _i64, _int, _vp, _sz, _vp]),
    "tcq_encode_launches": (_i64, [_i64, _int, _sz]),
    "tcq_decode_packed": (_int, [_vp, _i64, _int, _int, _vp, _vp]),
    "tcq_decode_matvec": (_int, [_vp, _i64, _i64, _int, _int, _vp, _i64, _int, _vp, _i64, _vp]),
    "tcq_decode_symbols": (_int, [_vp, _i64, _i64, _int, _int, _vp, _vp, _vp]),
    "tcq_pack_symbols": (_int, [_vp, _i64, _int, _vp, _vp]),
    "tcq_codebook_lut": (_int, [_int, _vp, _vp]),
    "tcq_ip_workspace_bytes": (_sz, [_i64, _i64]),
    "tcq_ip_forward": (_int, [_vp, _i64, _i64, _vp, _vp, ctypes.c_float, _int, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "tcq_ip_restore": (_int, [_vp, _int, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
}

_lib = None


class TcqError(RuntimeError):
    """A C-ABI call returned a negative status."""


def build(verbose: bool = False, jobs: int = 8) -> str:
    """Compile the CUDA sources for sm_100a with nvcc (``make`` in ``csrc/``)."""
    cmd = ["make", "-C", _CSRC, f"-j{jobs}", "libtcq_b200.so"]
    subprocess.check_call(cmd, stdout=None if verbose else subprocess.DEVNULL)
    return LIB_PATH


def lib() -> ctypes.CDLL:
    """The loaded library, with argument types set.  Raises if it was not built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} not found: the CUDA extension is not built. "
                "Run `python -c 'import __graft_entry__ as g; g.build()'` or `make -C <package>/csrc`. "
                "There is no CPU fallback.")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)       # AttributeError here = a declared symbol is not exported
            fn.restype = res
            fn.argtypes = args
        got = handle.tcq_abi_version()
        if got != ABI_VERSION:
            raise ImportError(f"libtcq_b200.so has ABI version {got}, this package needs {ABI_VERSION}: rebuild it")
        _lib = handle
    return _lib


def check(code: int, what: str) -> None:
    """Turn a negative status into an exception (ValueError for bad arguments)."""
    if code == 0:
        return
    L = lib()
    msg = L.tcq_strerror(code).decode()
    if code == -7:
        raise TcqError(f"{what}: {msg}: {L.tcq_last_cuda_error().decode()}")
    if code in (-6, -10, -11):
        raise TcqError(f"{what}: {msg}")
    raise ValueError(f"{what}: {msg}")
