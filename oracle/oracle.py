"""ctypes front end of the plain-C oracle (``tcq_oracle.c``).

TEST INFRASTRUCTURE ONLY: the shipped package never imports this module.  Each
wrapper mirrors one function of the reference (cited in ``tcq_oracle.c``) on numpy
arrays, so that tests can compare the CUDA path, the oracle and the committed
golden vectors with plain ``numpy.array_equal``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libtcq_oracle.so")
_lib = None

CODEBOOK_IDS = {"1mad": 0, "3inst": 1, "mcg": 2}
T_SEQ = 256
L = 16


def build(force: bool = False) -> str:
    """Compile ``tcq_oracle.c`` with gcc (``make`` in this folder); returns the .so path."""
    src = os.path.join(_HERE, "tcq_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libtcq_oracle.so"], stdout=subprocess.DEVNULL)
    return _SO


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        L_ = ctypes.CDLL(_SO)
        c_i64, c_int, c_vp = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p
        L_.tcq_oracle_codebook_value.restype = ctypes.c_float
        L_.tcq_oracle_codebook_value.argtypes = [c_int, ctypes.c_uint32]
        L_.tcq_oracle_codebook_lut.argtypes = [c_int, c_vp]
        L_.tcq_oracle_decode_recursive.argtypes = [c_vp, c_i64, c_i64, c_int, c_vp, c_vp, c_vp]
        L_.tcq_oracle_decode_window.argtypes = [c_vp, c_i64, c_i64, c_int, c_vp, c_vp, c_vp]
        L_.tcq_oracle_decode_wrapped.argtypes = [c_vp, c_i64, c_int, c_vp, c_vp]
        L_.tcq_oracle_pack_bits.argtypes = [c_vp, c_i64, c_int, c_vp]
        L_.tcq_oracle_decode_packed.argtypes = [c_vp, c_i64, c_int, c_int, c_vp]
        L_.tcq_oracle_viterbi_pass.argtypes = [c_vp, c_i64, c_int, c_vp, c_vp, c_vp, c_int]
        L_.tcq_oracle_viterbi_pass.restype = c_int
        L_.tcq_oracle_viterbi_tb.argtypes = [c_vp, c_i64, c_int, c_vp, c_vp, c_vp, c_vp, c_int]
        L_.tcq_oracle_viterbi_tb.restype = c_int
        L_.tcq_oracle_max_threads.restype = c_int
        _lib = L_
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _i64(a):
    return np.ascontiguousarray(a, dtype=np.int64)


def max_threads() -> int:
    return int(lib().tcq_oracle_max_threads())


def codebook_lut(name: str) -> np.ndarray:
    """``codebook_lut(name)`` of the reference: fp32 value of every 16-bit state."""
    out = np.empty(1 << L, dtype=np.float32)
    lib().tcq_oracle_codebook_lut(CODEBOOK_IDS[name], _p(out))
    return out


def decode_recursive(bits, K, lut, s0=None) -> np.ndarray:
    bits = _i64(bits)
    n, T = bits.shape
    lut = _f32(lut)
    s0 = _i64(s0) if s0 is not None else None
    out = np.empty((n, T), dtype=np.float32)
    lib().tcq_oracle_decode_recursive(_p(bits), n, T, K, _p(lut), _p(s0), _p(out))
    return out


def decode_window(bits, K, lut, s0=None) -> np.ndarray:
    bits = _i64(bits)
    n, T = bits.shape
    lut = _f32(lut)
    s0 = _i64(s0) if s0 is not None else None
    out = np.empty((n, T), dtype=np.float32)
    lib().tcq_oracle_decode_window(_p(bits), n, T, K, _p(lut), _p(s0), _p(out))
    return out


def decode_wrapped(bits, K, lut) -> np.ndarray:
    """Decode a tail-biting tile from its symbols alone (window primed from the tail)."""
    bits = _i64(bits)
    n, T = bits.shape
    assert T == T_SEQ
    lut = _f32(lut)
    out = np.empty((n, T), dtype=np.float32)
    lib().tcq_oracle_decode_wrapped(_p(bits), n, K, _p(lut), _p(out))
    return out


def pack_bits(bits, K) -> np.ndarray:
    """``pack_bits_np`` of the reference's exporter: u32 [n, 8K], reversed bit order."""
    bits = _i64(bits)
    n, T = bits.shape
    assert T == T_SEQ
    out = np.empty((n, T * K // 32), dtype=np.uint32)
    lib().tcq_oracle_pack_bits(_p(bits), n, K, _p(out))
    return out


def decode_packed(packed, K, name) -> np.ndarray:
    """CPU form of the reference's WGSL window decode of the packed words."""
    packed = np.ascontiguousarray(packed, dtype=np.uint32)
    n = packed.shape[0]
    assert packed.shape[1] == T_SEQ * K // 32
    out = np.empty((n, T_SEQ), dtype=np.float32)
    lib().tcq_oracle_decode_packed(_p(packed), n, K, CODEBOOK_IDS[name], _p(out))
    return out


def viterbi_pass(w, K, lut, overlap=None, nthreads: int = 0) -> np.ndarray:
    """``_viterbi_pass(w, K, lut, overlap)``: optimal state path int64 [n, 256]."""
    w = _f32(w)
    n, T = w.shape
    assert T == T_SEQ
    lut = _f32(lut)
    ov = np.ascontiguousarray(overlap, dtype=np.int32) if overlap is not None else None
    states = np.empty((n, T), dtype=np.int64)
    rc = lib().tcq_oracle_viterbi_pass(_p(w), n, K, _p(lut), _p(ov), _p(states), nthreads)
    if rc != 0:
        raise MemoryError("oracle scratch allocation failed")
    return states


def viterbi_tb(w, K, lut, nthreads: int = 0, with_sse: bool = False):
    """``viterbi_tb(w, K, lut)`` with the fp32 DP: (bits int64 [n,256], dq f32 [n,256])."""
    w = _f32(w)
    n, T = w.shape
    assert T == T_SEQ
    lut = _f32(lut)
    bits = np.empty((n, T), dtype=np.int64)
    dq = np.empty((n, T), dtype=np.float32)
    sse = np.empty(n, dtype=np.float32) if with_sse else None
    rc = lib().tcq_oracle_viterbi_tb(_p(w), n, K, _p(lut), _p(bits), _p(dq), _p(sse), nthreads)
    if rc != 0:
        raise MemoryError("oracle scratch allocation failed")
    return (bits, dq, sse) if with_sse else (bits, dq)
