"""Shared test configuration.

Markers:
  gpu   needs a CUDA device; run with ``-m gpu`` on a B200.  Everything else runs on CPU
        (``-m "not gpu"``).
The oracle under ``oracle/`` is test infrastructure: tests are the only place (besides the
smoke check and the benchmark's CPU legs) that may import it.
"""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG_DIR = os.path.join(ROOT, "trellis-everywhere_b200")
for p in (ROOT, PKG_DIR):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = os.path.join(ROOT, "tests", "golden")
CODEBOOKS = ("1mad", "3inst", "mcg")
KS = (2, 3, 4)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); selected with -m gpu")


@pytest.fixture(scope="session")
def golden():
    """name -> numpy archive of the committed outputs of the reference (see tests/golden/make_golden.py)."""
    return {n: np.load(os.path.join(GOLDEN, n + ".npz")) for n in ("codebooks", "encode", "encode_ip", "cfg2_probe", "decode", "ldlq", "quant", "shard")}


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O
    O.build()
    return O


@pytest.fixture(scope="session")
def luts(oracle):
    return {n: oracle.codebook_lut(n) for n in CODEBOOKS}


def same_bits(a, b) -> bool:
    """Bit-for-bit equality of two fp32 arrays."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    return a.shape == b.shape and np.array_equal(a.view(np.uint32), b.view(np.uint32))
