#!/usr/bin/env python
"""Stage the UNMODIFIED reference modules of the hot path under ``oracle/_ref/`` (git-ignored).

TEST / BASELINE INFRASTRUCTURE ONLY, like the rest of ``oracle/``: nothing under the shipped package may
import what this stages.  The reference (Azimml/trellis-everywhere) is pure Python on this path, so "building"
it means placing three of its files where a machine without the checkout can still import them:

    src/trellis/qtip.py            codebooks, viterbi_tb / _viterbi_pass (the fp32 PyTorch DP), IPContext,
                                   tcq_quantize_weight
    src/trellis/ldlq.py            ldlq, block_ldl, tcq_quantize_weight_ldlq
    src/trellis/viterbi_triton.py  the Triton encoder (the GPU kernel this library replaces)

The files are copied byte for byte (``staged()`` checks their sha256 against the checkout when it is there) and
are never committed.  Users: the benchmark's reference arms (``bench.py --impl reference`` times the reference's
own ``viterbi_tb`` on the host cores, ``--impl reference-triton`` its Triton encoder on the GPU) and the drop-in
tests, which run the reference's own matrix quantisers with this library's encoder swapped in.

    python oracle/make_ref.py [/path/to/trellis-everywhere]
"""
from __future__ import annotations

import hashlib
import importlib
import os
import shutil
import sys
from typing import Optional

_HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(_HERE, "_ref")
FILES = ("qtip.py", "ldlq.py", "viterbi_triton.py")


def default_checkout() -> str:
    """``$TRELLIS_REFERENCE_ROOT`` or a folder named ``reference`` beside this repository."""
    return os.environ.get("TRELLIS_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")


def _sha(path: str) -> str:
    return hashlib.sha256(open(path, "rb").read()).hexdigest()


def stage(checkout: Optional[str] = None) -> Optional[str]:
    """Copy the three modules from ``checkout``; returns ``oracle/_ref`` or None if there is no checkout."""
    checkout = checkout or default_checkout()
    src = os.path.join(checkout, "src", "trellis")
    if not all(os.path.isfile(os.path.join(src, f)) for f in FILES):
        return None
    dst = os.path.join(REF_DIR, "trellis")
    os.makedirs(dst, exist_ok=True)
    for f in FILES:
        shutil.copyfile(os.path.join(src, f), os.path.join(dst, f))
    with open(os.path.join(REF_DIR, "SHA256SUMS"), "w") as out:
        for f in FILES:
            out.write(f"{_sha(os.path.join(dst, f))}  trellis/{f}\n")
    return REF_DIR


def staged() -> Optional[str]:
    """``oracle/_ref`` if all three modules are there and match their recorded digests, else None."""
    dst = os.path.join(REF_DIR, "trellis")
    sums = os.path.join(REF_DIR, "SHA256SUMS")
    if not os.path.isfile(sums) or not all(os.path.isfile(os.path.join(dst, f)) for f in FILES):
        return None
    want = dict(reversed(line.split()) for line in open(sums).read().splitlines() if line.strip())
    for f in FILES:
        if want.get(f"trellis/{f}") != _sha(os.path.join(dst, f)):
            return None
    return REF_DIR


def import_reference():
    """``(trellis.qtip, trellis.ldlq)`` of the staged reference, or raises ImportError if it is not staged."""
    root = staged()
    if root is None:
        raise ImportError("the reference modules are not staged under oracle/_ref (run oracle/make_ref.py with a checkout)")
    if root not in sys.path:
        sys.path.insert(0, root)
    return importlib.import_module("trellis.qtip"), importlib.import_module("trellis.ldlq")


if __name__ == "__main__":
    got = stage(sys.argv[1] if len(sys.argv) > 1 else None)
    print(got if got else "no checkout found: nothing staged")
    sys.exit(0 if got else 1)
