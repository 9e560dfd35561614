"""Packed-model shard files in the layout the reference's exporter writes and its browser loader reads.

Layout facts restated from the reference (format only; no browser can be run here to load the result):

* A shard ``<file>.bin`` is the plain concatenation of tensors' little-endian bytes; ``<file>.bin.json`` maps
  tensor name -> ``{"offset", "shape", "dtype": "f16"|"u32"|"f32", "shard": <file name>}``
  (``scripts/export_packed_8b.py:65-79``).  A shard exists once both files do (``:81``).
* A quantised matrix ``<name>`` (e.g. ``model.layers.0.mlp.up_proj.weight``) is six tensors --
  ``.bits`` u32 ``[tiles, 8K]`` (tile = (row/16)*(k/16) + col/16, bit (255-t)*K+kb of the tile's stream),
  ``.su`` / ``.sv`` sign vectors, ``.isc`` / ``.osc`` channel scales (all f16), ``.scale`` f32 ``[1]`` -- plus a
  descriptor ``{"quant": true, "n_out", "k_in", "K", "block", "tiles_out", "tiles_in", "shard"}`` under the bare
  name (``scripts/export_packed_8b.py:134-143``).
* ``manifest.json`` is the union of all ``*.bin.json`` fragments (``scripts/export_packed_8b.py:268-272``).
* The consumer evaluates ``y = W_hat x`` without ever forming ``W_hat``: ``x`` is multiplied by ``su`` and
  ``isc * scale``, block-Hadamard-transformed, multiplied by the decoded code matrix, block-Hadamard-transformed
  over the output axis (block fitted to ``n_out``), and multiplied by ``osc`` and ``sv``
  (``web/packed.js:163-182``).  ``packed_linear`` below does the same with the CUDA decoder, and is how the tests
  check that a shard written here holds everything needed.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Optional

import numpy as np
import torch

from . import qtip

_DTYPE_TAG = {np.dtype(np.float16): "f16", np.dtype(np.uint32): "u32", np.dtype(np.float32): "f32"}
_TAG_DTYPE = {v: k for k, v in _DTYPE_TAG.items()}
_QUANT_PARTS = ("bits", "su", "sv", "isc", "osc", "scale")


class Shard:
    """Accumulates tensors in memory; ``flush`` writes ``path`` and ``path + '.json'`` (data first, then index)."""

    def __init__(self, path: str):
        self.path = path
        self.chunks = []
        self.size = 0
        self.index: Dict[str, dict] = {}

    def put(self, name: str, value, dtype) -> None:
        dt = np.dtype(dtype)
        if dt not in _DTYPE_TAG:
            raise ValueError(f"shards hold f16, u32 and f32 tensors, not {dt}")
        if name in self.index:
            raise KeyError(f"{name} is already in {os.path.basename(self.path)}")
        if isinstance(value, torch.Tensor):
            value = value.detach().cpu().numpy()
        arr = np.asarray(value)
        if dt == np.uint32 and arr.dtype == np.int32:
            arr = arr.view(np.uint32)                     # packed words come off the GPU as int32 bit patterns
        arr = np.ascontiguousarray(arr.astype(dt, copy=False))
        self.index[name] = {"offset": self.size, "shape": list(arr.shape), "dtype": _DTYPE_TAG[dt],
                            "shard": os.path.basename(self.path)}
        raw = arr.tobytes()
        self.chunks.append(raw)
        self.size += len(raw)

    def put_quant(self, name: str, packed, ip: "qtip.IPContext", n: int, k: int, K: int) -> None:
        """One quantised matrix: packed words + everything ``IPContext.restore`` needs."""
        nw = qtip.T_SEQ * K // 32
        if tuple(packed.shape) != ((n // 16) * (k // 16), nw):
            raise ValueError(f"packed words must be [{(n // 16) * (k // 16)}, {nw}], got {tuple(packed.shape)}")
        self.put(name + ".bits", packed, np.uint32)
        self.put(name + ".su", ip.su, np.float16)
        self.put(name + ".sv", ip.sv, np.float16)
        self.put(name + ".isc", ip.in_s, np.float16)
        self.put(name + ".osc", ip.out_s, np.float16)
        self.put(name + ".scale", np.array([ip.scale], dtype=np.float32), np.float32)
        self.index[name] = {"quant": True, "n_out": n, "k_in": k, "K": K, "block": qtip._pow2_block(k, 128),
                            "tiles_out": n // 16, "tiles_in": k // 16, "shard": os.path.basename(self.path)}

    def flush(self) -> None:
        tmp = self.path + ".part"
        with open(tmp, "wb") as f:
            for raw in self.chunks:
                f.write(raw)
        os.replace(tmp, self.path)
        with open(self.path + ".json.part", "w") as f:
            json.dump(self.index, f)
        os.replace(self.path + ".json.part", self.path + ".json")     # the index appears last: shard_done is atomic


def shard_done(path: str) -> bool:
    return os.path.exists(path) and os.path.exists(path + ".json")


def merge_manifest(out_dir: str) -> Dict[str, dict]:
    """Union of every ``*.bin.json`` in ``out_dir`` (sorted by file name), written to ``manifest.json``."""
    manifest: Dict[str, dict] = {}
    for fn in sorted(os.listdir(out_dir)):
        if fn.endswith(".bin.json"):
            with open(os.path.join(out_dir, fn)) as f:
                manifest.update(json.load(f))
    with open(os.path.join(out_dir, "manifest.json"), "w") as f:
        json.dump(manifest, f)
    return manifest


def read_tensor(out_dir: str, manifest: Dict[str, dict], name: str) -> np.ndarray:
    m = manifest[name]
    if m.get("quant"):
        raise KeyError(f"{name} is a quantised matrix; read it with read_quant")
    dt = _TAG_DTYPE[m["dtype"]]
    count = int(np.prod(m["shape"])) if m["shape"] else 1
    return np.fromfile(os.path.join(out_dir, m["shard"]), dtype=dt, count=count, offset=m["offset"]).reshape(m["shape"])


def read_quant(out_dir: str, manifest: Dict[str, dict], name: str) -> dict:
    """Descriptor of a quantised matrix plus its six tensors as numpy arrays."""
    desc = dict(manifest[name])
    if not desc.get("quant"):
        raise KeyError(f"{name} is not a quantised matrix")
    for part in _QUANT_PARTS:
        desc[part] = read_tensor(out_dir, manifest, f"{name}.{part}")
    return desc


@torch.no_grad()
def packed_linear(q: dict, x: torch.Tensor, codebook="mcg", device=None) -> torch.Tensor:
    """``y = W_hat x`` from a ``read_quant`` record, the way the reference's runtime folds the restore
    (``web/packed.js:163-182``); ``x`` is ``[k_in]`` or ``[k_in, m]``.  The product with the code matrix is the
    CUDA decode-matvec kernel (``qtip.decode_matvec``)."""
    dev = torch.device(device) if device is not None else qtip._cuda_device(x if x.is_cuda else None)
    n, k, K = q["n_out"], q["k_in"], q["K"]
    f = lambda a: torch.from_numpy(np.ascontiguousarray(a).astype(np.float32)).to(dev)
    col = x.to(dev, torch.float32).reshape(k, -1)
    xf = col * (f(q["su"]) * f(q["isc"]) * float(q["scale"][0]))[:, None]
    xf = qtip.block_hadamard(xf, 0, q["block"])
    packed = torch.from_numpy(np.ascontiguousarray(q["bits"]).view(np.int32)).to(dev)
    prod = qtip.decode_matvec(packed, n, k, K, codebook, xf.t().contiguous()).t()       # [n, m]; the code matrix is never formed
    t = qtip.block_hadamard(prod, 0, qtip._pow2_block(n, 128))
    y = t * (f(q["osc"]) * f(q["sv"]))[:, None]
    return y.reshape(n, *x.shape[1:])


def write_layer_shard(out_dir: str, layer: int, matrices: Dict[str, tuple], extras: Optional[Dict[str, np.ndarray]] = None) -> str:
    """``layer_<ll>.bin``: ``matrices`` maps a linear's name (without ``.weight``) to ``(packed, ip, n, k, K)``;
    ``extras`` are fp16 side tensors such as norm weights (``scripts/export_packed_8b.py:193-219``)."""
    path = os.path.join(out_dir, f"layer_{layer:02d}.bin")
    sh = Shard(path)
    for name, (packed, ip, n, k, K) in matrices.items():
        sh.put_quant(name + ".weight", packed, ip, n, k, K)
    for name, arr in (extras or {}).items():
        sh.put(name, arr, np.float16)
    sh.flush()
    return path
