"""Quantizer plug-in interface (``src/trellis/quant.py:20-26`` of the reference) for the B200 codec.

The reference's model-level drivers walk ``nn.Linear`` modules and call
``Quantizer.quantize_weight(w) -> w_fake``; ``TrellisQuantizer`` is that interface
on top of the CUDA encoder, with or without LDLQ feedback.
"""
from __future__ import annotations

import zlib
from typing import Callable, Optional

import torch
import torch.nn as nn

from .ldlq import tcq_quantize_weight_ldlq
from .qtip import CodebookLike, tcq_quantize_weight


class Quantizer:
    """Interface: map a weight matrix ``[out, in]`` to its fake-quantised version."""
    name: str = "identity"
    bpw: float = 16.0

    def quantize_weight(self, w: torch.Tensor) -> torch.Tensor:  # pragma: no cover - interface
        return w


class TrellisQuantizer(Quantizer):
    """Tail-biting trellis-coded quantisation at K bits per weight on the B200 encoder.

    ``hessian`` (optional): callable ``name -> H`` or a tensor; when given, LDLQ
    feedback is used for that matrix, as ``scripts/run_tcq_eval.py:113-127`` does.
    ``seed_from_name`` reproduces the driver's ``seed = crc32(name)``.
    """

    def __init__(self, K: int = 3, codebook: CodebookLike = "mcg", seed: int = 0, sigma_reg: float = 0.025):
        self.K, self.codebook, self.seed, self.sigma_reg = K, codebook, seed, sigma_reg
        self.name = f"tcq-b200-k{K}"
        self.bpw = float(K)

    def quantize_weight(self, w: torch.Tensor, H: Optional[torch.Tensor] = None, seed: Optional[int] = None) -> torch.Tensor:
        s = self.seed if seed is None else seed
        if H is None:
            return tcq_quantize_weight(w, self.K, self.codebook, seed=s, backend="b200")
        return tcq_quantize_weight_ldlq(w, self.K, self.codebook, H, seed=s, sigma_reg=self.sigma_reg, backend="b200")


def seed_from_name(name: str) -> int:
    """Per-matrix seed of the reference driver (``zlib.crc32(name)``, run_tcq_eval.py:115)."""
    return zlib.crc32(name.encode())


@torch.no_grad()
def apply_fake_quant(model: nn.Module, quantizer: Quantizer, skip: Callable[[str], bool] = lambda n: False) -> int:
    """Replace every ``nn.Linear`` weight by its fake-quantised version (quant.py:72-85). Returns the count."""
    count = 0
    for name, mod in model.named_modules():
        if isinstance(mod, nn.Linear) and not skip(name):
            mod.weight.data = quantizer.quantize_weight(mod.weight.data).to(mod.weight.dtype)
            count += 1
    return count
