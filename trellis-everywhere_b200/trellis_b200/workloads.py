"""Seeded synthetic inputs with the shapes and distributions of the benchmark configurations.

Real checkpoints and calibration activations are not available to the tests and the benchmark; these
generators stand in for them.  The generators that define a configuration bit for bit run on the CPU
generator (``torch.Generator()``), exactly as the configuration states them, so that the matrix is the
same on every machine; only the large random-init matrices of the whole-model case are drawn on the
device.

    second configuration   one 4096 x 4096 matrix, N(0, 0.02^2) with 1 % outliers x 20, incoherence-
                           processed with seed 0, cut into 65 536 tiles (plain TCQ, 3INST, K = 3)
    third configuration    one 12288 -> 4096 (down_proj-shaped) matrix N(0, 0.02^2) with the proxy Hessian
                           H = X^T X / 8192, X Gaussian with per-channel scales log-uniform in [0.1, 10]
"""
from __future__ import annotations

import math
from typing import Tuple

import torch

from . import qtip

CFG2_SHAPE = (4096, 4096)


def cfg2_matrix() -> torch.Tensor:
    """The second configuration's weight matrix (host tensor, CPU generator seed 0)."""
    g = torch.Generator().manual_seed(0)
    n, k = CFG2_SHAPE
    w = torch.randn(n, k, generator=g) * 0.02
    mask = torch.rand(n, k, generator=g) < 0.01
    return torch.where(mask, w * 20, w)


def cfg2_tiles(lut_cpu: torch.Tensor) -> torch.Tensor:
    """The second configuration's encoder input: ``[65536, 256]`` fp32 host tensor.

    ``lut_cpu`` is the codebook's table on the host; its RMS is taken there in fp32, as the reference's
    quantiser does (qtip.py:285), and incoherence processing runs on the host as well (qtip.py:238-260), so
    the tiles depend on nothing but the seed.  About a second of CPU time.
    """
    cb_rms = lut_cpu.float().square().mean().sqrt().item()
    ip = qtip.IPContext(cfg2_matrix(), cb_rms, seed=0)
    return qtip.to_tiles(ip.z).contiguous()


def cfg3_matrix(n_out: int = 4096, k_in: int = 12288, seed: int = 0) -> torch.Tensor:
    """A ``[n_out, k_in]`` matrix N(0, 0.02^2) from the CPU generator (the third configuration's weights)."""
    g = torch.Generator().manual_seed(seed)
    return torch.randn(n_out, k_in, generator=g) * 0.02


def cfg3_hessian(k_in: int = 12288, rows: int = 8192, seed: int = 1, device="cpu") -> torch.Tensor:
    """``H = X^T X / rows`` for ``rows`` Gaussian activations with per-channel scales log-uniform in [0.1, 10].

    The scales and the activations come from the CPU generator in blocks of 1024 rows (so the values do not depend
    on the device); the products are accumulated on ``device`` in fp32.
    """
    g = torch.Generator().manual_seed(seed)
    scales = torch.exp(torch.empty(k_in).uniform_(math.log(0.1), math.log(10.0), generator=g))
    H = torch.zeros(k_in, k_in, device=device)
    sc = scales.to(device)
    for r0 in range(0, rows, 1024):
        x = torch.randn(min(1024, rows - r0), k_in, generator=g).to(device) * sc
        H.addmm_(x.t(), x)
    return H / rows


def cfg3_case(n_out: int = 4096, k_in: int = 12288, rows: int = 8192, device="cpu") -> Tuple[torch.Tensor, torch.Tensor]:
    """``(w [n_out, k_in], H [k_in, k_in])`` of the third configuration on ``device``."""
    return cfg3_matrix(n_out, k_in).to(device), cfg3_hessian(k_in, rows, device=device)
