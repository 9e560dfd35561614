"""The drop-in itself: the REFERENCE's own matrix quantisers, unmodified, with this library's encoder in the place
where they import the Triton one (src/trellis/qtip.py:290-298, src/trellis/ldlq.py:129-134).

The reference modules are the staged copies under ``oracle/_ref`` (see ``oracle/make_ref.py``); the only thing changed
is the attribute their lazy ``from trellis.viterbi_triton import viterbi_tb_triton`` picks up, which is exactly the
one-line patch a maintainer would apply.  Everything around the encoder (incoherence processing, tiling, the LDLQ
recursion, restore) is then the reference's code running on the GPU.
"""
import sys
import types

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    from oracle import make_ref
    if make_ref.staged() is None:
        pytest.skip("reference modules are not staged under oracle/_ref")
    rq, rl = make_ref.import_reference()
    from trellis_b200 import qtip
    try:
        import trellis.viterbi_triton as vt                 # needs triton; only its module object is used
    except Exception:
        vt = types.ModuleType("trellis.viterbi_triton")
        sys.modules["trellis.viterbi_triton"] = vt
    saved = getattr(vt, "viterbi_tb_triton", None)
    vt.viterbi_tb_triton = qtip.viterbi_tb_b200             # <- the whole patch
    yield rq, rl, qtip
    if saved is not None:
        vt.viterbi_tb_triton = saved


def test_reference_plain_quantizer_with_this_encoder(ref, oracle, luts):
    """tcq_quantize_weight(..., backend="triton") of the reference, encoder swapped: equal, bit for bit, to the same
    function's steps with the CPU oracle (= the reference's fp32 DP) as the encoder."""
    rq, _, _ = ref
    torch.manual_seed(0)
    w = torch.randn(128, 256, device="cuda") * 0.02
    lut = rq.codebook_lut("mcg").cuda()
    for K in (2, 3, 4):
        got = rq.tcq_quantize_weight(w, K=K, lut=lut, seed=0, backend="triton")
        assert got.shape == w.shape and got.dtype == w.dtype
        ip = rq.IPContext(w.float(), lut.square().mean().sqrt().item(), seed=0)
        tiles = ip.z.view(8, 16, 16, 16).permute(0, 2, 1, 3).reshape(-1, 256)
        _, dq = oracle.viterbi_tb(tiles.cpu().numpy(), K, luts["mcg"])
        zq = torch.from_numpy(dq).cuda().view(8, 16, 16, 16).permute(0, 2, 1, 3).reshape(128, 256)
        want = ip.restore(zq).to(w.dtype)
        assert torch.equal(got, want), K
        rel = float(((w - got) ** 2).mean() / w.square().mean())
        assert rel < {2: 0.12, 3: 0.035, 4: 0.01}[K]


def test_reference_ldlq_with_this_encoder(ref):
    """The reference's own LDLQ invariants (tests/test_ldlq.py:20-72) through its own code with the encoder swapped:
    L = 0 reproduces the plain quantiser exactly, and a real Hessian lowers tr(E H E^T)."""
    rq, rl, _ = ref
    torch.manual_seed(0)
    lut = rq.codebook_lut("mcg").cuda()
    w = torch.randn(64, 256, device="cuda") * 0.02
    base = rq.tcq_quantize_weight(w, K=3, lut=lut, seed=0, backend="triton")
    orig = rl.block_ldl
    rl.block_ldl = lambda H, b=16: torch.zeros(H.shape[0], H.shape[0], device=H.device)
    try:
        ld0 = rl.tcq_quantize_weight_ldlq(w, K=3, lut=lut, H=torch.eye(256, device="cuda"), seed=0, sigma_reg=0.0,
                                          backend="triton")
    finally:
        rl.block_ldl = orig
    assert float(((base - ld0) ** 2).mean() / base.square().mean()) < 1e-8

    torch.manual_seed(1)
    w = torch.randn(64, 256, device="cuda") * 0.02
    A = torch.randn(256, 256, device="cuda")
    H = (A.T @ A) / 256 + torch.eye(256, device="cuda")
    base = rq.tcq_quantize_weight(w, K=3, lut=lut, seed=0, backend="triton")
    ld = rl.tcq_quantize_weight_ldlq(w, K=3, lut=lut, H=H, seed=0, backend="triton")

    def obj(wq):
        E = (w - wq).float()
        return float(torch.einsum("nk,kj,nj->", E, H, E))

    assert obj(ld) < obj(base)


def test_mirror_modules_agree_with_the_reference_callers(ref):
    """``trellis_b200.qtip.tcq_quantize_weight`` (device incoherence-processing kernels) against the reference's caller
    with the same encoder: the two incoherence-processing routes differ in the last ulps, so a few codes may flip;
    the quantisation errors must agree within 1 % and the results' difference stay below 1e-3 of their energy."""
    rq, _, q = ref
    torch.manual_seed(4)
    w = torch.randn(128, 256, device="cuda") * 0.02
    lut = rq.codebook_lut("mcg").cuda()
    theirs = rq.tcq_quantize_weight(w, K=3, lut=lut, seed=0, backend="triton")
    ours = q.tcq_quantize_weight(w, K=3, lut=lut, seed=0, backend="b200")
    rel = lambda x: float(((w - x) ** 2).mean() / w.square().mean())
    assert abs(rel(ours) - rel(theirs)) / rel(theirs) < 0.01
    assert float(((ours - theirs) ** 2).sum() / theirs.square().sum()) < 1e-3
