"""LDLQ error feedback around the B200 tile encoder.

Mirrors ``src/trellis/ldlq.py`` of the reference (same names, arguments and return
values).  The column-block recursion and its GEMMs stay in PyTorch on the matrix's
own GPU; the only part that runs in the CUDA extension is what the recursion
spends its time in, the ``enc`` step (ldlq.py:136-143): a 16-row block of the
transposed matrix is cut into 256-weight tiles, encoded, and the reconstruction
is handed back for the error update.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

from . import qtip as _qtip
from .qtip import (T_SEQ, CodebookLike, IPContext, _check_backend, _cuda_device, _pow2_block, block_hadamard,
                   codebook_id, codebook_lut, encode, encode_rows, CODEBOOK_NAMES)


def regularize_H(H: torch.Tensor, sigma_reg: float = 0.025) -> torch.Tensor:
    """H + sigma_reg * mean(diag H) * I  (ldlq.py:24-29)."""
    out = H.clone()
    out.diagonal().add_(sigma_reg * torch.diag(H).mean())
    return out


def block_ldl(H: torch.Tensor, b: int = 16) -> Optional[torch.Tensor]:
    """Block LDL factor of H with b x b unit diagonal blocks, returned with those blocks zeroed.

    Follows ldlq.py:32-70: Cholesky (retried up to 14 times with damping
    ``2^attempt * 0.01 * max(max|diag H|, 1)`` added to the diagonal of the original
    H), then every block column is multiplied by the inverse of its diagonal block,
    and the scalar diagonal is cleared.  Returns None if H never factorises; the
    caller then quantises without feedback.
    """
    k = H.shape[0]
    if k % b:
        raise ValueError(f"k={k} not divisible by block {b}")
    m = k // b
    damp = max(float(torch.diag(H).abs().max()), 1.0) * 0.01
    chol = None
    trial = H
    for attempt in range(14):
        chol, info = torch.linalg.cholesky_ex(trial)
        if int(info) == 0 and bool(torch.isfinite(chol).all()):
            break
        chol = None
        trial = H.clone()
        trial.diagonal().add_((2.0 ** attempt) * damp)
    if chol is None:
        return None
    blocks = chol.reshape(m, b, m, b)
    idx = torch.arange(m, device=H.device)
    dinv = torch.linalg.inv(blocks[idx, :, idx, :])                      # (m, b, b)
    out = torch.einsum("ibjc,jcd->ibjd", blocks, dinv).reshape(k, k).contiguous()
    out.diagonal().zero_()
    return out


@torch.no_grad()
def ldlq(Wt: torch.Tensor, L: torch.Tensor, enc: Callable[[torch.Tensor], torch.Tensor], buf: int = 128) -> torch.Tensor:
    """Reverse-order block error feedback (ldlq.py:72-99).

    ``Wt (k, n)`` is the transposed matrix in incoherence-processed space, ``L (k, k)``
    the factor from ``block_ldl``; ``enc`` quantises one compensated ``(16, n)`` row
    block.  Rows are visited from the last 16-row block to the first; inside a span
    of ``buf`` rows the correction uses the span's own errors, and after a span is
    finished its errors are pushed to all earlier rows with one fp32 GEMM.  (The
    reference pushes them to every row, ldlq.py:97-98; rows of finished spans are never
    read again and L is zero above its diagonal, so only the earlier rows are updated here.)

    This is the general form for any ``enc``; ``ldlq_b200`` is the same recursion with the
    encoder step fused into the B200 kernels.
    """
    k, n = Wt.shape
    src = Wt.float()
    Lf = L.float()
    Wq = torch.zeros_like(src)
    carry = torch.zeros_like(src)          # feedback owed to each row by finished spans (and, in place, by this span)
    hi = k
    while hi > 0:
        lo = max(hi - buf, 0)
        for bj in range(hi, lo, -16):
            bi = bj - 16
            if bj < hi:                                                   # errors of the span's later blocks
                carry[bi:bj].addmm_(Lf[bj:hi, bi:bj].t(), src[bj:hi] - Wq[bj:hi])
            Wq[bi:bj] = enc(src[bi:bj] + carry[bi:bj]).float()
        if lo > 0:
            carry[:lo].addmm_(Lf[lo:hi, :lo].t(), src[lo:hi] - Wq[lo:hi])
        hi = lo
    return Wq.to(Wt.dtype)


@torch.no_grad()
def ldlq_b200(Wt: torch.Tensor, L: torch.Tensor, K: int, codebook: CodebookLike, buf: int = 128,
              packed: Optional[torch.Tensor] = None, tap: Optional[Callable] = None) -> torch.Tensor:
    """``ldlq`` (ldlq.py:72-99) with the encoder step running in place on the recursion's matrices.

    Per 16-row block the general form costs a subtraction, a GEMM, an addition, a transposing copy, the
    encoder, another transposing copy, a copy into ``Wq`` and (for an exporter) a copy of the packed words;
    here it is the GEMM plus one ``encode_rows`` call: the step kernel reads ``src + carry`` straight from the
    row block, and the traceback kernel writes the reconstruction, the block error ``src - Wq`` and the packed
    words to their final places.  Same arithmetic in the same order, so the codes equal those of
    ``ldlq(Wt, L, make_enc(K, codebook))`` bit for bit.

    ``packed``: optional int32 ``[n/16, k/16, 8K]`` array that receives every tile's code words in the
    exporter's tile order (export_packed_8b.py:114-131).  ``tap(bi, src_block, carry_block, wq_block)`` (optional)
    is called after each block's encoder call has been queued, with views of that block's 16 rows (for tests that
    record what the encoder was given and what it returned).  Returns ``Wq (k, n)``.
    """
    k, n = Wt.shape
    if k % 16 or n % 16:
        raise ValueError(f"shape {(k, n)} not 16-divisible")
    src = Wt.float().contiguous()
    Lf = L.float()
    Wq = torch.empty_like(src)
    err = torch.empty_like(src)            # src - Wq of the finished blocks, written by the encoder
    carry = torch.zeros_like(src)
    cid = codebook_id(codebook)
    hi = k
    while hi > 0:
        lo = max(hi - buf, 0)
        for bj in range(hi, lo, -16):
            bi = bj - 16
            if bj < hi:
                carry[bi:bj].addmm_(Lf[bj:hi, bi:bj].t(), err[bj:hi])
            encode_rows(src[bi:bj], carry[bi:bj], K, cid, Wq[bi:bj], err[bi:bj],
                        packed[:, bi // 16] if packed is not None else None)
            if tap is not None:
                tap(bi, src[bi:bj], carry[bi:bj], Wq[bi:bj])
        if lo > 0:
            carry[:lo].addmm_(Lf[lo:hi, :lo].t(), err[lo:hi])
        hi = lo
    return Wq.to(Wt.dtype)


@torch.no_grad()
def ldlq_row_groups(Wt: torch.Tensor, L: torch.Tensor, make_enc_for: Optional[Callable[[int, int], Callable]], groups: int = 2,
                    buf: int = 128, fused: Optional[Callable[[torch.Tensor, int, int], torch.Tensor]] = None) -> torch.Tensor:
    """``ldlq`` with the output channels (columns of ``Wt``) cut into ``groups`` slices that run side by side.

    The recursion couples input channels only, so column slices of ``Wt`` are independent problems with the same
    ``L``.  One recursion issues encoder calls of ``n/16`` tiles one after another, which rarely fill the last round
    of SMs (256 tiles occupy 64 of a B200's 74 SM pairs); slices on separate CUDA streams (one host thread each) let
    one slice's kernels take the SMs the other leaves idle.  ``make_enc_for(a, b)`` returns the ``enc`` closure for
    columns ``a:b`` (16-aligned); alternatively ``fused(Wt_slice, a, b)`` runs a slice's whole recursion (the
    ``ldlq_b200`` form).  Equal to ``ldlq`` up to the summation order of the feedback GEMMs, whose column count differs.
    """
    import threading
    k, n = Wt.shape
    groups = max(1, min(int(groups), n // 16))

    def solve(part: torch.Tensor, a: int, b: int) -> torch.Tensor:
        return fused(part, a, b) if fused is not None else ldlq(part, L, make_enc_for(a, b), buf)

    if groups == 1:
        return solve(Wt, 0, n)
    per = -(-(n // 16) // groups) * 16
    bounds = [(a, min(a + per, n)) for a in range(0, n, per)]
    out = torch.empty_like(Wt)
    dev = Wt.device
    caller = torch.cuda.current_stream(dev)
    errors = []

    def run(a: int, b: int) -> None:
        try:
            with torch.cuda.device(dev):
                s = torch.cuda.Stream(dev)
                s.wait_stream(caller)
                try:
                    with torch.cuda.stream(s):
                        out[:, a:b] = solve(Wt[:, a:b].contiguous(), a, b)
                    s.synchronize()
                finally:
                    _qtip.release_workspace(dev, s)     # this stream is never used again
        except BaseException as e:          # surfaced by the caller below
            errors.append(e)

    threads = [threading.Thread(target=run, args=ab) for ab in bounds]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if errors:
        raise errors[0]
    return out


def _transform_H(H: torch.Tensor, su: torch.Tensor, block: int = 128) -> torch.Tensor:
    """Bring the input-axis Hessian into incoherence-processed space: signs + block-Hadamard on both sides (ldlq.py:102-109)."""
    H = su[:, None] * H * su[None, :]
    return block_hadamard(block_hadamard(H, 0, block), 1, block)


def rows_to_tiles(rows: torch.Tensor) -> torch.Tensor:
    """``(16 in-channels, n_out)`` row block -> ``(n_out/16, 256)`` tiles with t = (out % 16) * 16 + in (ldlq.py:138-140)."""
    n_out = rows.shape[1]
    return rows.t().reshape(n_out // 16, T_SEQ).contiguous()


def tiles_to_rows(dq: torch.Tensor, n_out: int) -> torch.Tensor:
    """Inverse of ``rows_to_tiles`` (ldlq.py:142-143)."""
    return dq.reshape(n_out, 16).t().contiguous()


def make_enc(K: int, codebook: CodebookLike, sink: Optional[Callable] = None) -> Callable[[torch.Tensor], torch.Tensor]:
    """The ``enc`` closure of ldlq.py:136-143 on the B200 encoder.

    ``sink(packed_words)`` (optional) receives each call's packed codes, which is what
    the reference's exporter captures in its twin closure (export_packed_8b.py:117-125).
    """
    cid = codebook_id(codebook)

    def enc(rows: torch.Tensor) -> torch.Tensor:
        r = encode(rows_to_tiles(rows), K, cid, want_dq=True, want_sse=False)
        if sink is not None:
            sink(r.packed)
        return tiles_to_rows(r.dq, rows.shape[1])

    return enc


@torch.no_grad()
def tcq_quantize_weight_ldlq(w: torch.Tensor, K: int, lut: CodebookLike, H: torch.Tensor, seed: int = 0,
                             sigma_reg: float = 0.025, dp_dtype=torch.float32, backend: str = "auto",
                             row_groups: int = 1) -> torch.Tensor:
    """LDLQ variant of ``tcq_quantize_weight`` with the signature of ldlq.py:112-154.

    ``w (n_out, k_in)``; ``H (k_in, k_in)`` proxy Hessian in the original space.
    ``dp_dtype`` is ignored (path metrics are always fp32).  ``row_groups`` > 1 (not in the reference) runs that
    many slices of output channels side by side on separate streams (``ldlq_row_groups``).
    """
    _check_backend(backend)
    n, k = w.shape
    if n % 16 or k % 16:
        raise ValueError(f"shape {tuple(w.shape)} not 16-divisible")
    dev = _cuda_device(w)
    lut_t = lut if isinstance(lut, torch.Tensor) else codebook_lut(CODEBOOK_NAMES[codebook_id(lut)], dev)
    cb_rms = lut_t.float().square().mean().sqrt().item()
    ip = IPContext(w.to(dev).float(), cb_rms, seed=seed)
    Ht = _transform_H(H.to(dev).float(), ip.su, block=_pow2_block(k, 128))
    Lm = block_ldl(regularize_H(Ht, sigma_reg), b=16)
    if Lm is None:                                  # degenerate Hessian: no feedback for this matrix (ldlq.py:148-151)
        Lm = torch.zeros(k, k, device=dev)
    zq_t = ldlq_row_groups(ip.z.t().contiguous(), Lm, None, row_groups,
                           fused=lambda part, a, b: ldlq_b200(part, Lm, K, lut))
    return ip.restore(zq_t.t().contiguous()).to(dtype=w.dtype, device=w.device)
