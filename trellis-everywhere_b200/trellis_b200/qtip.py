"""Host-side mirror of the reference's tile codec interface, running on the B200 kernels.

Mirrors ``src/trellis/qtip.py`` and ``src/trellis/viterbi_triton.py`` of
Azimml/trellis-everywhere: same function names, argument meaning and return
types, so callers switch by changing an import:

    reference                                      this module
    ---------------------------------------------  -----------------------------------
    codebook_lut(name, device)      qtip.py:59     codebook_lut(name, device)
    viterbi_tb(w, K, lut)           qtip.py:124    viterbi_tb_b200(w, K, lut)  /  viterbi_tb
    viterbi_tb_triton(w, K, lut)    v_triton:121   viterbi_tb_b200(w, K, lut)
    _viterbi_pass / viterbi_pass_triton            viterbi_pass_b200(w, K, overlap, lut)
    decode_recursive / decode_window qtip.py:70,82 decode_recursive / decode_window
    pack_bits_np  export_packed_8b.py:52           pack_bits(bits, K)
    IPContext                       qtip.py:226    IPContext
    tcq_quantize_weight             qtip.py:272    tcq_quantize_weight(..., backend="b200")

plus the richer ``encode`` / ``decode_packed`` pair that returns what the kernels
produce natively (packed code words, reconstruction, per-tile squared error).

The dynamic programme always runs in fp32 and is bit-identical to the reference's
``viterbi_tb(..., dp_dtype=torch.float32)``.  Everything here needs the CUDA
extension and a GPU; there is no CPU implementation and no other backend.
"""
from __future__ import annotations

import threading
import weakref
from typing import NamedTuple, Optional, Union

import torch

from . import _lib

L = 16
S = 1 << L
T_SEQ = 256
CODEBOOK_IDS = {"1mad": 0, "3inst": 1, "mcg": 2}
CODEBOOK_NAMES = {v: k for k, v in CODEBOOK_IDS.items()}

CodebookLike = Union[str, int, torch.Tensor]


# --------------------------------------------------------------------------- plumbing
def _cuda_device(t: Optional[torch.Tensor] = None) -> torch.device:
    if not torch.cuda.is_available():
        raise RuntimeError("trellis_b200 needs a CUDA device (sm_100a); there is no CPU fallback")
    if t is not None and t.is_cuda:
        return t.device
    return torch.device("cuda", torch.cuda.current_device())


def _stream(dev: torch.device) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


def _to_dev(t: torch.Tensor, dev: torch.device, dtype: torch.dtype) -> torch.Tensor:
    """Contiguous tensor of `dtype` on `dev`; host tensors go through pinned memory."""
    if t.is_cuda:
        return t.to(device=dev, dtype=dtype).contiguous()
    t = t.to(dtype).contiguous()
    if not t.is_pinned():
        t = t.pin_memory()
    return t.to(dev, non_blocking=True)


_workspaces: dict = {}
_workspaces_lock = threading.Lock()


def _workspace(dev: torch.device, n_tiles: int, K: int) -> torch.Tensor:
    """Grow-only scratch per (device, stream): backpointers and per-tile hand-off words.

    Kernels of one stream run one after another, so a stream's calls can share one block; calls on
    different streams may overlap and get different blocks.  Code that creates streams of its own
    (``ldlq.ldlq_row_groups``, ``model.encode_model``) hands the block back with
    ``release_workspace`` when its stream is done, otherwise every short-lived stream would keep
    gigabytes alive.
    """
    need = int(_lib.lib().tcq_workspace_bytes(n_tiles, K))
    key = (dev.index, _stream(dev))
    with _workspaces_lock:
        ws = _workspaces.get(key)
        if ws is None or ws.numel() < need:
            _workspaces[key] = None          # drop the old block before asking for a larger one
            ws = torch.empty(need, dtype=torch.uint8, device=dev)
            _workspaces[key] = ws
    return ws


def release_workspace(dev: torch.device, stream: Optional[torch.cuda.Stream] = None) -> None:
    """Free the scratch block cached for ``stream`` (default: the current stream) of ``dev``.

    Call it after the stream's work has finished (the block goes back to the allocator at once).
    """
    handle = stream.cuda_stream if stream is not None else _stream(dev)
    with _workspaces_lock:
        _workspaces.pop((dev.index, handle), None)


def workspace_status(n_tiles: int, K: int, device=None) -> None:
    """Health of the last device encode of ``n_tiles`` tiles at ``K`` on the current stream (synchronises).

    Raises ``TcqError`` if a bounded in-kernel wait gave up (outputs invalid) or if some weight of
    that call was NaN or infinite (its tile's codes are meaningless); returns None otherwise.
    """
    dev = torch.device(device) if device is not None else _cuda_device()
    ws = _workspace(dev, n_tiles, K)
    with torch.cuda.device(dev):
        rc = _lib.lib().tcq_workspace_status(ws.data_ptr(), ws.numel(), n_tiles, K, _stream(dev))
    _lib.check(rc, "tcq_workspace_status")


def release_workspaces() -> None:
    """Free the cached scratch buffers of every stream."""
    with _workspaces_lock:
        _workspaces.clear()


# --------------------------------------------------------------------------- codebooks
_lut_cache: dict = {}
_id_cache: dict = {}


def codebook_lut(name: str, device="cpu") -> torch.Tensor:
    """fp32 value of every 16-bit state, computed by the device codebook functions.

    Same contract as the reference's ``codebook_lut`` (qtip.py:59-66): ``[65536]`` fp32,
    default device "cpu".  The table is an encode-time convenience for callers that
    index it; the kernels never read it.
    """
    if name not in CODEBOOK_IDS:
        raise KeyError(name)
    dev = _cuda_device()
    key = (name, dev.index)
    lut = _lut_cache.get(key)
    if lut is None:
        lut = torch.empty(S, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().tcq_codebook_lut(CODEBOOK_IDS[name], lut.data_ptr(), _stream(dev)), "tcq_codebook_lut")
            torch.cuda.current_stream(dev).synchronize()      # other streams (threads) read the cached table
        _lut_cache[key] = lut
    return lut.to(device).clone()


def codebook_id(codebook: CodebookLike) -> int:
    """Map a codebook name, id or 65536-entry table to the id the kernels take.

    The reference passes the table around as "the codebook"; the kernels compute
    values from the state number instead, so a table is accepted only if it is
    bit-identical to one of the three computed codebooks.
    """
    if isinstance(codebook, str):
        if codebook not in CODEBOOK_IDS:
            raise ValueError(f"unknown codebook {codebook!r}; expected one of {sorted(CODEBOOK_IDS)}")
        return CODEBOOK_IDS[codebook]
    if isinstance(codebook, int):
        if codebook not in CODEBOOK_NAMES:
            raise ValueError(f"unknown codebook id {codebook}")
        return codebook
    if not isinstance(codebook, torch.Tensor) or codebook.numel() != S:
        raise ValueError("codebook must be a name, an id or a [65536] table")
    # Remember the answer per tensor OBJECT (weak reference + version counter): LDLQ hands the
    # same table to hundreds of encoder calls, and a freed table's address may be reused.
    key = id(codebook)
    hit = _id_cache.get(key)
    if hit is not None and hit[0]() is codebook and hit[1] == codebook._version:
        return hit[2]
    flat = codebook.reshape(-1).float()
    for name, cid in CODEBOOK_IDS.items():
        if torch.equal(flat, codebook_lut(name, flat.device)):
            if len(_id_cache) > 64:
                _id_cache.clear()
            _id_cache[key] = (weakref.ref(codebook), codebook._version, cid)
            return cid
    raise ValueError("table is not one of the computed codebooks (1mad, 3inst, mcg); arbitrary tables are not supported")


# --------------------------------------------------------------------------- encode
class Encoded(NamedTuple):
    packed: torch.Tensor                 # int32 [n, 8K]: the u32 code words (bit kb of symbol t at bit (255-t)*K+kb)
    dq: Optional[torch.Tensor]           # fp32 [n, 256] reconstruction
    sse: Optional[torch.Tensor]          # fp32 [n] squared error per tile
    bits: Optional[torch.Tensor]         # int64 [n, 256] symbols


def _encode_device(wd: torch.Tensor, K: int, cid: int, packed, dq, sse, bits) -> None:
    """One C-ABI call on device tensors (outputs preallocated; None = not wanted).  No host sync."""
    n = wd.shape[0]
    if not n:
        return
    dev = wd.device
    ws = _workspace(dev, n, K)
    with torch.cuda.device(dev):
        rc = _lib.lib().tcq_encode_tb(wd.data_ptr(), n, K, cid, packed.data_ptr(),
                                      bits.data_ptr() if bits is not None else None,
                                      dq.data_ptr() if dq is not None else None,
                                      sse.data_ptr() if sse is not None else None,
                                      ws.data_ptr(), ws.numel(), _stream(dev))
    _lib.check(rc, "tcq_encode_tb")


@torch.no_grad()
def encode_rows(src: torch.Tensor, comp: Optional[torch.Tensor], K: int, codebook: CodebookLike, wq: torch.Tensor,
                err: Optional[torch.Tensor] = None, packed: Optional[torch.Tensor] = None,
                sse: Optional[torch.Tensor] = None) -> None:
    """Encode one LDLQ row block where it lies: the ``enc`` step of ldlq.py:136-143 without its copies.

    ``src`` is a ``(16, n_out)`` slice of the transposed matrix (rows = 16 consecutive input channels; any row
    stride, unit column stride), ``comp`` the feedback owed to it (same strides) or None.  The block
    ``src + comp`` is cut into ``n_out/16`` tiles (tile i = columns 16i..16i+15, t = (col % 16) * 16 + row),
    encoded, and written back in the same layout: ``wq`` the reconstruction, ``err = src - wq``.
    ``packed``: int32 view ``[n_out/16, 8K]`` whose rows may be strided (a column of the matrix's
    ``[n_out/16, k_in/16, 8K]`` code array).  All tensors on one CUDA device; nothing synchronises.
    """
    if src.dim() != 2 or src.shape[0] != 16 or src.shape[1] % 16:
        raise ValueError(f"expected a (16, n_out) block with n_out % 16 == 0, got {tuple(src.shape)}")
    if K not in (2, 3, 4):
        raise ValueError("K must be 2, 3 or 4")
    cid = codebook_id(codebook)
    if not src.is_cuda:
        raise ValueError("encode_rows works on CUDA tensors only")
    dev = src.device
    n_out = src.shape[1]
    ld = src.stride(0)
    for name, t in (("src", src), ("comp", comp), ("wq", wq), ("err", err)):
        if t is None:
            continue
        if t.dtype != torch.float32 or t.device != dev or tuple(t.shape) != (16, n_out) or t.stride(1) != 1 or t.stride(0) != ld:
            raise ValueError(f"{name} must be a float32 (16, {n_out}) block on {dev} with the strides of src")
    nw = T_SEQ * K // 32
    pstride = 0
    if packed is not None:
        if packed.dtype != torch.int32 or packed.device != dev or tuple(packed.shape) != (n_out // 16, nw) or packed.stride(1) != 1:
            raise ValueError(f"packed must be an int32 [{n_out // 16}, {nw}] view on {dev} with contiguous rows")
        pstride = packed.stride(0) if n_out > 16 else nw
    if sse is not None and (sse.dtype != torch.float32 or sse.device != dev or tuple(sse.shape) != (n_out // 16,) or not sse.is_contiguous()):
        raise ValueError("sse must be a contiguous float32 [n_out/16] tensor")
    if n_out == 0:
        return
    ws = _workspace(dev, n_out // 16, K)
    with torch.cuda.device(dev):
        rc = _lib.lib().tcq_encode_tb_rows(src.data_ptr(), comp.data_ptr() if comp is not None else None, ld, n_out, K, cid,
                                           packed.data_ptr() if packed is not None else None, pstride, wq.data_ptr(),
                                           err.data_ptr() if err is not None else None,
                                           sse.data_ptr() if sse is not None else None, ws.data_ptr(), ws.numel(), _stream(dev))
    _lib.check(rc, "tcq_encode_tb_rows")


_HOST_CHUNK = 2 * 3552          # tiles per pipelined chunk of a host-tensor encode (two workspace chunks)
_copy_streams: dict = {}


def _encode_host(w: torch.Tensor, K: int, cid: int, dev: torch.device, want_dq: bool, want_sse: bool, want_bits: bool,
                 out: Optional["Encoded"]) -> "Encoded":
    """Encode host tiles: chunks are copied in, encoded and copied out on three streams that overlap.

    The copy of chunk i+1 to the device and the copy of chunk i-1's results to the host run under the
    encode of chunk i, so the PCIe traffic costs one chunk of latency, not a pass over the data.
    Results land in pinned host tensors (``out`` if given, else freshly allocated); the call returns
    after the last copy has finished.
    """
    n = w.shape[0]
    nw = T_SEQ * K // 32
    wh = w.to(torch.float32).contiguous()
    if not wh.is_pinned():
        wh = wh.pin_memory()

    def host(shape, dtype, given):
        if given is not None:
            if tuple(given.shape) != tuple(shape) or given.dtype != dtype or given.is_cuda:
                raise ValueError("`out` tensors must be host tensors of the result's shape and dtype")
            return given
        return torch.empty(shape, dtype=dtype, pin_memory=True)

    h_packed = host((n, nw), torch.int32, out.packed if out else None)
    h_dq = host((n, T_SEQ), torch.float32, out.dq if out else None) if want_dq else None
    h_sse = host((n,), torch.float32, out.sse if out else None) if want_sse else None
    h_bits = host((n, T_SEQ), torch.int64, out.bits if out else None) if want_bits else None
    if n == 0:
        return Encoded(h_packed, h_dq, h_sse, h_bits)

    key = dev.index
    if key not in _copy_streams:
        _copy_streams[key] = (torch.cuda.Stream(dev), torch.cuda.Stream(dev))
    s_in, s_out = _copy_streams[key]
    main = torch.cuda.current_stream(dev)
    c = min(n, _HOST_CHUNK)
    d_w = [torch.empty((c, T_SEQ), dtype=torch.float32, device=dev) for _ in range(2)]
    d_packed = [torch.empty((c, nw), dtype=torch.int32, device=dev) for _ in range(2)]
    d_dq = [torch.empty((c, T_SEQ), dtype=torch.float32, device=dev) if want_dq else None for _ in range(2)]
    d_sse = [torch.empty((c,), dtype=torch.float32, device=dev) if want_sse else None for _ in range(2)]
    d_bits = [torch.empty((c, T_SEQ), dtype=torch.int64, device=dev) if want_bits else None for _ in range(2)]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_done = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]
    s_in.wait_stream(main)
    starts = list(range(0, n, c))
    for i, lo in enumerate(starts):
        b, m = i & 1, min(c, n - lo)
        with torch.cuda.stream(s_in):
            if i >= 2:
                s_in.wait_event(ev_done[b])            # the encode that read this input buffer has finished
            d_w[b][:m].copy_(wh[lo:lo + m], non_blocking=True)
            ev_in[b].record(s_in)
        main.wait_event(ev_in[b])
        if i >= 2:
            main.wait_event(ev_out[b])                 # this buffer's previous results are on the host
        _encode_device(d_w[b][:m], K, cid, d_packed[b][:m], d_dq[b][:m] if want_dq else None,
                       d_sse[b][:m] if want_sse else None, d_bits[b][:m] if want_bits else None)
        ev_done[b].record(main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_done[b])
            h_packed[lo:lo + m].copy_(d_packed[b][:m], non_blocking=True)
            if want_dq:
                h_dq[lo:lo + m].copy_(d_dq[b][:m], non_blocking=True)
            if want_sse:
                h_sse[lo:lo + m].copy_(d_sse[b][:m], non_blocking=True)
            if want_bits:
                h_bits[lo:lo + m].copy_(d_bits[b][:m], non_blocking=True)
            ev_out[b].record(s_out)
    for t in d_w + d_packed + d_dq + d_sse + d_bits:      # keep the staging buffers alive on the side streams
        if t is not None:
            t.record_stream(s_in)
            t.record_stream(s_out)
    s_out.synchronize()                                   # the caller reads host memory next
    return Encoded(h_packed, h_dq, h_sse, h_bits)


@torch.no_grad()
def encode(w: torch.Tensor, K: int, codebook: CodebookLike, *, want_dq: bool = True, want_sse: bool = True,
           want_bits: bool = False, out: Optional[Encoded] = None) -> Encoded:
    """Tail-biting trellis encode of ``w [n, 256]``.

    Device tensors: one C-ABI call, nothing synchronises, outputs on the same device.
    Host tensors: the tiles are streamed through the GPU in chunks (copy in, encode, copy out
    overlap) and the results come back as pinned host tensors; pass pinned tiles and preallocated
    pinned ``out`` tensors (an ``Encoded`` with the wanted fields) to avoid per-call pinning.
    """
    if w.dim() != 2 or w.shape[1] != T_SEQ:
        raise ValueError(f"expected tiles of shape [n, {T_SEQ}], got {tuple(w.shape)}")
    if K not in (2, 3, 4):
        raise ValueError("K must be 2, 3 or 4")
    cid = codebook_id(codebook)
    dev = _cuda_device(w)
    n = w.shape[0]
    if not w.is_cuda:
        return _encode_host(w, K, cid, dev, want_dq, want_sse, want_bits, out)
    if out is not None:
        raise ValueError("`out` is for host-tensor encodes; device results are allocated by the call")
    wd = _to_dev(w, dev, torch.float32)
    packed = torch.empty((n, T_SEQ * K // 32), dtype=torch.int32, device=dev)
    dq = torch.empty((n, T_SEQ), dtype=torch.float32, device=dev) if want_dq else None
    sse = torch.empty((n,), dtype=torch.float32, device=dev) if want_sse else None
    bits = torch.empty((n, T_SEQ), dtype=torch.int64, device=dev) if want_bits else None
    _encode_device(wd, K, cid, packed, dq, sse, bits)
    return Encoded(packed, dq, sse, bits)


@torch.no_grad()
def viterbi_tb_b200(w: torch.Tensor, K: int, lut: CodebookLike):
    """Drop-in for ``viterbi_tb(w, K, lut)`` / ``viterbi_tb_triton(w, K, lut)``.

    Returns ``(bits int64 [n,256], dq fp32 [n,256])`` exactly as qtip.py:124-144 does
    with the fp32 dynamic programme.
    """
    r = encode(w, K, lut, want_dq=True, want_sse=False, want_bits=True)
    return r.bits, r.dq


def viterbi_tb(w: torch.Tensor, K: int, lut: CodebookLike, dp_dtype=None):
    """Same signature as the reference's ``viterbi_tb``; ``dp_dtype`` must be None or fp32."""
    if dp_dtype not in (None, torch.float32):
        raise ValueError("the B200 encoder computes path metrics in fp32 only")
    return viterbi_tb_b200(w, K, lut)


@torch.no_grad()
def viterbi_pass_b200(w: torch.Tensor, K: int, overlap: Optional[torch.Tensor], lut: CodebookLike = "mcg",
                      roll: int = 0) -> torch.Tensor:
    """Drop-in for ``_viterbi_pass(w, K, lut, overlap)`` / ``viterbi_pass_triton(w, K, overlap)``.

    Returns the optimal state path int64 ``[n, 256]``.  ``roll=128`` runs on
    ``torch.roll(w, 128, dims=1)`` without materialising it.
    """
    if w.dim() != 2 or w.shape[1] != T_SEQ:
        raise ValueError(f"expected tiles of shape [n, {T_SEQ}], got {tuple(w.shape)}")
    cid = codebook_id(lut)
    dev = _cuda_device(w)
    n = w.shape[0]
    wd = _to_dev(w, dev, torch.float32)
    ov = _to_dev(overlap, dev, torch.int32) if overlap is not None else None
    if ov is not None and ov.shape != (n,):
        raise ValueError("overlap must have one entry per tile")
    states = torch.empty((n, T_SEQ), dtype=torch.int64, device=dev)
    if n:
        ws = _workspace(dev, n, K)
        with torch.cuda.device(dev):
            rc = _lib.lib().tcq_viterbi_pass(wd.data_ptr(), n, K, cid, ov.data_ptr() if ov is not None else None,
                                             roll, states.data_ptr(), ws.data_ptr(), ws.numel(), _stream(dev))
        _lib.check(rc, "tcq_viterbi_pass")
    return states if w.is_cuda else states.cpu()


# --------------------------------------------------------------------------- decode
@torch.no_grad()
def decode_packed(packed: torch.Tensor, K: int, codebook: CodebookLike) -> torch.Tensor:
    """Packed code words ``[n, 8K]`` (int32/uint32) -> reconstruction fp32 ``[n, 256]``."""
    if K not in (2, 3, 4):
        raise ValueError("K must be 2, 3 or 4")
    if packed.dim() != 2 or packed.shape[1] != T_SEQ * K // 32:
        raise ValueError(f"expected packed words of shape [n, {T_SEQ * K // 32}], got {tuple(packed.shape)}")
    cid = codebook_id(codebook)
    dev = _cuda_device(packed)
    if packed.dtype not in (torch.int32, torch.uint32):
        raise ValueError("packed words must be int32 or uint32")
    pd = _to_dev(packed.view(torch.int32), dev, torch.int32)
    n = pd.shape[0]
    dq = torch.empty((n, T_SEQ), dtype=torch.float32, device=dev)
    if n:
        with torch.cuda.device(dev):
            rc = _lib.lib().tcq_decode_packed(pd.data_ptr(), n, K, cid, dq.data_ptr(), _stream(dev))
        _lib.check(rc, "tcq_decode_packed")
    return dq if packed.is_cuda else dq.cpu()


@torch.no_grad()
def decode_matvec(packed: torch.Tensor, n_out: int, k_in: int, K: int, codebook: CodebookLike, x: torch.Tensor) -> torch.Tensor:
    """``x @ Zq.T`` straight from packed codes: ``x [k_in]`` or ``[m, k_in]`` -> ``[n_out]`` or ``[m, n_out]`` fp32.

    ``Zq`` is the ``[n_out, k_in]`` code matrix in the exporter's tile order (tile ``(row/16)*(k_in/16) + col/16``);
    it is decoded on the fly and never stored.  CUDA form of the reference's DECODE_MATMUL shader
    (web/kernels.js:105-128); the incoherence-processing fold stays with the caller (``shards.packed_linear``).
    """
    if K not in (2, 3, 4):
        raise ValueError("K must be 2, 3 or 4")
    if n_out % 16 or k_in % 16 or n_out < 0 or k_in < 0:
        raise ValueError(f"n_out={n_out} and k_in={k_in} must be non-negative multiples of 16")
    tiles = (n_out // 16) * (k_in // 16)
    if packed.dim() != 2 or tuple(packed.shape) != (tiles, T_SEQ * K // 32):
        raise ValueError(f"expected packed words of shape [{tiles}, {T_SEQ * K // 32}], got {tuple(packed.shape)}")
    if packed.dtype not in (torch.int32, torch.uint32):
        raise ValueError("packed words must be int32 or uint32")
    if x.dim() not in (1, 2) or x.shape[-1] != k_in:
        raise ValueError(f"x must be [{k_in}] or [m, {k_in}], got {tuple(x.shape)}")
    cid = codebook_id(codebook)
    dev = _cuda_device(packed if packed.is_cuda else (x if x.is_cuda else None))
    pd = _to_dev(packed.view(torch.int32), dev, torch.int32)
    xd = _to_dev(x.reshape(-1, k_in), dev, torch.float32)
    m = xd.shape[0]
    y = torch.empty((m, n_out), dtype=torch.float32, device=dev)
    if k_in == 0:
        y.zero_()
    elif m and n_out:
        with torch.cuda.device(dev):
            rc = _lib.lib().tcq_decode_matvec(pd.data_ptr(), n_out, k_in, K, cid, xd.data_ptr(), k_in, m, y.data_ptr(), n_out,
                                              _stream(dev))
        _lib.check(rc, "tcq_decode_matvec")
    y = y.reshape(*x.shape[:-1], n_out)
    return y if (packed.is_cuda or x.is_cuda) else y.cpu()


@torch.no_grad()
def decode_recursive(bits: torch.Tensor, K: int, lut: CodebookLike, s0: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``decode_recursive(bits, K, lut, s0)`` of qtip.py:70-79: symbols ``[n,T]`` -> values ``[n,T]``."""
    if bits.dim() != 2:
        raise ValueError("bits must be [n, T]")
    if K not in (2, 3, 4):
        raise ValueError("K must be 2, 3 or 4")
    cid = codebook_id(lut)
    dev = _cuda_device(bits)
    bd = _to_dev(bits, dev, torch.int64)
    sd = _to_dev(s0, dev, torch.int64) if s0 is not None else None
    n, T = bd.shape
    out = torch.empty((n, T), dtype=torch.float32, device=dev)
    if n and T:
        with torch.cuda.device(dev):
            rc = _lib.lib().tcq_decode_symbols(bd.data_ptr(), n, T, K, cid, sd.data_ptr() if sd is not None else None,
                                               out.data_ptr(), _stream(dev))
        _lib.check(rc, "tcq_decode_symbols")
    return out if bits.is_cuda else out.cpu()


# The reference keeps two formulations (a recursion and a window) and tests that they
# agree (tests/test_qtip.py:36-45); on the GPU both are the same window kernel.
decode_window = decode_recursive


@torch.no_grad()
def pack_bits(bits: torch.Tensor, K: int) -> torch.Tensor:
    """``pack_bits_np(bits, K)`` of the reference's exporter: symbols ``[n,256]`` -> int32 words ``[n, 8K]``."""
    if bits.dim() != 2 or bits.shape[1] != T_SEQ:
        raise ValueError(f"expected symbols of shape [n, {T_SEQ}]")
    if K not in (2, 3, 4):
        raise ValueError("K must be 2, 3 or 4")
    dev = _cuda_device(bits)
    bd = _to_dev(bits, dev, torch.int64)
    n = bd.shape[0]
    out = torch.empty((n, T_SEQ * K // 32), dtype=torch.int32, device=dev)
    if n:
        with torch.cuda.device(dev):
            rc = _lib.lib().tcq_pack_symbols(bd.data_ptr(), n, K, out.data_ptr(), _stream(dev))
        _lib.check(rc, "tcq_pack_symbols")
    return out if bits.is_cuda else out.cpu()


# --------------------------------------------------------------------------- incoherence processing
def _pow2_block(d: int, cap: int) -> int:
    """Largest power of two that divides d, at most `cap` (qtip.py:208-213)."""
    b = 1
    while b < cap and d % (2 * b) == 0:
        b *= 2
    return b


def _sylvester(n: int, device, dtype=torch.float32) -> torch.Tensor:
    """Orthonormal Sylvester-Hadamard matrix of order n (a power of two)."""
    h = torch.ones((1, 1), device=device, dtype=dtype)
    while h.shape[0] < n:
        h = torch.cat((torch.cat((h, h), dim=1), torch.cat((h, -h), dim=1)), dim=0)
    return h * (n ** -0.5)


def block_hadamard(x: torch.Tensor, dim: int, block: int = 128) -> torch.Tensor:
    """Block-diagonal orthonormal Hadamard along ``dim`` (qtip.py:216-223); its own inverse."""
    xt = x.movedim(dim, -1)
    d = xt.shape[-1]
    b = _pow2_block(d, block)
    y = xt.reshape(*xt.shape[:-1], d // b, b) @ _sylvester(b, x.device, x.dtype)
    return y.reshape(xt.shape).movedim(-1, dim)


class IPContext:
    """Incoherence processing around the codec, same recipe and seed use as qtip.py:226-268.

    sign flips on both axes (signs drawn from ``torch.Generator('cpu').manual_seed(seed)``,
    out axis first), per-output-channel RMS scaling + block-Hadamard over the out axis,
    per-input-channel RMS scaling + block-Hadamard over the in axis, then one global
    scale so that ``z`` has the codebook's RMS.  ``restore`` inverts every step.

    For a CUDA matrix (16-divisible shape, default block) the work is done by the library's
    kernels (``tcq_ip_forward`` / ``tcq_ip_restore``: fast Walsh-Hadamard transforms, output
    directly in the encoder's tile order); ``tiles`` is then the primary result and ``z`` is
    formed from it on first use, and ``scale`` is read back from the device on first use.
    Host tensors, odd shapes and other block sizes take the PyTorch restatement below.
    """

    def __init__(self, w: torch.Tensor, cb_rms: float, seed: int = 0, block: int = 128):
        gen = torch.Generator(device="cpu").manual_seed(seed)
        n, k = w.shape
        self.block = block
        self.shape = (n, k)
        self.sv = (torch.randint(0, 2, (n,), generator=gen).float() * 2 - 1).to(w.device)
        self.su = (torch.randint(0, 2, (k,), generator=gen).float() * 2 - 1).to(w.device)
        self._z = self._tiles = self._scale = self._scale_t = None
        self.on_device = bool(w.is_cuda and block == 128 and n % 16 == 0 and k % 16 == 0 and 0 < n <= 16 * 65535 and k > 0)
        if self.on_device:
            dev = w.device
            wd = w.to(torch.float32).contiguous()
            self._tiles = torch.empty((n // 16 * (k // 16), T_SEQ), dtype=torch.float32, device=dev)
            self.out_s = torch.empty(n, dtype=torch.float32, device=dev)
            self.in_s = torch.empty(k, dtype=torch.float32, device=dev)
            self._scale_t = torch.empty(1, dtype=torch.float32, device=dev)
            ws = self._ip_workspace(dev)
            with torch.cuda.device(dev):
                rc = _lib.lib().tcq_ip_forward(wd.data_ptr(), n, k, self.sv.data_ptr(), self.su.data_ptr(), float(cb_rms), 1,
                                               self._tiles.data_ptr(), self.out_s.data_ptr(), self.in_s.data_ptr(),
                                               self._scale_t.data_ptr(), ws.data_ptr(), ws.numel(), _stream(dev))
            _lib.check(rc, "tcq_ip_forward")
            return
        z = w * self.sv[:, None] * self.su[None, :]
        out_s = z.square().mean(dim=1).sqrt().clamp_min(1e-8)
        self.out_s = out_s / out_s.mean()
        z = block_hadamard(z / self.out_s[:, None], 0, block)
        in_s = z.square().mean(dim=0).sqrt().clamp_min(1e-8)
        self.in_s = in_s / in_s.mean()
        z = block_hadamard(z / self.in_s[None, :], 1, block)
        self._scale = z.square().mean().sqrt().item() / cb_rms
        self._z = z / self._scale

    def _ip_workspace(self, dev: torch.device) -> torch.Tensor:
        n, k = self.shape
        return torch.empty(int(_lib.lib().tcq_ip_workspace_bytes(n, k)), dtype=torch.uint8, device=dev)

    @property
    def scale(self) -> float:
        if self._scale is None:
            self._scale = float(self._scale_t.item())
        return self._scale

    @property
    def z(self) -> torch.Tensor:
        """The processed matrix ``[n, k]``."""
        if self._z is None:
            self._z = from_tiles(self._tiles, *self.shape).contiguous()
        return self._z

    @property
    def tiles(self) -> torch.Tensor:
        """The processed matrix as encoder tiles ``[n/16 * k/16, 256]`` (qtip.py:288)."""
        if self._tiles is None:
            self._tiles = to_tiles(self._z).contiguous()
        return self._tiles

    def _restore_device(self, zq: torch.Tensor, tiled: bool) -> torch.Tensor:
        n, k = self.shape
        dev = self.sv.device
        zd = zq.to(device=dev, dtype=torch.float32).contiguous()
        out = torch.empty((n, k), dtype=torch.float32, device=dev)
        ws = self._ip_workspace(dev)
        with torch.cuda.device(dev):
            rc = _lib.lib().tcq_ip_restore(zd.data_ptr(), int(tiled), n, k, self.sv.data_ptr(), self.su.data_ptr(),
                                           self.out_s.data_ptr(), self.in_s.data_ptr(), self._scale_t.data_ptr(),
                                           out.data_ptr(), ws.data_ptr(), ws.numel(), _stream(dev))
        _lib.check(rc, "tcq_ip_restore")
        return out

    def restore(self, zq: torch.Tensor) -> torch.Tensor:
        if self.on_device:
            if tuple(zq.shape) != self.shape:
                raise ValueError(f"expected a {self.shape} matrix, got {tuple(zq.shape)}")
            return self._restore_device(zq, tiled=False)
        y = block_hadamard(zq * self.scale, 1, self.block) * self.in_s[None, :]
        y = block_hadamard(y, 0, self.block) * self.out_s[:, None]
        return y * self.sv[:, None] * self.su[None, :]

    def restore_tiles(self, dq: torch.Tensor) -> torch.Tensor:
        """``restore`` of a reconstruction still in tile order ``[n/16 * k/16, 256]`` (skips the untiling copy)."""
        n, k = self.shape
        if tuple(dq.shape) != (n // 16 * (k // 16), T_SEQ):
            raise ValueError(f"expected [{n // 16 * (k // 16)}, {T_SEQ}] tiles, got {tuple(dq.shape)}")
        if self.on_device:
            return self._restore_device(dq, tiled=True)
        return self.restore(from_tiles(dq, n, k))


def to_tiles(z: torch.Tensor) -> torch.Tensor:
    """``[n, k]`` matrix -> ``[n/16 * k/16, 256]`` tiles of 16 out rows x 16 in columns (qtip.py:288)."""
    n, k = z.shape
    return z.reshape(n // 16, 16, k // 16, 16).permute(0, 2, 1, 3).reshape(-1, T_SEQ)


def from_tiles(tiles: torch.Tensor, n: int, k: int) -> torch.Tensor:
    """Inverse of ``to_tiles`` (qtip.py:303)."""
    return tiles.reshape(n // 16, k // 16, 16, 16).permute(0, 2, 1, 3).reshape(n, k)


# --------------------------------------------------------------------------- matrix quantizer
def _check_backend(backend: str) -> None:
    if backend not in ("auto", "b200"):
        raise ValueError(f"backend {backend!r} is not available here: this package has only the B200 CUDA encoder "
                         "(backend='b200' or 'auto')")


@torch.no_grad()
def tcq_quantize_weight(w: torch.Tensor, K: int, lut: CodebookLike, seed: int = 0, tile_batch: int = 16384,
                        dp_dtype=torch.float32, backend: str = "auto") -> torch.Tensor:
    """Fake-quantise one ``[n_out, n_in]`` matrix: incoherence processing + tail-biting TCQ.

    Same signature and result layout as qtip.py:272-304.  ``tile_batch`` is accepted for
    compatibility (the extension chunks internally); ``dp_dtype`` is ignored because the
    path metrics are always fp32 (the reference's bit-exact mode).
    """
    _check_backend(backend)
    n, k = w.shape
    if n % 16 or k % 16:
        raise ValueError(f"shape {tuple(w.shape)} not 16-divisible")
    dev = _cuda_device(w)
    wd = w.to(dev)
    lut_t = lut if isinstance(lut, torch.Tensor) else codebook_lut(CODEBOOK_NAMES[codebook_id(lut)], dev)
    cb_rms = lut_t.float().square().mean().sqrt().item()
    ip = IPContext(wd.float(), cb_rms, seed=seed)
    tiles = ip.tiles
    dq = encode(tiles, K, lut, want_dq=True, want_sse=False).dq
    return ip.restore_tiles(dq).to(dtype=w.dtype, device=w.device)
