#!/usr/bin/env python
"""Generate the golden vectors in this folder by RUNNING THE REFERENCE ITSELF.

Usage (needs a checkout of Azimml/trellis-everywhere; CPU only, about a minute):

    python tests/golden/make_golden.py /path/to/trellis-everywhere

The script imports ``trellis.qtip`` / ``trellis.ldlq`` from ``<checkout>/src`` and
executes the reference's ``pack_bits_np`` straight out of
``<checkout>/scripts/export_packed_8b.py`` (that script cannot be imported on a CPU
box because it moves tensors to CUDA at import time, so only that one function
definition is compiled from the file's syntax tree).  Nothing of the reference is
copied here: the outputs are data.

Files written (all small, committed):
  codebooks.npz   sha256 of the three 65 536-entry fp32 tables + every 251st entry
  encode.npz      torch.manual_seed(0) Gaussian tiles: per codebook x K the pass-1
                  state path, overlap, pass-2 state path, symbols and reconstruction (6 tiles),
                  and the symbols + a digest of the reconstruction for the first 64 tiles
  cfg2_probe.npz  16 tiles spread over the second benchmark configuration's matrix (4096 x 4096,
                  CPU generator seed 0, outliers, IPContext(seed=0)) as the reference's own
                  IPContext produced them, with the reference's symbols (3INST, K=3)
  encode_ip.npz   tiles of an outlier-heavy matrix after incoherence processing
                  (3INST, K=3), the second benchmark configuration in miniature
  decode.npz      decode_recursive / decode_window on random symbols (with and
                  without a start state), pack_bits_np words, wrapped decode
  quant.npz       tcq_quantize_weight (incoherence processing + plain TCQ, fp32 DP) on a small matrix
  ldlq.npz        teacher-forced LDLQ: the compensated row blocks the reference's
                  ``enc`` closure received and the reconstructions it returned
  shard.npz       one packed-model shard written by the reference's own ``Shard`` / ``put_quant``
                  (compiled from the exporter's syntax tree like ``pack_bits_np``): the .bin bytes,
                  the .bin.json text and the inputs that went in.  ``... <checkout> shard`` makes only this file.
"""
from __future__ import annotations

import ast
import hashlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _load_pack_bits_np(ref_root: str):
    path = os.path.join(ref_root, "scripts", "export_packed_8b.py")
    tree = ast.parse(open(path).read(), filename=path)
    fn = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "pack_bits_np")
    ns = {"np": np}
    exec(compile(ast.Module(body=[fn], type_ignores=[]), path, "exec"), ns)
    return ns["pack_bits_np"]


def _load_shard_writer(ref_root: str):
    """The reference's Shard class and put_quant function, compiled alone from the exporter's syntax tree."""
    import json
    from trellis.qtip import _fit_block
    path = os.path.join(ref_root, "scripts", "export_packed_8b.py")
    tree = ast.parse(open(path).read(), filename=path)
    want = [n for n in tree.body if (isinstance(n, ast.ClassDef) and n.name == "Shard")
            or (isinstance(n, ast.FunctionDef) and n.name == "put_quant")]
    ns = {"np": np, "os": os, "json": json, "_fit_block": _fit_block, "print": lambda *a, **k: None}
    exec(compile(ast.Module(body=want, type_ignores=[]), path, "exec"), ns)
    return ns["Shard"], ns["put_quant"]


def make_shard(ref_root: str) -> None:
    import tempfile
    import zlib
    from trellis.qtip import IPContext, T_SEQ, codebook_lut, viterbi_tb
    Shard, put_quant = _load_shard_writer(ref_root)
    pack_bits_np = _load_pack_bits_np(ref_root)
    lut = codebook_lut("mcg")
    torch.manual_seed(5)
    n, k, K = 32, 64, 3
    w = torch.randn(n, k) * 0.02
    ip = IPContext(w, lut.square().mean().sqrt().item(), seed=zlib.crc32(b"x"))
    tiles = ip.z.view(n // 16, 16, k // 16, 16).permute(0, 2, 1, 3).reshape(-1, T_SEQ)
    bits, dq = viterbi_tb(tiles.contiguous(), K, lut, dp_dtype=torch.float32)
    packed = pack_bits_np(bits.numpy().astype(np.int64), K)
    w_hat = ip.restore(dq.view(n // 16, k // 16, 16, 16).permute(0, 2, 1, 3).reshape(n, k))
    norm = torch.rand(k) + 0.5
    name = "model.layers.0.self_attn.q_proj.weight"
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "layer_00.bin")
        sh = Shard(path)
        put_quant(sh, name, packed, ip, n, k, K)
        sh.put("model.layers.0.input_layernorm.weight", norm.numpy(), np.float16)
        sh.flush()
        blob = np.fromfile(path, dtype=np.uint8)
        index = open(path + ".json").read()
    np.savez_compressed(os.path.join(HERE, "shard.npz"), w=w.numpy(), packed=packed, su=ip.su.numpy(), sv=ip.sv.numpy(),
                        in_s=ip.in_s.numpy(), out_s=ip.out_s.numpy(), scale=np.float64(ip.scale), norm=norm.numpy(),
                        w_hat=w_hat.numpy(), bin=blob, index=np.frombuffer(index.encode(), dtype=np.uint8),
                        name=np.frombuffer(name.encode(), dtype=np.uint8), K=np.int64(K))


def main(ref_root: str, only: str = "") -> None:
    sys.path.insert(0, os.path.join(ref_root, "src"))
    if only == "shard":
        make_shard(ref_root)
        return
    import trellis.ldlq as ldlq_mod
    from trellis.qtip import (IPContext, T_SEQ, _viterbi_pass, codebook_lut, decode_recursive,
                              decode_window, viterbi_tb)

    pack_bits_np = _load_pack_bits_np(ref_root)
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    names = ("1mad", "3inst", "mcg")
    luts = {n: codebook_lut(n) for n in names}

    # ---- codebooks -----------------------------------------------------------------
    cb = {}
    for n in names:
        a = luts[n].numpy()
        cb[f"{n}_sha256"] = np.frombuffer(hashlib.sha256(a.tobytes()).digest(), dtype=np.uint8)
        cb[f"{n}_sample"] = a[::251].copy()
    np.savez_compressed(os.path.join(HERE, "codebooks.npz"), **cb)

    # ---- encoder: Gaussian tiles ---------------------------------------------------
    torch.manual_seed(0)
    w_all = torch.randn(256, T_SEQ)          # the first benchmark configuration's generator
    n_tiles = 6
    w = w_all[:n_tiles].contiguous()
    enc = {"w": w.numpy()}
    for n in names:
        for K in (2, 3, 4):
            lut = luts[n]
            s1 = _viterbi_pass(torch.roll(w, T_SEQ // 2, dims=1), K, lut, None, None)
            ov = s1[:, T_SEQ // 2] >> K
            s2 = _viterbi_pass(w, K, lut, ov, None)
            bits, dq = viterbi_tb(w, K, lut)
            assert torch.equal(bits, s2 & ((1 << K) - 1))
            key = f"{n}_K{K}"
            enc[key + "_states1"] = s1.numpy().astype(np.uint16)
            enc[key + "_overlap"] = ov.numpy().astype(np.int32)
            enc[key + "_states2"] = s2.numpy().astype(np.uint16)
            enc[key + "_bits"] = bits.numpy().astype(np.uint8)
            enc[key + "_dq"] = dq.numpy()
            print(key, "mse", float(((w - dq) ** 2).mean()))
    # the same generator's first 64 tiles: symbols in full, reconstruction as a digest (it follows from the symbols)
    w64 = w_all[:64].contiguous()
    enc["w64"] = w64.numpy()
    for n in names:
        for K in (2, 3, 4):
            bits, dq = viterbi_tb(w64, K, luts[n])
            key = f"{n}_K{K}"
            assert np.array_equal(bits[:n_tiles].numpy().astype(np.uint8), enc[key + "_bits"])
            enc[key + "_bits64"] = bits.numpy().astype(np.uint8)
            enc[key + "_dq64_sha256"] = np.frombuffer(hashlib.sha256(dq.numpy().tobytes()).digest(), dtype=np.uint8)
            print(key, "64 tiles: sha256(bits)[:16]", hashlib.sha256(bits.numpy().astype(np.uint8).tobytes()).hexdigest()[:16],
                  "mse", float(((w64 - dq) ** 2).mean()))
    np.savez_compressed(os.path.join(HERE, "encode.npz"), **enc)

    # ---- the second benchmark configuration itself: 16 tiles spread over its 65 536 ----
    g = torch.Generator().manual_seed(0)
    m2 = torch.randn(4096, 4096, generator=g) * 0.02
    mask2 = torch.rand(4096, 4096, generator=g) < 0.01
    m2 = torch.where(mask2, m2 * 20, m2)
    lut = luts["3inst"]
    ip2 = IPContext(m2, lut.square().mean().sqrt().item(), seed=0)
    tiles2 = ip2.z.view(256, 16, 256, 16).permute(0, 2, 1, 3).reshape(-1, T_SEQ)
    idx2 = torch.tensor([min(i * 4369, 65535) for i in range(16)])
    sel2 = tiles2[idx2].contiguous()
    bits2, dq2 = viterbi_tb(sel2, 3, lut)
    np.savez_compressed(os.path.join(HERE, "cfg2_probe.npz"), index=idx2.numpy(), tiles=sel2.numpy(),
                        bits=bits2.numpy().astype(np.uint8), dq=dq2.numpy(),
                        z_rms=np.float64(ip2.z.square().mean().sqrt().item()), scale=np.float64(ip2.scale))

    # ---- encoder: incoherence-processed outlier matrix (3INST, K=3) ----------------
    g = torch.Generator().manual_seed(0)
    m = torch.randn(256, 512, generator=g) * 0.02
    mask = torch.rand(256, 512, generator=g) < 0.01
    m = torch.where(mask, m * 20, m)
    lut = luts["3inst"]
    ip = IPContext(m, lut.square().mean().sqrt().item(), seed=0)
    tiles = ip.z.view(16, 16, 32, 16).permute(0, 2, 1, 3).reshape(-1, T_SEQ)
    sel = tiles[torch.arange(0, tiles.shape[0], 64)].contiguous()    # 8 tiles, fed as DATA to both sides
    bits, dq = viterbi_tb(sel, 3, lut)
    np.savez_compressed(os.path.join(HERE, "encode_ip.npz"), w=sel.numpy(),
                        bits=bits.numpy().astype(np.uint8), dq=dq.numpy())

    # ---- decode + packing ------------------------------------------------------------
    dec = {}
    torch.manual_seed(0)
    for K in (2, 3, 4):
        b = torch.randint(0, 1 << K, (8, 64))
        s0 = torch.randint(0, 1 << 16, (8,))
        dec[f"K{K}_bits"] = b.numpy().astype(np.uint8)
        dec[f"K{K}_s0"] = s0.numpy().astype(np.int64)
        for n in names:
            dec[f"{n}_K{K}_recursive"] = decode_recursive(b, K, luts[n]).numpy()
            dec[f"{n}_K{K}_window"] = decode_window(b, K, luts[n]).numpy()
            dec[f"{n}_K{K}_recursive_s0"] = decode_recursive(b, K, luts[n], s0).numpy()
            dec[f"{n}_K{K}_window_s0"] = decode_window(b, K, luts[n], s0).numpy()
        tb = enc[f"mcg_K{K}_bits"].astype(np.int64)
        dec[f"K{K}_packed"] = pack_bits_np(tb, K)
    np.savez_compressed(os.path.join(HERE, "decode.npz"), **dec)

    # ---- matrix quantizer end to end (plain) ----
    from trellis.qtip import tcq_quantize_weight
    torch.manual_seed(4)
    wq_in = torch.randn(128, 256) * 0.02
    qd = {"w": wq_in.numpy()}
    for K in (2, 3, 4):
        qd[f"mcg_K{K}_w_hat"] = tcq_quantize_weight(wq_in, K=K, lut=luts["mcg"], seed=0, tile_batch=256,
                                                    dp_dtype=torch.float32, backend="torch").numpy()
    np.savez_compressed(os.path.join(HERE, "quant.npz"), **qd)

    # ---- LDLQ, teacher forced ----------------------------------------------------------
    torch.manual_seed(1)
    lut = luts["mcg"]
    wm = torch.randn(64, 256) * 0.02
    A = torch.randn(256, 256)
    H = (A.T @ A) / 256 + torch.eye(256)
    calls = []
    orig = ldlq_mod.viterbi_tb

    def spy(t, K, lut_, dp_dtype=None):
        bits_, dq_ = orig(t, K, lut_, dp_dtype=dp_dtype)
        calls.append((t.clone(), bits_.clone(), dq_.clone()))
        return bits_, dq_

    ldlq_mod.viterbi_tb = spy
    try:
        what = ldlq_mod.tcq_quantize_weight_ldlq(wm, K=3, lut=lut, H=H, seed=0, dp_dtype=torch.float32,
                                                 backend="torch")
    finally:
        ldlq_mod.viterbi_tb = orig
    keep = [0, 5, 15]                        # first, middle and last of the 16 enc calls
    np.savez_compressed(
        os.path.join(HERE, "ldlq.npz"),
        tiles=np.stack([calls[i][0].numpy() for i in keep]),
        bits=np.stack([calls[i][1].numpy().astype(np.uint8) for i in keep]),
        dq=np.stack([calls[i][2].numpy() for i in keep]),
        n_calls=np.int64(len(calls)),
        w=wm.numpy(), H=H.numpy().astype(np.float32), w_hat=what.numpy(),
    )
    make_shard(ref_root)
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    if len(sys.argv) not in (2, 3):
        sys.exit(__doc__)
    main(*sys.argv[1:])
