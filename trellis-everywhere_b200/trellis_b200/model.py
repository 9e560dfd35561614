"""Model-level encode: every linear of a transformer-shaped model through the B200 codec, sharded by matrix.

The multi-GPU form of the reference's per-matrix loops (``scripts/run_tcq_eval.py:104-132`` ``apply_tcq``,
``scripts/export_packed_8b.py:193-219``): incoherence processing, then plain tail-biting TCQ or LDLQ
(MLP matrices only, as ``--ldlq-mlp-only`` does), with the reference's per-matrix seed ``crc32(name)``.

One process per GPU.  Whole matrices are assigned to ranks longest-processing-time first
(``dist.model_plan``), an LDLQ recursion never leaves its GPU, and nothing is exchanged until the end,
when the packed code words are gathered over ``torch.distributed``.  Each finished matrix appends one
JSON line to a per-rank log (tiles, seconds, weights/s, error) and, with ``out_dir``, writes its packed
words to ``<name>.bits.npy`` so that an interrupted run resumes by skipping finished matrices, the way
the reference's exporter skips finished shards (``export_packed_8b.py:81,195-196``).

Real checkpoints and calibration activations are not needed here: ``synthetic_weight`` /
``synthetic_hessian`` generate stand-ins with the reference configurations' shapes and distributions.
"""
from __future__ import annotations

import argparse
import json
import os
import threading
import time
import zlib
from typing import Callable, Dict, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.distributed as dist

from . import dist as tdist
from . import ldlq as tldlq
from . import qtip
from . import shards


_linalg_lock = threading.Lock()


def qwen3_8b_shapes(layers: int = 36, hidden: int = 4096, inter: int = 12288, q_heads: int = 32, kv_heads: int = 8,
                    head_dim: int = 128, embeddings: bool = False, vocab: int = 151936) -> Dict[str, Tuple[int, int]]:
    """``name -> (n_out, k_in)`` of the linears ``apply_tcq`` walks in a Qwen3-8B-shaped model (252 matrices).

    ``embeddings`` adds the two ``[vocab, hidden]`` matrices that the reference's exporter also packs
    (``export_packed_8b.py:221-253``) and that ``apply_tcq`` skips because they are not ``nn.Linear``.
    """
    shapes = {}
    if embeddings:
        shapes["model.embed_tokens"] = (vocab, hidden)
        shapes["lm_head"] = (vocab, hidden)
    for i in range(layers):
        p = f"model.layers.{i}."
        shapes[p + "self_attn.q_proj"] = (q_heads * head_dim, hidden)
        shapes[p + "self_attn.k_proj"] = (kv_heads * head_dim, hidden)
        shapes[p + "self_attn.v_proj"] = (kv_heads * head_dim, hidden)
        shapes[p + "self_attn.o_proj"] = (hidden, q_heads * head_dim)
        shapes[p + "mlp.gate_proj"] = (inter, hidden)
        shapes[p + "mlp.up_proj"] = (inter, hidden)
        shapes[p + "mlp.down_proj"] = (hidden, inter)
    return shapes


def is_mlp(name: str) -> bool:
    return ".mlp." in name


def seed_of(name: str) -> int:
    return zlib.crc32(name.encode())


def synthetic_weight(name: str, shape: Tuple[int, int], device) -> torch.Tensor:
    """Random-init weights N(0, 0.02^2), reproducible per matrix name."""
    g = torch.Generator(device=device).manual_seed(seed_of(name))
    return torch.randn(shape, generator=g, device=device) * 0.02


def synthetic_hessian(name: str, k: int, device, rows: int = 8192) -> torch.Tensor:
    """H = X^T X / rows for Gaussian activations with per-channel scales log-uniform in [0.1, 10]."""
    g = torch.Generator(device=device).manual_seed(seed_of(name) ^ 0x5EED)
    scales = torch.exp(torch.empty(k, device=device).uniform_(float(np.log(0.1)), float(np.log(10.0)), generator=g))
    H = torch.zeros(k, k, device=device)
    step = 2048
    for r0 in range(0, rows, step):
        x = torch.randn(min(step, rows - r0), k, generator=g, device=device) * scales
        H.addmm_(x.t(), x)
    return H / rows


@torch.no_grad()
def encode_matrix(w: torch.Tensor, K: int, codebook, seed: int, H: Optional[torch.Tensor] = None,
                  sigma_reg: float = 0.025, row_groups: int = 1, return_ip: bool = False):
    """One matrix: returns (packed int32 [n_tiles, 8K] in the reference's tile order, W_hat, relative error).

    Plain: tiles ordered ``(row/16) * (k/16) + col/16`` (qtip.py:288).  LDLQ: the same order, assembled from the
    per-row-block encoder calls as the reference's exporter does (export_packed_8b.py:114-131); ``row_groups`` > 1
    runs that many slices of output channels side by side (``ldlq.ldlq_row_groups``), for a matrix encoded alone.
    """
    n, k = w.shape
    dev = w.device
    lut = qtip.codebook_lut(qtip.CODEBOOK_NAMES[qtip.codebook_id(codebook)], dev)
    ip = qtip.IPContext(w.float(), lut.square().mean().sqrt().item(), seed=seed)
    nw = qtip.T_SEQ * K // 32
    if H is None:
        r = qtip.encode(ip.tiles, K, codebook, want_dq=True, want_sse=False)
        packed, w_hat = r.packed, ip.restore_tiles(r.dq)
    else:
        Ht = tldlq._transform_H(H.float(), ip.su, block=qtip._pow2_block(k, 128))
        with _linalg_lock:                 # torch's lazily initialised linalg backends must not be entered by two threads at once
            Lm = tldlq.block_ldl(tldlq.regularize_H(Ht, sigma_reg), b=16)
        if Lm is None:
            Lm = torch.zeros(k, k, device=dev)
        store = torch.empty((n // 16, k // 16, nw), dtype=torch.int32, device=dev)
        # every 16-row block's encoder call writes its code words straight into its column of `store`
        zq = tldlq.ldlq_row_groups(ip.z.t().contiguous(), Lm, None, row_groups,
                                   fused=lambda part, a, b: tldlq.ldlq_b200(part, Lm, K, codebook, packed=store[a // 16:b // 16])
                                   ).t().contiguous()
        packed = store.reshape(-1, nw)
        w_hat = ip.restore(zq)
    rel = float(((w - w_hat) ** 2).mean() / w.square().mean())
    if return_ip:                          # the sign and scale vectors a shard needs next to the packed words
        return packed, w_hat, rel, ip
    return packed, w_hat, rel


def encode_model(shapes: Dict[str, Tuple[int, int]], K: int = 3, codebook="mcg", ldlq_filter: Callable[[str], bool] = is_mlp,
                 weight_fn: Callable = synthetic_weight, hessian_fn: Optional[Callable] = synthetic_hessian,
                 out_dir: Optional[str] = None, device=None, group=None, gather: bool = True,
                 log: Optional[Callable[[dict], None]] = None, streams: int = 1, shard_dir: Optional[str] = None,
                 seed_fn: Callable[[str], int] = seed_of):
    """Encode this rank's share of the model; returns (results of this rank, gathered packed words on rank 0).

    With ``gather=False`` the second value is this rank's own ``name -> packed words`` instead, and no collective runs.

    ``seed_fn(name)`` gives the incoherence-processing seed of a matrix.  The default, ``crc32(name)``, is what the
    reference's model-level quantiser uses (``scripts/run_tcq_eval.py:115``); its packed exporter uses one seed for
    every matrix, ``crc32(b"x")`` (``scripts/export_packed_8b.py:91,108``): pass ``lambda name: zlib.crc32(b"x")``
    to reproduce that script's shards.

    ``results``: name -> {"tiles", "seconds", "weights_per_s", "rel_err", "ldlq", "skipped"}.
    ``streams`` > 1 keeps that many matrices in flight on this GPU (one host thread + CUDA stream each).
    ``shard_dir``: every finished matrix is also written as a packed-model shard ``<name>.bin`` + ``.bin.json`` in the
    reference exporter's format (``shards.Shard``); ``shards.merge_manifest(shard_dir)`` then builds ``manifest.json``.
    Works without an initialised process group (single process = rank 0 of 1).
    """
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
    ldlq_names = [n for n in shapes if hessian_fn is not None and ldlq_filter(n)]
    mine = tdist.model_plan(shapes, ldlq_names, world)[rank]
    results, packed_out = {}, {}
    if out_dir:
        os.makedirs(out_dir, exist_ok=True)
    if shard_dir:
        os.makedirs(shard_dir, exist_ok=True)

    cb_name = qtip.CODEBOOK_NAMES[qtip.codebook_id(codebook)]

    def finished_earlier(name: str, path: Optional[str]):
        """Packed words of ``name`` left by an earlier run with the SAME settings, else None (then it is encoded again).

        A matrix counts as finished only if its words have this run's shape, its side-car names this run's K, codebook,
        seed and LDLQ choice, and (with ``shard_dir``) its shard is there too; anything else is stale."""
        if not path or not os.path.exists(path) or not os.path.exists(path + ".json"):
            return None
        n_out, k_in = shapes[name]
        try:
            meta = json.load(open(path + ".json"))
            arr = np.load(path)
        except Exception:
            return None
        want = {"K": K, "codebook": cb_name, "shape": [n_out, k_in], "seed": int(seed_fn(name)), "ldlq": name in ldlq_names}
        if meta != want or arr.dtype != np.int32 or arr.shape != ((n_out // 16) * (k_in // 16), qtip.T_SEQ * K // 32):
            return None
        if shard_dir and not shards.shard_done(os.path.join(shard_dir, name + ".bin")):
            return None
        return arr

    def one(name: str, stream) -> None:
        n_out, k_in = shapes[name]
        path = os.path.join(out_dir, name + ".bits.npy") if out_dir else None
        old = finished_earlier(name, path)
        if old is not None:                                     # resume: finished in an earlier run
            packed_out[name] = torch.from_numpy(old).to(dev)
            results[name] = {"tiles": packed_out[name].shape[0], "skipped": True}
            return
        use_ldlq = name in ldlq_names
        w = weight_fn(name, (n_out, k_in), dev)
        H = hessian_fn(name, k_in, dev) if use_ldlq else None
        stream.synchronize()
        t0 = time.perf_counter()
        packed, _, rel, ip = encode_matrix(w, K, codebook, seed_fn(name), H, return_ip=True)
        # synchronises, and raises if a bounded in-kernel wait gave up or a weight was not finite: such codes
        # must not reach a shard or the gather
        qtip.workspace_status(n_out // 16 if use_ldlq else (n_out // 16) * (k_in // 16), K, dev)
        dt = time.perf_counter() - t0
        if shard_dir:
            sh = shards.Shard(os.path.join(shard_dir, name + ".bin"))
            sh.put_quant(name + ".weight", packed, ip, n_out, k_in, K)
            sh.flush()
        rec = {"name": name, "rank": rank, "gpu": dev.index, "tiles": packed.shape[0], "seconds": dt,
               "weights_per_s": n_out * k_in / dt, "rel_err": rel, "ldlq": use_ldlq, "skipped": False}
        results[name] = rec
        packed_out[name] = packed
        if path:
            tmp = path + ".tmp.npy"
            np.save(tmp, packed.cpu().numpy())
            os.replace(tmp, path)
            with open(path + ".json.tmp", "w") as f:            # written last: its presence marks the matrix as finished
                json.dump({"K": K, "codebook": cb_name, "shape": [n_out, k_in], "seed": int(seed_fn(name)), "ldlq": use_ldlq}, f)
            os.replace(path + ".json.tmp", path + ".json")
        if log:
            log(rec)

    if streams <= 1:
        for name in mine:
            one(name, torch.cuda.current_stream(dev))
    else:
        # Several matrices in flight, one host thread and one CUDA stream each.  An LDLQ recursion is a serial
        # chain of encoder calls of n_out/16 tiles, which rarely fill the last round of SMs; kernels of another
        # matrix's chain take the idle SMs.  Results do not depend on the interleaving: every matrix has its own
        # stream, scratch and seed.  "seconds" of a matrix then overlaps with its neighbours'.
        todo = list(mine)
        lock = threading.Lock()
        errors = []
        caller = torch.cuda.current_stream(dev)

        def worker() -> None:
            with torch.cuda.device(dev):
                s = torch.cuda.Stream(dev)
                s.wait_stream(caller)
                with torch.cuda.stream(s):
                    while True:
                        with lock:
                            if not todo or errors:
                                break
                            name = todo.pop(0)
                        try:
                            one(name, s)
                        except BaseException as e:      # surfaced by the caller below
                            with lock:
                                errors.append(e)
                            break
                s.synchronize()
                qtip.release_workspace(dev, s)          # the stream dies with this thread; so does its scratch

        threads = [threading.Thread(target=worker, name=f"encode-stream-{i}") for i in range(min(streams, max(1, len(todo))))]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        if errors:
            raise errors[0]
    if not gather:
        return results, packed_out          # this rank's own matrices; ``gather_model_codes`` can collect them later
    return results, gather_model_codes(shapes, ldlq_names, packed_out, K, world, rank, dev, group)


def gather_model_codes(shapes, ldlq_names: Sequence[str], packed_out: Dict[str, torch.Tensor], K: int, world: int,
                       rank: int, dev, group=None):
    """The one collective of the path: every rank's packed words to rank 0 (name -> int32 [tiles, 8K]).

    Each rank sends its matrices' words concatenated in sorted-name order, padded to the longest rank; the
    assignment is a deterministic function of ``shapes``, so rank 0 replays it to cut the buffers apart.
    """
    if world == 1:
        return dict(packed_out)
    nw = qtip.T_SEQ * K // 32
    owners = [sorted(names) for names in tdist.model_plan(shapes, ldlq_names, world)]
    tiles_of = lambda n: (shapes[n][0] // 16) * (shapes[n][1] // 16)
    longest = max(sum(tiles_of(n) for n in names) for names in owners)
    send = torch.zeros((longest, nw), dtype=torch.int32, device=dev)
    off = 0
    for n in owners[rank]:
        send[off:off + tiles_of(n)] = packed_out[n].reshape(-1, nw)
        off += tiles_of(n)
    parts = [torch.empty_like(send) for _ in range(world)] if rank == 0 else None
    dist.gather(send, parts, dst=0, group=group)
    if rank != 0:
        return None
    out = {}
    for r in range(world):
        off = 0
        for n in owners[r]:
            out[n] = parts[r][off:off + tiles_of(n)]
            off += tiles_of(n)
    return out


def main(argv=None) -> None:
    """``[torchrun --nproc-per-node N] python -m trellis_b200.model``: encode a Qwen3-8B-shaped random-init model."""
    ap = argparse.ArgumentParser(description=main.__doc__)
    ap.add_argument("--layers", type=int, default=36)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--inter", type=int, default=12288)
    ap.add_argument("--K", type=int, default=3)
    ap.add_argument("--codebook", default="mcg")
    ap.add_argument("--with-embeddings", action="store_true", help="also encode embed_tokens and lm_head ([151936, hidden])")
    ap.add_argument("--no-ldlq", action="store_true", help="plain TCQ everywhere (the reference's Hessian-free mode)")
    ap.add_argument("--hessian-rows", type=int, default=8192)
    ap.add_argument("--streams", type=int, default=3, help="matrices in flight per GPU (1 = one after another)")
    ap.add_argument("--shards", default=None, help="folder for packed-model shards in the reference exporter's format")
    ap.add_argument("--out", default=None, help="folder for <name>.bits.npy files and per-rank JSONL logs (enables resume)")
    args = ap.parse_args(argv)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    rank = dist.get_rank() if world > 1 else 0
    shapes = qwen3_8b_shapes(args.layers, args.hidden, args.inter, q_heads=args.hidden // 128, kv_heads=max(1, args.hidden // 512),
                             embeddings=args.with_embeddings)
    logf = open(os.path.join(args.out, f"rank{rank}.jsonl"), "a") if args.out and (os.makedirs(args.out, exist_ok=True) or True) else None

    def log(rec):
        line = json.dumps(rec)
        print(line, flush=True)
        if logf:
            logf.write(line + "\n")
            logf.flush()

    hess = None if args.no_ldlq else (lambda name, k, d: synthetic_hessian(name, k, d, rows=args.hessian_rows))
    torch.cuda.synchronize(dev)
    t0 = time.perf_counter()
    results, gathered = encode_model(shapes, args.K, args.codebook, hessian_fn=hess, out_dir=args.out, device=dev, log=log,
                                     streams=args.streams, shard_dir=args.shards)
    torch.cuda.synchronize(dev)
    if world > 1:
        dist.barrier()
    dt = time.perf_counter() - t0
    if rank == 0:
        total = sum(a * b for a, b in shapes.values())
        print(json.dumps({"summary": True, "matrices": len(shapes), "weights": total, "seconds": dt, "weights_per_s": total / dt,
                          "world": world, "streams": args.streams, "gathered_matrices": len(gathered) if gathered is not None else 0}), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
