"""Multi-GPU sharding of the encoder: one process per GPU, no exchange during compute.

Tiles are independent (tail-biting closes every tile on itself) and so are weight
matrices, so the work shards without any data-path collective:

  * one large matrix  -> contiguous tile ranges, one per rank (``tile_range``);
  * a whole model     -> whole matrices per rank, longest-processing-time first
                         (``assign_matrices``); an LDLQ matrix never leaves its GPU.

The only collective is the gather of the packed code words after the compute
(``gather_packed``), over ``torch.distributed`` (NCCL on GPUs; gloo works too and
is what the CPU tests use).  The reference is single-process
(``scripts/run_tcq_eval.py:104-132`` loops over matrices serially); this module is
the multi-GPU form of that loop.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def tile_range(n_tiles: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous ``[lo, hi)`` slice of ``n_tiles`` for ``rank``; sizes differ by at most one."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("bad rank / world size")
    base, extra = divmod(n_tiles, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def matrix_cost(n_out: int, k_in: int, ldlq: bool, sms: int = 148, group: int = 3) -> float:
    """Relative encode time of one matrix, used to balance ranks.

    Plain: proportional to the tile count.  LDLQ: ``k_in/16`` strictly serial encoder
    calls of ``n_out/16`` tiles each, every call costing whole rounds of tile groups
    over the SMs.
    """
    if not ldlq:
        return float((n_out // 16) * (k_in // 16))
    per_call = n_out // 16
    rounds = -(-(-(-per_call // group)) // sms)
    return float((k_in // 16) * rounds * group * sms)


def assign_matrices(costs: Sequence[float], world: int) -> List[List[int]]:
    """Longest-processing-time-first assignment: returns the matrix indices of each rank.

    Deterministic (ties broken by index), so every rank computes the same plan
    without communication.
    """
    order = sorted(range(len(costs)), key=lambda i: (-costs[i], i))
    load = [0.0] * world
    plan: List[List[int]] = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda j: (load[j], j))
        plan[r].append(i)
        load[r] += costs[i]
    return plan


def gather_packed(local: torch.Tensor, n_total: int, group: Optional[dist.ProcessGroup] = None,
                  dst: Optional[int] = None) -> Optional[torch.Tensor]:
    """Gather the ranks' packed code words ``[n_local, words]`` (split by ``tile_range``) into ``[n_total, words]``.

    ``dst=None``: every rank gets the result (all-gather); otherwise only rank ``dst``
    does and the others return None.  Shards are padded to a common length so that a
    single fixed-size collective is used.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    words = local.shape[1]
    lo, hi = tile_range(n_total, rank, world)
    if local.shape[0] != hi - lo:
        raise ValueError(f"rank {rank} holds {local.shape[0]} tiles, expected {hi - lo}")
    longest = -(-n_total // world)
    send = local if local.shape[0] == longest else torch.cat(
        (local, local.new_zeros((longest - local.shape[0], words))), dim=0)
    send = send.contiguous()
    if dst is None:
        recv = local.new_empty((world * longest, words))
        dist.all_gather_into_tensor(recv, send, group=group)
    else:
        parts = [local.new_empty((longest, words)) for _ in range(world)] if rank == dst else None
        dist.gather(send, parts, dst=dst, group=group)
        if rank != dst:
            return None
        recv = torch.cat(parts, dim=0)
    out = local.new_empty((n_total, words))
    for r in range(world):
        a, b = tile_range(n_total, r, world)
        out[a:b] = recv[r * longest:r * longest + (b - a)]
    return out


def encode_sharded(tiles: torch.Tensor, K: int, codebook, group: Optional[dist.ProcessGroup] = None,
                   dst: Optional[int] = None, encoder: Optional[Callable] = None):
    """Encode this rank's slice of ``tiles [n, 256]`` and gather the packed codes.

    Every rank passes the same ``tiles`` shape (only its own slice is read).  Returns
    ``(packed_all or None, local Encoded, (lo, hi))``.  ``encoder`` defaults to the CUDA
    ``qtip.encode``.
    """
    if encoder is None:
        from .qtip import encode as encoder
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    lo, hi = tile_range(tiles.shape[0], rank, world)
    local = encoder(tiles[lo:hi], K, codebook)
    packed_all = gather_packed(local.packed, tiles.shape[0], group=group, dst=dst)
    return packed_all, local, (lo, hi)


def model_plan(shapes: Dict[str, Tuple[int, int]], ldlq_names: Sequence[str], world: int) -> List[List[str]]:
    """Matrix names per rank for a whole model (``shapes``: name -> (n_out, k_in))."""
    names = sorted(shapes)
    costs = [matrix_cost(*shapes[n], ldlq=n in set(ldlq_names)) for n in names]
    return [[names[i] for i in idx] for idx in assign_matrices(costs, world)]
