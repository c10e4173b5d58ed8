"""Batch-major sharding of the attention forward over the GPUs of one box.

Every (batch, head) pair of the reference's kernels is independent (src/hip_kernels.cpp:269-277
reads and writes only its own slices), so the path shards without any exchange inside the
kernels: rank r owns batches [b0, b1) (hipgpt_shard_range), which are contiguous slabs of
every [B*S, E] plane and of the output.  The only collective is the all-gather of the output
slabs afterwards, and only for callers that need the whole output on every rank.

One process per GPU; torch.distributed provides the plumbing (NCCL on GPUs, gloo on CPU for
the tests of this host logic).
"""
from __future__ import annotations

import ctypes as C
from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist

from . import _capi


def shard_range(B: int, world: int, rank: int) -> Tuple[int, int]:
    """Batches [b0, b1) owned by `rank`: contiguous, ordered, sizes differ by at most one."""
    b0, b1 = C.c_int(), C.c_int()
    _capi.check(_capi.lib().hipgpt_shard_range(B, world, rank, C.byref(b0), C.byref(b1)))
    return b0.value, b1.value


def local_planes(qkv: torch.Tensor, B: int, S: int, E: int, b0: int, b1: int) -> torch.Tensor:
    """This rank's slab of three stacked [B*S, E] planes, as a contiguous [3, (b1-b0)*S, E] tensor."""
    return qkv.view(3, B, S, E)[:, b0:b1].reshape(3, (b1 - b0) * S, E).contiguous()


def all_gather_output(out_local: torch.Tensor, B: int, S: int, E: int, group=None) -> torch.Tensor:
    """All ranks' output slabs, in batch order, as one [B*S, E] tensor on every rank.  Slabs of
    unequal size (B not divisible by the world size) are padded to the largest for the
    collective and trimmed afterwards."""
    world = dist.get_world_size(group)
    ranges = [shard_range(B, world, r) for r in range(world)]
    biggest = max(b1 - b0 for b0, b1 in ranges)
    rows = biggest * S
    send = out_local
    if out_local.shape[0] != rows:
        send = out_local.new_zeros((rows, E))
        send[: out_local.shape[0]] = out_local
    recv = out_local.new_empty((world, rows, E))
    dist.all_gather_into_tensor(recv.view(-1), send.reshape(-1), group=group)
    if all(b1 - b0 == biggest for b0, b1 in ranges):
        return recv.view(B * S, E)
    return torch.cat([recv[r, : (b1 - b0) * S] for r, (b0, b1) in enumerate(ranges)], dim=0)


def sharded_forward(qkv_local: torch.Tensor, B: int, S: int, E: int, H: int, *, causal: bool = False,
                    gather: bool = True, group=None,
                    compute: Optional[Callable[[torch.Tensor, int], torch.Tensor]] = None) -> torch.Tensor:
    """Attention forward of this rank's batches and, if `gather`, the all-gather of every rank's
    output.  qkv_local: [3, Bl*S, E] with Bl = this rank's number of batches.  `compute` maps
    (qkv_local, Bl) -> out_local [Bl*S, E]; it defaults to the CUDA kernels and exists so that
    the host logic can be exercised on CPU ranks."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    b0, b1 = shard_range(B, world, rank)
    Bl = b1 - b0
    if qkv_local.shape != (3, Bl * S, E):
        raise ValueError(f"rank {rank} owns batches [{b0},{b1}) and expects planes of shape {(3, Bl * S, E)}")
    if compute is None:
        from . import launchers
        out_local = torch.empty((Bl * S, E), dtype=torch.float32, device=qkv_local.device)
        if Bl > 0:
            launchers.launch_multihead_attention(qkv_local, out_local, None, Bl, S, E, H, causal=causal)
    else:
        out_local = compute(qkv_local, Bl)
    if not gather or world == 1:
        return out_local
    return all_gather_output(out_local, B, S, E, group)
