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
import sys
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


# ---- the library's own multi-GPU driver (hipgpt_mha_forward_sharded in include/hipgpt_attn.h) -------------------
def chunk_range(B: int, world: int, rank: int, chunks: int, chunk: int) -> Tuple[int, int]:
    """Global batches [b0, b1) that `rank` owns in chunk `chunk` (B a multiple of world * chunks)."""
    b0, b1 = C.c_int(), C.c_int()
    _capi.check(_capi.lib().hipgpt_shard_chunk_range(B, world, rank, chunks, chunk, C.byref(b0), C.byref(b1)))
    return b0.value, b1.value


def local_planes_chunked(qkv: torch.Tensor, B: int, S: int, E: int, world: int, rank: int, chunks: int) -> torch.Tensor:
    """This rank's batches of three stacked [B*S, E] planes in the order the driver wants them: chunk after chunk."""
    view = qkv.view(3, B, S, E)
    parts = [view[:, slice(*chunk_range(B, world, rank, chunks, c))] for c in range(chunks)]
    return torch.cat(parts, dim=1).reshape(3, (B // world) * S, E).contiguous()


GATHER_NONE, GATHER_NCCL, GATHER_PEER_STORES, GATHER_PEER_COPIES, GATHER_PEER_BOTH = 0, 1, 2, 3, 4


class ShardedAttention:
    """One per process (= per GPU): an NCCL communicator of the library's own, a high-priority communication stream
    and the per-chunk events.  torch.distributed only carries the 128-byte id from rank 0 to the other ranks."""

    def __init__(self, group=None):
        lib = _capi.lib()
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        ident = (C.c_char * 128)()
        if self.world > 1:
            if self.rank == 0:
                _capi.check(lib.hipgpt_shard_unique_id(ident))
            box = [bytes(ident)]
            dist.broadcast_object_list(box, src=0, group=group)
            ident = (C.c_char * 128).from_buffer_copy(box[0])
        self._h = C.c_void_p()
        _capi.check(lib.hipgpt_shard_create(C.byref(self._h), ident, self.rank, self.world))

    def output_tensor(self, rows: int, cols: int, dtype: torch.dtype) -> torch.Tensor:
        """Collective.  A [rows, cols] tensor in memory that the library allocated on every rank and mapped into every
        other rank (hipgpt_shard_output_buffer): the `out` that forward(..., gather=GATHER_PEER_STORES) needs.  One per
        object; asking again releases the previous one (collectively)."""
        nbytes = rows * cols * torch.empty((), dtype=dtype).element_size()
        ptr = C.c_void_p()
        _capi.check(_capi.lib().hipgpt_shard_output_buffer(self._h, C.c_size_t(nbytes), C.byref(ptr)))
        typestr = {torch.float32: "<f4", torch.bfloat16: "<u2", torch.float16: "<f2"}[dtype]

        class _Raw:                                # the CUDA array interface: torch wraps the memory without copying it
            __cuda_array_interface__ = {"shape": (rows, cols), "typestr": typestr, "data": (ptr.value, False), "version": 3, "strides": None}

        t = torch.as_tensor(_Raw(), device=torch.device("cuda", torch.cuda.current_device()))
        return t.view(dtype) if t.dtype != dtype else t

    def forward(self, q, k, v, out, B: int, S: int, E: int, H: int, *, causal: bool = False, chunks: int = 1, gather=True):
        """q, k, v: this rank's batches (local_planes_chunked order), fp32 or bf16 CUDA tensors (or raw addresses with
        elem_bytes given by `out`'s dtype); out: the whole [B*S, E] output.  Asynchronous on torch's current stream.
        gather: False / True (NCCL all-gather per chunk) / GATHER_PEER_STORES (the library's own copy kernel into the
        peers' buffers; `out` must come from output_tensor)."""
        esz = out.element_size()
        ptr = lambda t: t if isinstance(t, int) else t.data_ptr()
        _capi.check(_capi.lib().hipgpt_mha_forward_sharded(self._h, ptr(q), ptr(k), ptr(v), out.data_ptr(), B, S, E, H, int(causal),
                                                           esz, chunks, int(gather), torch.cuda.current_stream().cuda_stream))

    def close(self):
        if self._h:
            _capi.lib().hipgpt_shard_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        if sys is None or sys.is_finalizing():                    # releasing the mapped buffers is a collective: not at interpreter exit
            return
        try:
            self.close()
        except Exception:
            pass
