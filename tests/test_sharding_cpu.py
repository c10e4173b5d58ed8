"""The multi-GPU host logic on CPU: two and three gloo ranks shard a batch, each computes its
slab (the CPU oracle stands in for the kernels here), the outputs are all-gathered, and every
rank must hold exactly the bits of the unsharded computation."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from hipgpt_b200 import sharding, synth


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, B, S, E, H, causal, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import bindings as ob
        qkv = torch.from_numpy(synth.qkv_planes(31, B, S, E))
        b0, b1 = sharding.shard_range(B, world, rank)
        local = sharding.local_planes(qkv, B, S, E, b0, b1)

        def compute(planes, Bl):
            if Bl == 0:
                return torch.empty((0, E))
            out, _ = ob.mha(planes.numpy(), Bl, S, E, H, causal=causal)
            return torch.from_numpy(out)

        full = sharding.sharded_forward(local, B, S, E, H, causal=causal, gather=True, compute=compute)
        ref, _ = ob.mha(qkv.numpy(), B, S, E, H, causal=causal)
        ret[rank] = bool(np.array_equal(full.numpy(), ref)) and full.shape == (B * S, E)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,B", [(2, 4), (2, 5), (3, 2), (2, 1)])
def test_sharded_forward_equals_unsharded(world, B):
    S, H, D = 24, 2, 32
    E = H * D
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), B, S, E, H, True, ret), nprocs=world, join=True)
    assert [ret.get(r) for r in range(world)] == [True] * world


def test_shard_range_matches_c_abi_contract():
    assert sharding.shard_range(64, 8, 3) == (24, 32)
    assert sharding.shard_range(10, 4, 0) == (0, 3) and sharding.shard_range(10, 4, 3) == (8, 10)
    assert sharding.shard_range(2, 4, 3) == (2, 2)          # more ranks than batches: empty shard


def test_local_planes_are_contiguous_slabs():
    B, S, E = 4, 3, 8
    qkv = torch.arange(3 * B * S * E, dtype=torch.float32).view(3, B * S, E)
    loc = sharding.local_planes(qkv, B, S, E, 1, 3)
    assert loc.shape == (3, 2 * S, E) and loc.is_contiguous()
    assert torch.equal(loc[1], qkv[1, S:3 * S])


@pytest.mark.parametrize("B,world,chunks", [(64, 8, 4), (32, 2, 16), (8, 2, 2), (6, 3, 1), (4, 4, 1)])
def test_chunk_ranges_tile_the_batches_in_gather_order(B, world, chunks):
    """Chunk c of the output must be one contiguous block holding the ranks' parts in rank order: that is what lets
    ncclAllGather work in place (sendbuff = recvbuff + rank * count)."""
    k = B // (world * chunks)
    seen = []
    for c in range(chunks):
        for r in range(world):
            b0, b1 = sharding.chunk_range(B, world, r, chunks, c)
            assert b1 - b0 == k and b0 == c * world * k + r * k
            seen += list(range(b0, b1))
    assert seen == list(range(B))
    qkv = torch.arange(3 * B * 2 * 4, dtype=torch.float32).view(3, B * 2, 4)
    for r in range(world):
        loc = sharding.local_planes_chunked(qkv, B, 2, 4, world, r, chunks)
        want = torch.cat([qkv.view(3, B, 2, 4)[:, slice(*sharding.chunk_range(B, world, r, chunks, c))] for c in range(chunks)], dim=1)
        assert torch.equal(loc, want.reshape(3, -1, 4))


def test_chunk_range_refuses_uneven_splits():
    from hipgpt_b200 import _capi
    with pytest.raises(_capi.HipGPTError, match="not a multiple"):
        sharding.chunk_range(10, 4, 0, 1, 0)
    with pytest.raises(_capi.HipGPTError):
        sharding.chunk_range(8, 2, 0, 2, 2)
