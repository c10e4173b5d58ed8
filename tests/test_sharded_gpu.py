"""The library's multi-GPU driver on two real GPUs: each rank computes its chunks of batches, the chunks are
all-gathered in place by NCCL while the next chunk computes (or stored into the peers' mapped buffers by the
library's own copy kernel), and every rank must end with exactly the bits of the unsharded call.  Skipped on a box with one GPU.  No rank leaves mid-step, nothing is made to fail."""
import os
import socket

import numpy as np
import pytest

from hipgpt_b200 import synth

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")
import torch.distributed as dist  # noqa: E402
import torch.multiprocessing as mp  # noqa: E402


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from hipgpt_b200 import launchers, sharding
        sh = sharding.ShardedAttention()
        ok = True
        for (B, H, S, D, chunks, dtype) in [(8, 4, 256, 32, 2, torch.float32), (4, 2, 300, 64, 1, torch.float32),
                                            (8, 2, 512, 64, 4, torch.bfloat16), (16, 8, 1024, 64, 4, torch.float32)]:
            E = H * D
            for causal in (True, False):
                qkv = torch.from_numpy(synth.qkv_planes(77 + S, B, S, E)).view(3, B * S, E).cuda().to(dtype)
                whole = torch.full((B * S, E), float("nan"), device="cuda", dtype=dtype)
                if dtype == torch.float32:
                    launchers.launch_multihead_attention(qkv, whole, None, B, S, E, H, causal=causal)
                else:
                    launchers.mha_forward_bf16(qkv, whole, B, S, E, H, causal=causal)
                loc = sharding.local_planes_chunked(qkv, B, S, E, world, rank, chunks)
                out = torch.full((B * S, E), float("nan"), device="cuda", dtype=dtype)
                sh.forward(loc[0], loc[1], loc[2], out, B, S, E, H, causal=causal, chunks=chunks, gather=True)
                torch.cuda.synchronize()
                ok = ok and bool(torch.equal(out, whole))
                # the library's own transport: stores into the peers' mapped buffers instead of the collective's kernels
                pout = sh.output_tensor(B * S, E, dtype)
                pout.fill_(float("nan"))
                torch.cuda.synchronize()
                dist.barrier()                       # every rank's buffer is filled before any peer writes into it
                for mode in (sharding.GATHER_PEER_STORES, sharding.GATHER_PEER_STORES, sharding.GATHER_PEER_COPIES, sharding.GATHER_PEER_COPIES,
                             sharding.GATHER_PEER_BOTH):
                    # each twice: the second call writes over a buffer the peers have just read
                    sh.forward(loc[0], loc[1], loc[2], pout, B, S, E, H, causal=causal, chunks=chunks, gather=mode)
                    torch.cuda.synchronize()
                    ok = ok and bool(torch.equal(pout, whole))
                    pout.fill_(float("nan"))
                    torch.cuda.synchronize()
                    dist.barrier()
                # without the gather only this rank's batches are written
                out2 = torch.full((B * S, E), float("nan"), device="cuda", dtype=dtype)
                sh.forward(loc[0], loc[1], loc[2], out2, B, S, E, H, causal=causal, chunks=chunks, gather=False)
                torch.cuda.synchronize()
                mine = torch.zeros(B, dtype=torch.bool)
                for c in range(chunks):
                    b0, b1 = sharding.chunk_range(B, world, rank, chunks, c)
                    mine[b0:b1] = True
                o3 = out2.view(B, S * E).float().cpu()
                ok = ok and bool(torch.equal(o3[mine], whole.view(B, S * E).float().cpu()[mine])) and bool(torch.isnan(o3[~mine]).all())
        sh.close()
        ret[rank] = ok
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_forward_with_nccl_gather_equals_unsharded():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert [ret.get(r) for r in range(world)] == [True] * world
