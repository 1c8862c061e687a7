"""Sequence-parallel path across real GPUs: one process per GPU, NCCL point-to-point for the state
chain.  Skipped on boxes with a single GPU (the single-GPU tests emulate the ranks instead)."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import PKG_DIR, ROOT

pytestmark = pytest.mark.gpu


def _inputs(K, V):
    from oracle import delta_oracle as O
    B, L, Hk, Hv = 1, 2048, 2, 4
    q, k, v, g, b, w = O.make_inputs(123, B, L, Hk, Hv, K, V, qkv_scale=0.5)
    seg = torch.repeat_interleave(torch.tensor([0, 1, 2], dtype=torch.int32), torch.tensor([700, 324, 1024]))[None]
    gen = torch.Generator().manual_seed(9)
    return (q, k, v, g, b, w), seg, torch.randn(B, L, Hv, V, generator=gen), torch.randn(B, Hv, K, V, generator=gen) * 0.1


def _worker(rank, world, port, ret):
    for p in (ROOT, PKG_DIR):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from deltanet_b200 import sp
    ins, seg, do, dfs = _inputs(128, 128)
    L = ins[0].shape[1]
    lo, hi = rank * L // world, (rank + 1) * L // world
    shard = [t[:, lo:hi].contiguous().cuda().requires_grad_() for t in ins]
    out, final = sp.chunk_gdn2_sp(*shard, segment_ids=seg[:, lo:hi].contiguous().cuda(), chunk_size=128,
                                  precision="bf16", qk_l2norm=True)
    loss = (out.float() * do[:, lo:hi].cuda()).sum()
    if rank == world - 1:
        loss = loss + (final * dfs.cuda()).sum()
    grads = torch.autograd.grad(loss, shard)
    torch.cuda.synchronize()
    ret[rank] = dict(out=out.detach().cpu(), final=final.detach().cpu(), grads=[x.cpu() for x in grads])
    dist.barrier()
    dist.destroy_process_group()


def test_sp_over_nccl_matches_single_gpu():
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    import deltanet_b200 as dn
    from oracle import delta_oracle as O
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    ins, seg, do, dfs = _inputs(128, 128)
    leaves = [t.cuda().requires_grad_() for t in ins]
    o1, f1 = dn.chunk_gdn2(*leaves, segment_ids=seg.cuda(), output_final_state=True, chunk_size=128,
                           precision="bf16", qk_l2norm=True)
    g1 = torch.autograd.grad((o1.float() * do.cuda()).sum() + (f1 * dfs.cuda()).sum(), leaves)
    out = torch.cat([ret[r]["out"] for r in range(world)], 1)
    assert O.rel_l2(out, o1.detach().cpu()) < 2e-2
    assert O.rel_l2(ret[world - 1]["final"], f1.detach().cpu()) < 2e-2
    for i in range(6):
        assert O.rel_l2(torch.cat([ret[r]["grads"][i] for r in range(world)], 1), g1[i].cpu()) < 2e-2, i
