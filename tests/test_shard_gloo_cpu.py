"""world_size-2 gloo run of the multi-GPU host logic on CPU: shard-invariant data through the
amax all-reduce, and the optional gather of O."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cutlass_flash_atten_fp8_b200 import synth
from cutlass_flash_atten_fp8_b200.shard import gather_output, shard_range


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, n_slices, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        w = synth.Workload("t", 1, n_slices, 128, 64, True, outliers=True, seed=5)
        lo, hi = shard_range(w.n_slices, world, rank)
        q, k, v, d = synth.make_qkv(w, "cpu", lo, hi)
        full = synth.make_qkv(w, "cpu")           # every rank can afford the whole thing here
        assert torch.equal(q.view(torch.uint8), full[0][lo:hi].view(torch.uint8))
        assert torch.equal(v.view(torch.uint8), full[2][lo:hi].view(torch.uint8))
        assert d == full[3]
        o_local = (q.float() * 0 + torch.arange(lo, hi).view(-1, 1, 1)).half()
        got = gather_output(o_local, w.n_slices, dst=0)
        if rank == 0:
            want = torch.arange(w.n_slices).view(-1, 1, 1).expand(-1, 128, 64).half()
            assert torch.equal(got, want)
        else:
            assert got is None
        ret[rank] = True
    finally:
        dist.destroy_process_group()


def _run(n_slices):
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(2, port, n_slices, ret), nprocs=2, join=True)
        assert ret.get(0) and ret.get(1)


def test_two_ranks_even_split():
    _run(4)


def test_two_ranks_uneven_split():
    _run(5)


def _subgroup_worker(rank, world, port, n_slices, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        grp = dist.new_group([1, 2])              # every rank takes part in creating it
        if rank in (1, 2):
            g_rank, g_world = dist.get_rank(grp), dist.get_world_size(grp)
            lo, hi = shard_range(n_slices, g_world, g_rank)
            o_local = (torch.zeros(hi - lo, 4, 8) + torch.arange(lo, hi).view(-1, 1, 1)).half()
            got = gather_output(o_local, n_slices, dst=0, group=grp)     # group rank 0 = global rank 1
            if rank == 1:
                assert torch.equal(got, torch.arange(n_slices).view(-1, 1, 1).expand(-1, 4, 8).half())
            else:
                assert got is None
        ret[rank] = True
    finally:
        dist.destroy_process_group()


def test_gather_inside_a_sub_group_uses_global_ranks():
    # even (4 slices over 2 ranks: gather) and uneven (5: send / irecv) splits inside group {1, 2} of 3 ranks
    for n_slices in (4, 5):
        port = _free_port()
        with mp.Manager() as mgr:
            ret = mgr.dict()
            mp.spawn(_subgroup_worker, args=(3, port, n_slices, ret), nprocs=3, join=True)
            assert all(ret.get(r) for r in range(3))
