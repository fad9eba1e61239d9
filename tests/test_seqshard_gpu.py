"""Sequence sharding over real GPUs (NCCL), one process per GPU.  Needs at
least two devices; skipped on a single-GPU machine (the same protocol runs on
CPU ranks in test_seqshard_gloo.py and, serially on one device, in
test_tensor_path_gpu.py::test_sequence_shards_on_one_gpu)."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, dtype_name, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port), NCCL_NVLS_ENABLE='0')
    torch.cuda.set_device(rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=torch.device('cuda', rank))
    try:
        from fly_b200.seqshard import sblocal_forward_seqshard, shard_bounds
        from oracle import sblocal_oracle as so
        dtype = getattr(torch, dtype_name)
        B, N, H, E, w, r = 1, 2000, 2, 64, 256, 128
        g = torch.Generator().manual_seed(99)
        q, k, v = ((torch.randn(B, N, H, E, generator=g) / E ** 0.25).to(dtype) for _ in range(3))
        torch.manual_seed(99)
        W = so.gaussian_orthogonal_random_matrix(r, E)
        bounds = shard_bounds(N, world)
        lo, hi = bounds[rank], bounds[rank + 1]
        dev = torch.device('cuda', rank)
        out = sblocal_forward_seqshard(q[:, lo:hi].to(dev), k[:, lo:hi].to(dev), v[:, lo:hi].to(dev), W.to(dev), w, N)
        torch.cuda.synchronize()
        ref, _ = so.sblocal_forward(q.float(), k.float(), v.float(), W, w)
        ret[rank] = so.rel_err(out.float().cpu(), ref[:, lo:hi])
        # the same with the shard's K/V written in place into caller-owned halo-extended buffers
        from fly_b200.seqshard import HaloBuffers
        hb = HaloBuffers(B, N, H, E, E, w, dtype, dev)
        hb.k_local.copy_(k[:, lo:hi])
        hb.v_local.copy_(v[:, lo:hi])
        out2 = sblocal_forward_seqshard(q[:, lo:hi].to(dev), hb.k_local, hb.v_local, W.to(dev), w, N, halo_buffers=hb)
        torch.cuda.synchronize()
        ret[rank] = max(ret[rank], so.rel_err(out2.float().cpu(), ref[:, lo:hi]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize('dtype_name,tol', [('float32', 1e-4), ('bfloat16', 2e-2)])
def test_two_gpus_match_single_sequence(dtype_name, tol, sbl_lib):
    if torch.cuda.device_count() < 2:
        pytest.skip('needs two GPUs')
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        port = s.getsockname()[1]
    ret = mp.get_context('spawn').Manager().dict()
    mp.spawn(_worker, args=(2, port, dtype_name, ret), nprocs=2, join=True)
    for rank in range(2):
        assert ret[rank] <= tol, f'rank {rank}: rel err {ret[rank]}'
