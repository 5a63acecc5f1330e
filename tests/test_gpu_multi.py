"""Two-GPU run of the sharded operator: each rank computes its KV-head groups
with the CUDA path and the NCCL all-gather of the outputs equals the
single-GPU result.  Skipped when fewer than two GPUs are visible."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    import torch.distributed as dist
    import kernelfuser_b200 as kf
    from kernelfuser_b200.shard import gather_heads, head_shard, shard_inputs
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        xs = kf.make_inputs(2, 300, 8, 4, 128, seed=5)
        dx = [x.cuda() for x in xs]
        full = kf.optimized_attention(*dx, causal=True)
        sh = head_shard(8, 4, rank, world)
        qs, ks, vs = shard_inputs(dx[0], dx[1], dx[2], sh)
        local = kf.optimized_attention(qs, ks, vs, *dx[3:], causal=True)
        got = gather_heads(local)
        torch.cuda.synchronize()
        kf.check_status()
        ret[rank] = bool(torch.equal(got.view(torch.int16), full.view(torch.int16)))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_shard_and_gather():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = _free_port()
        procs = [ctx.Process(target=_worker, args=(r, 2, port, ret)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(300)
            assert p.exitcode == 0
        assert dict(ret) == {0: True, 1: True}
