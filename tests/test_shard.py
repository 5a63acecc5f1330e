"""CPU tests of head-group sharding, including a 2-rank gloo run: each rank
evaluates the oracle on its shard and the gathered result equals the
unsharded one."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from kernelfuser_b200.inputs import make_inputs
from kernelfuser_b200.shard import gather_heads, head_shard, shard_inputs
from oracle import oracle as orc


@pytest.mark.parametrize("hq,hkv", [(32, 8), (16, 8), (8, 8)])
@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_every_head_owned_exactly_once(hq, hkv, world):
    g = hq // hkv
    seen_q, seen_kv = [], []
    for r in range(world):
        sh = head_shard(hq, hkv, r, world)
        seen_q += list(range(sh.q_lo, sh.q_hi))
        seen_kv += list(range(sh.kv_lo, sh.kv_hi))
        # local GQA mapping equals the global one
        for hl in range(sh.n_q):
            assert (sh.q_lo + hl) // g == sh.kv_lo + hl // g
    assert seen_q == list(range(hq)) and seen_kv == list(range(hkv))


def test_bad_shard_specs_are_rejected():
    with pytest.raises(ValueError):
        head_shard(32, 8, 0, 3)
    with pytest.raises(ValueError):
        head_shard(32, 8, 2, 2)
    with pytest.raises(ValueError):
        head_shard(30, 8, 0, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        q, k, v, gq, gk, cos, sin = make_inputs(2, 70, 8, 4, 128, seed=11)
        sh = head_shard(8, 4, rank, world)
        qs, ks, vs = shard_inputs(q, k, v, sh)
        local = orc.oracle_fp32(qs, ks, vs, gq, gk, cos, sin, True)
        full = gather_heads(local)
        want = orc.oracle_fp32(q, k, v, gq, gk, cos, sin, True)
        ret[rank] = bool(torch.allclose(full, want, atol=1e-5)) and tuple(full.shape) == tuple(want.shape)
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_shard_and_gather():
    world = 2
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = _free_port()
        procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0
        assert dict(ret) == {0: True, 1: True}
