"""CPU tests of the multi-rank host logic: world_size-2 and -3 gloo groups, each rank computing its
N-slice of a GEMM with the oracle; the gathered result must equal the unsharded one."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from apnn_tc_b200 import shard


def test_shard_range_covers_without_overlap():
    for total, world, mult in [(8192, 8, 256), (1000, 3, 32), (64, 8, 128), (1024, 5, 1), (7, 2, 4)]:
        edges = [shard.shard_range(total, world, r, mult) for r in range(world)]
        assert edges[0][0] == 0 and edges[-1][1] == total
        for (a0, a1), (b0, b1) in zip(edges, edges[1:]):
            assert a1 == b0 and a0 <= a1
        assert all((a % mult == 0) for a, _ in edges if a < total)
    with pytest.raises(ValueError):
        shard.shard_range(10, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, M, N, K, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(5)                    # same operands on every rank
        W, _ = oracle.value_planes(rng, M, K, 1)
        X, _ = oracle.value_planes(rng, N, K, 2)
        n0, n1 = shard.shard_range(N, world, rank, 32)
        local = torch.from_numpy(oracle.gemm_popc(W, np.ascontiguousarray(X[:, n0:n1])))
        gathered = shard.allgather_columns(local)
        full = shard.assemble_columns(gathered)
        slowest = shard.max_over_ranks(float(rank + 1), torch.device("cpu"))
        if rank == 0:
            ret["ok"] = bool(np.array_equal(full.numpy(), oracle.gemm_popc(W, X))) and slowest == float(world)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_n_sharded_gemm_allgather_gloo(world):
    M, N, K = 24, 64 * world, 256
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), M, N, K, ret), nprocs=world, join=True)
    assert ret.get("ok") is True
