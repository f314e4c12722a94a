"""World-size-2 gloo checks of the sharding logic used by the N-sharded GEMM and the batch-sharded
bmm: each rank computes its shard with the CPU oracle, the gathered result must equal the
unsharded product. CPU only."""
import os
import sys

import numpy as np
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    import torch
    from beantensor_b200 import _lib, sharding, synth
    from oracle import oracle as O
    from tests.helpers import store
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # N-sharded GEMM: all of A, a column block of B, all-gather of C column blocks.
        M, N, K = 48, 64, 40
        A = store(synth.normal((M, K), K ** -0.5, 4, 0), _lib.BF16)
        B = store(synth.normal((K, N), K ** -0.5, 4, 1), _lib.BF16)
        c0, c1 = sharding.column_block(N, rank, world)
        C_loc = O.gemm(_lib.BF16, A, np.ascontiguousarray(B[:, c0:c1]))
        parts = [torch.zeros((M, N // world), dtype=torch.float64) for _ in range(world)]
        dist.all_gather(parts, torch.from_numpy(C_loc))
        C = np.concatenate([p.numpy() for p in parts], axis=1)
        ok_gemm = np.array_equal(C, O.gemm(_lib.BF16, A, B))
        # the fused epilogue's destination order covers every rank exactly once, local first
        order = sharding.peer_order(rank, world)
        ok_order = order[0] == rank and sorted(order) == list(range(world))
        # batch-sharded bmm: no collective on the data path; gather only to compare
        Bn = 5
        A3 = store(synth.normal((Bn, 8, 16), 0.25, 3, 0), _lib.F16)
        B3 = store(synth.normal((Bn, 16, 24), 0.25, 3, 1), _lib.F16)
        lo, hi = sharding.batch_slice(Bn, rank, world)
        mine = O.bmm(_lib.F16, A3[lo:hi], B3[lo:hi]) if hi > lo else np.zeros((0, 8, 24))
        gathered = [None] * world
        dist.all_gather_object(gathered, (lo, hi, mine))
        full = np.concatenate([g[2] for g in sorted(gathered, key=lambda g: g[0])], axis=0)
        ok_bmm = np.array_equal(full, O.bmm(_lib.F16, A3, B3))
        q.put((rank, bool(ok_gemm), bool(ok_order), bool(ok_bmm)))
    finally:
        dist.destroy_process_group()


def test_sharding_world2():
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r[0] for r in results) == [0, 1]
    assert all(r[1] and r[2] and r[3] for r in results), results


def test_partition_rules():
    from beantensor_b200 import sharding
    assert [sharding.batch_slice(64, r, 8) for r in (0, 7)] == [(0, 8), (56, 64)]
    assert [sharding.batch_slice(5, r, 4) for r in range(4)] == [(0, 2), (2, 4), (4, 5), (5, 5)]
    assert sharding.column_block(16384, 3, 8) == (6144, 8192)
    import pytest
    with pytest.raises(ValueError):
        sharding.column_block(100, 0, 8)
