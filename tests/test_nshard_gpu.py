"""N-sharded matmul with the all-gather fused into the epilogue (btm_gemm_nshard).

On one GPU the ranks are emulated one after the other: every "rank" owns a full copy of C on the
same device and stores its column block into all copies. With two or more GPUs the same call runs
as real ranks in child processes over peer-mapped memory (plain peer stores, NVLS off)."""
import ctypes as C
import os
import sys

import numpy as np
import pytest

from beantensor_b200 import _lib, sharding
from tests.helpers import TOL, gemm_inputs, to_gpu, to_host_bits, torch_dtype

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("dtype", [_lib.F16, _lib.BF16])
@pytest.mark.parametrize("world,shape", [(2, (256, 512, 128)), (4, (300, 1024, 200)), (8, (128, 2048, 64)), (3, (130, 24 * 3, 72)),
                                         (2, (100, 40, 64)), (2, (200, 2 * 136, 96))])
def test_emulated_ranks_on_one_gpu(btm, oracle, dtype, world, shape):
    import torch
    M, N, K = shape
    A, B = gemm_inputs(dtype, M, N, K, 21)
    a, b = to_gpu(A, dtype), to_gpu(B, dtype)
    copies = [torch.full((M, N), float("nan"), dtype=torch_dtype(dtype), device="cuda") for _ in range(world)]
    table = (C.c_void_p * world)(*[c.data_ptr() for c in copies])
    L = _lib.lib()
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for r in range(world):
        c0, c1 = sharding.column_block(N, r, world)
        if (c1 - c0) % 8 == 0:
            b_loc, ldb = b[:, c0:c1].contiguous(), c1 - c0
        else:  # a ragged block width: B stays a strided view so that rank 0 still takes the TMA path
            b_loc, ldb = b[:, c0:c1], N
        rc = L.btm_gemm_nshard(0, st, dtype, M, c1 - c0, K, a.data_ptr(), K, b_loc.data_ptr(), ldb, table, N, r, world)
        assert rc == _lib.OK, _lib.last_error()
    btm.check_device_status(0)
    ref = oracle.gemm(dtype, A, B)
    for c in copies:
        assert oracle.rel_frobenius(to_host_bits(c, dtype), dtype, ref) <= TOL[dtype]
    for c in copies[1:]:
        assert torch.equal(c, copies[0])


def test_bad_rank_arguments(btm):
    L = _lib.lib()
    p = C.c_void_p(256)
    table = (C.c_void_p * 2)(256, 512)
    assert L.btm_gemm_nshard(0, None, _lib.F16, 8, 8, 8, p, 8, p, 8, table, 16, 2, 2) == _lib.ERR_INVALID
    assert L.btm_gemm_nshard(0, None, _lib.F16, 8, 8, 8, p, 8, p, 8, table, 8, 0, 2) == _lib.ERR_INVALID  # ldc < nranks*Nloc
    assert L.btm_gemm_nshard(0, None, _lib.F32, 8, 8, 8, p, 8, p, 8, table, 16, 0, 2) == _lib.ERR_UNSUPPORTED


def _rank_main(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "NCCL_NVLS_ENABLE": "0"})
    import torch
    import torch.distributed as dist
    from beantensor_b200 import ops
    from beantensor_b200.errors import raise_for_status
    from oracle import oracle as O
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        ops.init(rank)
        L = _lib.lib()
        dtype = _lib.BF16
        M, N, K = 384, 256 * world, 320
        A, B = gemm_inputs(dtype, M, N, K, 33)
        c0, c1 = sharding.column_block(N, rank, world)
        a = to_gpu(A, dtype)
        b_loc = to_gpu(np.ascontiguousarray(B[:, c0:c1]), dtype)
        ptr, handle = C.c_void_p(), C.create_string_buffer(64)
        raise_for_status(L.btm_ipc_alloc(rank, M * N * 2, C.byref(ptr), handle))
        handles = [None] * world
        dist.all_gather_object(handles, handle.raw)
        peers = []
        for r in range(world):
            if r == rank:
                peers.append(ptr.value)
            else:
                p = C.c_void_p()
                raise_for_status(L.btm_ipc_open(rank, handles[r], C.byref(p)))
                peers.append(p.value)
        table = (C.c_void_p * world)(*peers)
        st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        raise_for_status(L.btm_gemm_nshard(rank, st, dtype, M, c1 - c0, K, a.data_ptr(), K, b_loc.data_ptr(), c1 - c0, table, N, rank, world))
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        ops.check_device_status(rank)

        class Raw:
            __cuda_array_interface__ = {"shape": (M, N), "typestr": "<i2", "data": (ptr.value, False), "version": 2}

        got = torch.as_tensor(Raw(), device="cuda").cpu().numpy().view(np.uint16)
        err = O.rel_frobenius(got, dtype, O.gemm(dtype, A, B))
        dist.barrier()
        for r in range(world):
            if r != rank:
                L.btm_ipc_close(rank, C.c_void_p(peers[r]))
        dist.barrier()
        L.btm_ipc_free(rank, ptr)
        q.put((rank, float(err)))
    finally:
        dist.destroy_process_group()


def test_real_ranks_over_peer_memory(oracle):
    import torch
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    import socket
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, err in results:
        assert err <= TOL[_lib.BF16], (rank, err)


def _rank_main_multicast(rank, world, port, q):
    # The same product with the output in NVSwitch multicast memory: one multimem store per tile reaches every rank.
    # No rank leaves while memory is bound: results travel through the queue only after release().
    sys.path.insert(0, ROOT)
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
    import torch
    import torch.distributed as dist
    from beantensor_b200 import multicast, ops
    from oracle import oracle as O
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    result = (rank, "error", "did not finish")
    try:
        ops.init(rank)
        L = _lib.lib()
        dtype = _lib.BF16
        M, N, K = 384, 256 * world, 320
        A, B = gemm_inputs(dtype, M, N, K, 35)
        c0, c1 = sharding.column_block(N, rank, world)
        a = to_gpu(A, dtype)
        b_loc = to_gpu(np.ascontiguousarray(B[:, c0:c1]), dtype)
        try:
            buf = multicast.MulticastBuffer(dist, rank, rank, world, M * N * 2)
        except NotImplementedError as e:
            result = (rank, "unsupported", str(e))
            buf = None
        if buf is not None:
            err, rc = float("inf"), _lib.OK
            try:
                class Raw:
                    __cuda_array_interface__ = {"shape": (M, N), "typestr": "<i2", "data": (buf.local_ptr, False), "version": 2}

                c_local = torch.as_tensor(Raw(), device="cuda")
                c_local.fill_(-1)
                torch.cuda.synchronize()
                dist.barrier()
                st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
                rc = L.btm_gemm_nshard_mc(rank, st, dtype, M, c1 - c0, K, a.data_ptr(), K, b_loc.data_ptr(), c1 - c0,
                                          buf.local_ptr, buf.mc_ptr, N, rank, world)
                msg = _lib.last_error() if rc else ""
                torch.cuda.synchronize()
                dist.barrier()
                torch.cuda.synchronize()
                if rc == _lib.OK:
                    ops.check_device_status(rank)
                    got = c_local.cpu().numpy().view(np.uint16)
                    err = O.rel_frobenius(got, dtype, O.gemm(dtype, A, B))
                    result = (rank, "ok", float(err))
                else:
                    result = (rank, "error", msg)
            finally:
                buf.release()
    except Exception as e:  # reported through the queue; the process still leaves in order
        result = (rank, "error", repr(e))
    finally:
        q.put(result)
        dist.destroy_process_group()


def test_real_ranks_over_multicast_memory(oracle):
    import torch
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    import socket
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main_multicast, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    if all(kind == "unsupported" for _, kind, _ in results):
        pytest.skip("multicast objects are not available here: " + str(results[0][2]))
    for rank, kind, val in results:
        assert kind == "ok", (rank, kind, val)
        assert val <= TOL[_lib.BF16], (rank, val)


def test_multicast_entry_refuses_what_it_cannot_store(btm):
    L = _lib.lib()
    p = C.c_void_p(256)
    # Nloc not a multiple of 8: the 16-byte multimem stores could not be clipped
    assert L.btm_gemm_nshard_mc(0, None, _lib.F16, 8, 12, 64, p, 64, p, 12, p, p, 24, 0, 2) == _lib.ERR_UNSUPPORTED
    assert L.btm_gemm_nshard_mc(0, None, _lib.F32, 8, 8, 64, p, 64, p, 8, p, p, 16, 0, 2) == _lib.ERR_UNSUPPORTED
    assert L.btm_gemm_nshard_mc(0, None, _lib.F16, 8, 8, 64, p, 64, p, 8, None, p, 16, 0, 2) == _lib.ERR_INVALID


def _rank_main_two_layer(rank, world, port, q):
    # GEMM -> all-gather -> next GEMM, whole and pipelined by row panels, over plain peer memory.
    sys.path.insert(0, ROOT)
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "NCCL_NVLS_ENABLE": "0"})
    import torch
    import torch.distributed as dist
    from beantensor_b200 import ops
    from beantensor_b200.errors import raise_for_status
    from beantensor_b200.pipeline import TwoLayerNShard
    from oracle import oracle as O
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        ops.init(rank)
        L = _lib.lib()
        dtype = _lib.BF16
        M, K1, N1, N2 = 512, 320, 256 * world, 128 * world
        A, B1 = gemm_inputs(dtype, M, N1, K1, 71)
        _, B2 = gemm_inputs(dtype, M, N2, N1, 72)
        c0, c1 = sharding.column_block(N1, rank, world)
        d0, d1 = sharding.column_block(N2, rank, world)
        a = to_gpu(A, dtype)
        b1 = to_gpu(np.ascontiguousarray(B1[:, c0:c1]), dtype)
        b2 = to_gpu(np.ascontiguousarray(B2[:, d0:d1]), dtype)
        ptr, handle = C.c_void_p(), C.create_string_buffer(64)
        raise_for_status(L.btm_ipc_alloc(rank, M * N1 * 2, C.byref(ptr), handle))
        handles = [None] * world
        dist.all_gather_object(handles, handle.raw)
        peers = []
        for r in range(world):
            if r == rank:
                peers.append(ptr.value)
            else:
                p = C.c_void_p()
                raise_for_status(L.btm_ipc_open(rank, handles[r], C.byref(p)))
                peers.append(p.value)

        class Raw:
            __cuda_array_interface__ = {"shape": (M, N1), "typestr": "<i2", "data": (ptr.value, False), "version": 2}

        c1_view = torch.as_tensor(Raw(), device="cuda").view(torch.bfloat16)
        c2 = torch.full((M, d1 - d0), float("nan"), dtype=torch.bfloat16, device="cuda")
        chain = TwoLayerNShard(dist, rank, rank, world, dtype, a, b1, b2, None, None, peers, c1_view, c2, panels=4)
        # what layer 2 multiplies is the ROUNDED C1, so the checker rounds it too
        c1_ref = O.narrow(O.gemm(dtype, A, B1), dtype)
        ref = O.gemm(dtype, c1_ref, np.ascontiguousarray(B2[:, d0:d1]))
        errs = []
        for run in (chain.run_sequential, chain.run_pipelined):
            c1_view.fill_(float("nan"))
            c2.fill_(float("nan"))
            torch.cuda.synchronize()
            dist.barrier()
            run()
            torch.cuda.synchronize()
            dist.barrier()
            ops.check_device_status(rank)
            errs.append(float(O.rel_frobenius(c2.cpu().view(torch.uint16).numpy(), dtype, ref)))
        for r in range(world):
            if r != rank:
                L.btm_ipc_close(rank, C.c_void_p(peers[r]))
        dist.barrier()
        L.btm_ipc_free(rank, ptr)
        q.put((rank, errs))
    finally:
        dist.destroy_process_group()


def test_two_layer_chain_whole_and_pipelined(oracle):
    import torch
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    import socket
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main_two_layer, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, errs in results:
        for err in errs:
            assert err <= 2 * TOL[_lib.BF16], (rank, errs)  # two roundings to bf16 on the way
