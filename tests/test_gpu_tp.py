"""GPU: the tensor-parallel pieces.

One GPU: the silu*mul glue kernel against torch; the one-shot all-reduce with a single rank (a copy through the
receive area); and a wait that runs out: a two-rank communicator whose second "rank" is a buffer that nobody ever
signals, with a wait budget of about a millisecond -- the kernel must return, record the time-out in the status word
and leave the stream usable (nothing traps, nothing hangs).

Two or more GPUs (child processes, one per GPU, NCCL for the plumbing): the one-shot all-reduce against NCCL's on the
same tensors, bit-identical on all ranks; and the Llama decoder-layer linears sharded column / row parallel against
the same layers unsharded on one GPU, relative Frobenius 1e-2, for M in {1, 8, 64}."""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _local_comm(lib, world, slot_bytes, wait_cycles=0):
    from gemlite_b200 import _lib
    comm = _lib.GLTpComm()
    comm.rank, comm.world, comm.slot_bytes, comm.wait_cycles = 0, world, slot_bytes, wait_cycles
    ptrs = []
    for r in range(world):
        p, h = ctypes.c_void_p(), (ctypes.c_uint8 * 64)()
        assert lib.gl_tp_buffer_create(int(lib.gl_tp_buffer_bytes(world, slot_bytes)), ctypes.byref(p), h) == 0, lib.gl_last_error()
        comm.buffers[r] = p.value
        ptrs.append(p.value)
    return comm, ptrs


def test_silu_mul_matches_torch(lib):
    from gemlite_b200 import tp
    for M, inter, dtype in ((1, 3584, torch.bfloat16), (5, 1000, torch.float16), (64, 3584, torch.bfloat16)):
        gu = torch.randn(M, 2 * inter, device="cuda", dtype=dtype) * 2
        got = tp.silu_mul(gu)
        want = torch.nn.functional.silu(gu[:, :inter]) * gu[:, inter:]
        assert got.shape == want.shape
        err = (got.float() - want.float()).abs()
        assert bool((err <= 2.0 ** -6 * want.float().abs() + 1e-6).all())    # at most one rounding step of the dtype apart


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_allreduce_single_rank_is_a_copy(lib, dtype):
    from gemlite_b200 import _lib
    from gemlite_b200.dtypes import TORCH_TO_DTYPE
    comm, ptrs = _local_comm(lib, 1, 4 << 20)
    st = torch.cuda.current_stream().cuda_stream
    try:
        for n in (8192, 64 * 8192, 16):
            x = torch.randn(n, device="cuda").to(dtype)
            for _ in range(3):                       # the epoch advances, the receive areas alternate
                out = torch.zeros_like(x)
                assert lib.gl_tp_allreduce(ctypes.byref(comm), x.data_ptr(), out.data_ptr(), n, TORCH_TO_DTYPE[dtype].value,
                                           TORCH_TO_DTYPE[dtype].value, st) == 0, lib.gl_last_error()
                torch.cuda.synchronize()
                assert torch.equal(out, x)
        status, epoch = ctypes.c_int32(), ctypes.c_uint32()
        assert lib.gl_tp_status(ctypes.byref(comm), ctypes.byref(status), ctypes.byref(epoch)) == 0
        assert status.value == 0 and epoch.value == 9
        # too large for the receive slots: an error, nothing is launched
        big = torch.zeros((4 << 20) // 4 + 8, device="cuda", dtype=torch.float32)
        assert lib.gl_tp_allreduce(ctypes.byref(comm), big.data_ptr(), big.data_ptr(), big.numel(), 0, 0, st) == _lib.GL_E_WORKSPACE
    finally:
        torch.cuda.synchronize()
        for p in ptrs:
            lib.gl_tp_buffer_destroy(p)


def test_allreduce_wait_runs_out_and_reports(lib):
    """A peer that never signals: the flag wait gives up after its cycle budget, the status word names the rank, the
    kernel returns and later work on the stream runs normally."""
    from gemlite_b200.dtypes import TORCH_TO_DTYPE
    comm, ptrs = _local_comm(lib, 2, 1 << 16, wait_cycles=2_000_000)      # about a millisecond
    st = torch.cuda.current_stream().cuda_stream
    try:
        x = torch.ones(4096, device="cuda", dtype=torch.bfloat16)
        out = torch.full_like(x, 7.0)
        code = TORCH_TO_DTYPE[torch.bfloat16].value
        assert lib.gl_tp_allreduce(ctypes.byref(comm), x.data_ptr(), out.data_ptr(), x.numel(), code, code, st) == 0
        torch.cuda.synchronize()                                          # returns: the wait is bounded
        status, epoch = ctypes.c_int32(), ctypes.c_uint32()
        assert lib.gl_tp_status(ctypes.byref(comm), ctypes.byref(status), ctypes.byref(epoch)) == 0
        assert status.value == 101                                        # 100 + the rank that never arrived
        assert bool((out == 7.0).all())                                   # the affected chunks are left unwritten
        y = (x.float() * 2).sum()                                         # the context is alive
        assert float(y) == 8192.0
    finally:
        torch.cuda.synchronize()
        for p in ptrs:
            lib.gl_tp_buffer_destroy(p)


# ---- two or more GPUs ---------------------------------------------------------------------------------------
def _tp_worker(rank, world, port, results):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from gemlite_b200 import tp
    out = {}
    comm = tp.PeerComm(dev, slot_bytes=2 << 20)
    try:
        # (1) one-shot all-reduce against NCCL, repeated so that both receive areas and several epochs are used
        g = torch.Generator(device=dev).manual_seed(100 + rank)
        ok_sum, ok_same = True, True
        for n in (8192, 8 * 8192, 64 * 8192, 128):
            for rep in range(4):
                x = torch.randn(n, generator=g, device=dev).to(torch.bfloat16)
                got = comm.all_reduce(x)
                parts = [torch.empty_like(x) for _ in range(world)]
                dist.all_gather(parts, x)
                want = parts[0].float()
                for q in parts[1:]:
                    want = want + q.float()                                # rank order, fp32: what the kernel computes
                ok_sum &= bool(torch.equal(got, want.to(torch.bfloat16)))
                gathered = [torch.empty_like(got) for _ in range(world)]
                dist.all_gather(gathered, got)
                ok_same &= all(bool(torch.equal(gathered[0], t)) for t in gathered)
        out["allreduce_exact"], out["allreduce_same_on_all_ranks"] = ok_sum, ok_same
        out["status"] = comm.status()[0]
        # (2) sharded decoder-layer linears against the unsharded ones
        dims = dict(hidden=2048, intermediate=7168, n_heads=16, n_kv_heads=8, head_dim=128)
        blk = tp.LlamaLinears(world=world, rank=rank, device=dev, seed=3, comm=comm, **dims)
        full = tp.LlamaLinears(world=1, rank=0, device=dev, seed=3, **dims)
        errs = {}
        for M in (1, 8, 64):
            gx = torch.Generator(device=dev).manual_seed(7 + M)                # same x on every rank
            x = (torch.randn(M, dims["hidden"], generator=gx, device=dev) * 0.5).to(torch.bfloat16)
            y, y1 = blk(x).float(), full(x).float()
            errs[M] = float((y - y1).norm() / y1.norm())
        out["tp_rel_err"] = errs
        out["status_after"] = comm.status()[0]
    finally:
        comm.close()
    results[rank] = out
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
def test_tensor_parallel_on_gpus(lib):
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 8)
    world = 1 << (world.bit_length() - 1)           # 2, 4 or 8
    ctx = mp.get_context("spawn")
    mgr = ctx.Manager()
    results = mgr.dict()
    port = 29500 + (os.getpid() % 1000)
    procs = [ctx.Process(target=_tp_worker, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(600)
        assert p.exitcode == 0
    for r in range(world):
        res = results[r]
        assert res["allreduce_exact"] and res["allreduce_same_on_all_ranks"], res
        assert res["status"] == 0 and res["status_after"] == 0
        for M, e in res["tp_rel_err"].items():
            assert e < 1e-2, (r, M, e)
