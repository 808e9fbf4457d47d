"""CPU, world size 2 over gloo: the tensor-parallel sharding and its collective.  Each rank's matmul is the
oracle (test infrastructure) so that no GPU is needed; what is under test is the host logic: column shards
concatenate to the full output, row shards plus all-reduce equal the full output, the bias is added once."""
import os

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests.util import make_a16wn


class OracleLayer:
    """x -> x @ ((W_q - z) * s).T + bias on the CPU (stands in for a packed GemLiteLinear)."""

    def __init__(self, W_q, s, z, bias, gs):
        N, K = W_q.shape
        self.W = ((W_q.double().view(N, -1, gs) - z.double().view(N, -1, 1)) * s.double().view(N, -1, 1)).view(N, K)
        self.bias = bias

    def __call__(self, x):
        y = x.double() @ self.W.T
        return y + self.bias.double() if self.bias is not None else y


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from gemlite_b200 import tp
    N, K, gs = 64, 512, 128
    x, W_q, s, z, b = make_a16wn(N, K, 4, gs, torch.float32, seed=5, M=3)
    full = OracleLayer(W_q, s, z, b, gs)(x)
    # column parallel
    Wc, sc, zc, bc = tp.shard_column(W_q, s, z, b, world, rank, gs)
    yc = tp.TPLinear(OracleLayer(Wc, sc, zc, bc, gs), "column")(x)
    gathered = [torch.empty_like(yc) for _ in range(world)]
    dist.all_gather(gathered, yc)
    ok_col = torch.allclose(torch.cat(gathered, -1), full, atol=1e-9)
    # row parallel: x is sharded along K, output all-reduced, bias only on rank 0
    Wr, sr, zr, br = tp.shard_row(W_q, s, z, b, world, rank, gs)
    a, e = tp.shard_bounds(K, world, rank, gs)
    yr = tp.TPLinear(OracleLayer(Wr, sr, zr, br, gs), "row")(x[:, a:e])
    ok_row = torch.allclose(yr, full, atol=1e-9)
    ok_bias = (br is not None) == (rank == 0)
    results[rank] = (ok_col, ok_row, ok_bias)
    dist.barrier()
    dist.destroy_process_group()


def test_column_and_row_parallel_world2():
    mp.set_start_method("spawn", force=True)
    mgr = mp.Manager()
    results = mgr.dict()
    port = 29000 + (os.getpid() % 2000)
    procs = [mp.Process(target=_worker, args=(r, 2, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert dict(results) == {0: (True, True, True), 1: (True, True, True)}


def test_shard_bounds_and_quantizer():
    from gemlite_b200 import tp
    assert tp.shard_bounds(8192, 8, 3, 128) == (3072, 4096)
    assert tp.shard_bounds(28672, 8, 7, 128) == (25088, 28672)
    try:
        tp.shard_bounds(4224, 8, 0, 128)
        assert False
    except ValueError:
        pass
    g = torch.Generator().manual_seed(1)
    W = (torch.randn(32, 256, generator=g) * 0.02)
    W_q, s, z = tp.quantize_affine_minmax(W, 4, 128)
    rec = ((W_q.float().view(32, -1, 128) - z.view(32, -1, 1)) * s.view(32, -1, 1)).view(32, 256)
    assert W_q.dtype == torch.uint8 and int(W_q.max()) <= 15
    assert (rec - W).abs().max() <= s.max() * 0.51
