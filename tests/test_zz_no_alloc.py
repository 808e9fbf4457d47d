"""GPU: gl_matmul_noalloc -- the matmul entry point for callers that cannot allocate device memory.

Some users of the C ABI never get to call cudaMalloc: a plug-in that is only handed tensors by its host
framework, a serving loop that must not stall the device with an allocation, a binding from a runtime without a
device allocator.  For them the library carries its own 4 MiB scratch array and this entry point uses it instead
of a caller workspace.  The test calls it through the C ABI twice in a row on the same inputs (the second call
finds the array as the first one left it) and compares each result with the ordinary entry point, within the
tolerance the other A16Wn tests use; it also checks the documented limits.  It does not depend on any other test
having run (or not run) in the same process.
"""
import ctypes
import gc

import pytest
import torch

from tests.util import make_a16wn, exact_a16wn, rel_fro

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _args(layer, x, out):
    from gemlite_b200 import core
    return core._fill_args(x, layer.bias, layer.W_q, layer.scales, layer.zeros, None, None, out, layer.get_meta_args(), -1)


@pytest.mark.parametrize("M,nbits,gs,dtype", [(1, 4, 128, torch.bfloat16), (5, 2, 64, torch.float16), (16, 4, 128, torch.bfloat16), (3, 1, 128, torch.float16)])
def test_noalloc_matches_regular_entry_point_twice(lib, M, nbits, gs, dtype):
    from gemlite_b200 import helper, core, _lib
    N, K = 2032, 3968
    x, W_q, s, z, b = make_a16wn(N, K, nbits, gs, dtype, seed=900 + M, M=M)
    b = (b.float() * 500).to(dtype)          # a bias as large as the outputs: a dropped or shifted bias must show
    layer = helper.A16Wn_HQQ_INT(device="cuda:0", dtype=dtype, W_nbits=nbits).from_weights(W_q.cuda(), s.cuda(), z.cuda(), bias=b.cuda())
    xd = x.cuda()
    stream = torch.cuda.current_stream().cuda_stream

    # ordinary entry point, caller-provided workspace
    ref = torch.empty((M, N), dtype=dtype, device="cuda")
    a = _args(layer, xd, ref)
    ws = core._workspace(xd.device, int(lib.gl_matmul_workspace_bytes(ctypes.byref(a))))
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    assert lib.gl_matmul(ctypes.byref(a), stream) == 0, lib.gl_last_error()

    want = exact_a16wn(x, W_q, s, z, b, gs)
    for call in range(2):
        out = torch.full((M, N), float("nan"), dtype=dtype, device="cuda")
        an = _args(layer, xd, out)           # no workspace given: the fields stay NULL / 0
        # nothing may be allocated by the call: neither through torch's allocator nor behind its back (cudaMalloc
        # shows in the driver's free-memory figure; tensors of earlier tests are collected first so that their
        # release does not land inside the window)
        gc.collect()
        torch.cuda.synchronize()
        before, free_before = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
        assert lib.gl_matmul_noalloc(ctypes.byref(an), stream) == 0, lib.gl_last_error()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() <= before
        assert torch.cuda.mem_get_info()[0] >= free_before - (1 << 20)
        assert rel_fro(out.float().cpu().numpy(), ref.float().cpu().numpy()) < TOL, call
        assert rel_fro(out.float().cpu().numpy(), want) < TOL, call
        # element by element: the two entry points may differ by the rounding of the output dtype only
        d = (out.float() - ref.float()).abs()
        assert bool((d <= 2.0 ** -6 * ref.float().abs() + 1e-3 * float(ref.float().abs().mean())).all()), call


def test_noalloc_limits_are_reported(lib):
    from gemlite_b200 import helper, _lib
    # partial sums of M = 32, N = 16384 do not fit the 4 MiB array: a clear error, not a silent fallback
    N, K = 16384, 1024
    x, W_q, s, z, b = make_a16wn(N, K, 4, 128, torch.bfloat16, seed=7, M=32, with_bias=False)
    layer = helper.A16W4_HQQ_INT(device="cuda:0", dtype=torch.bfloat16).from_weights(W_q.cuda(), s.cuda(), z.cuda())
    out = torch.empty((32, N), dtype=torch.bfloat16, device="cuda")
    a = _args(layer, x.cuda(), out)
    assert lib.gl_matmul_noalloc(ctypes.byref(a), torch.cuda.current_stream().cuda_stream) == _lib.GL_E_WORKSPACE
    msg = lib.gl_last_error().decode()
    assert "4194304" in msg and "scratch" in msg
    # a problem the streaming kernel does not serve (M = 64) is refused as unsupported
    x2 = torch.randn(64, K, dtype=torch.bfloat16, device="cuda")
    out2 = torch.empty((64, N), dtype=torch.bfloat16, device="cuda")
    a2 = _args(layer, x2, out2)
    assert lib.gl_matmul_noalloc(ctypes.byref(a2), torch.cuda.current_stream().cuda_stream) == _lib.GL_E_UNSUPPORTED
