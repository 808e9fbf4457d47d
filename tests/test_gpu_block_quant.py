"""GPU: 128 x 128 block quantisation (channel_scale_mode 5; the reference's A8W8_*_dynamic(block_quant=True), tested
there by tests/test_int.py:342-379): the per-block activation quantiser against the oracle and the reference's torch
function, and the layer against the oracle fed with the identical quantised operands (5e-3) and against the
unquantised product."""
import numpy as np
import pytest
import torch

from oracle import oracle
from tests import golden_inputs as gi
from tests.util import rel_fro

pytestmark = pytest.mark.gpu


def test_per_block_quantiser_matches_oracle_and_golden(lib):
    from gemlite_b200 import quant_utils as qu
    gold = np.load(gi.GOLDEN_BLOCK_QUANT)
    for seed, M, K in gi.BLOCK_QUANT_CASES:
        x = gi.block_quant_input(seed, M, K)
        for kind, dt in (("fp8", torch.float8_e4m3fn), ("int8", torch.int8)):
            q, s = qu.scale_activations_per_block(x.cuda(), dt)
            qo, so = oracle.scale_activations_per_block(x.float().numpy(), kind)
            assert s.shape == (M, K // 128) and s.dtype == torch.float32
            assert np.array_equal(s.cpu().numpy(), so) and np.array_equal(so, gold["s_%s_s%d" % (kind, seed)])
            got = q.view(torch.uint8).cpu().numpy() if kind == "fp8" else q.cpu().numpy()
            assert np.array_equal(got, qo)                                        # bit-exact against the oracle
            qt, st = qu.scale_activations_per_block_torch(x, dt)                  # the torch restatement kept beside it
            assert np.array_equal(st.numpy(), so)


def _kernel_name(layer, x, fp8):
    import ctypes
    from gemlite_b200 import core, quant_utils as qu, _lib
    xq, sx = qu.scale_activations_per_block(x, torch.float8_e4m3fn if fp8 else torch.int8)
    out = torch.empty((x.shape[0], layer.out_features), dtype=x.dtype, device="cuda")
    a = core._fill_args(xq, layer.bias, layer.W_q, layer.scales, layer.zeros, sx, None, out, layer.get_meta_args(), -1)
    return _lib.lib().gl_matmul_kernel_name(ctypes.byref(a)).decode()


@pytest.mark.parametrize("fp8", [True, False])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_block_quant_layer(lib, fp8, dtype):
    from gemlite_b200 import helper
    for (N, K) in ((2032, 3968), (512, 1024)):                                    # the reference's test shape (ragged N) and a small one
        g = torch.Generator().manual_seed(7200 + N)
        W = (torch.randn(N, K, generator=g) * 0.05).to(dtype)
        bias = (torch.randn(N, generator=g) * 0.5).to(dtype)
        lin = torch.nn.Linear(K, N, bias=True, dtype=dtype)
        lin.weight.data, lin.bias.data = W.clone(), bias.clone()
        proc = (helper.A8W8_FP8_dynamic if fp8 else helper.A8W8_INT8_dynamic)(device="cuda:0", dtype=dtype, block_quant=True)
        layer = proc.from_linear(lin.cuda(), del_orig=False)
        assert (layer.W_group_mode, layer.channel_scale_mode) == (0, 5)
        assert layer.scales.shape == ((K + 127) // 128, (N + 127) // 128) and layer.scales.dtype == torch.float32
        kind = "fp8" if fp8 else "int8"
        wq_o, sw_o = oracle.quantize_block_weights(W.float().numpy(), kind)
        # the weights are quantised with torch ops on the GPU, where a division by a scalar is a multiplication by its
        # reciprocal: scales within one ulp of the oracle's, codes equal except where that flips a rounding
        assert np.allclose(layer.scales.t().cpu().numpy(), sw_o, rtol=3e-7, atol=0)
        wq = layer.W_q.t().contiguous()
        wq = wq.view(torch.uint8).cpu().numpy() if fp8 else wq.cpu().numpy()
        assert (wq != wq_o).mean() < 5e-3
        for M in (1, 3, 16, 17, 65, 130, 300, 700):
            x = (torch.randn(M, K, generator=g) / 10.0).to(dtype)
            y = layer(x.cuda()).float().cpu().numpy()
            # the tensor-core kernel (one partial sum per K tile, scaled into register accumulators) at every batch size
            assert _kernel_name(layer, x.cuda(), fp8) == "gl_gemm_tc_kernel"
            from gemlite_b200 import core
            core.set_kernel_override(1)                                            # ... and the general kernel agrees with it
            try:
                y_gen = layer(x.cuda()).float().cpu().numpy()
            finally:
                core.set_kernel_override(0)
            assert rel_fro(y, y_gen) < 5e-3
            xq, sx = oracle.scale_activations_per_block(x.float().numpy(), kind)
            want_q = oracle.matmul_block_quant(xq, sx, wq, layer.scales.t().cpu().numpy(), kind, bias=bias.double().numpy())
            assert rel_fro(y, want_q) < 5e-3, (N, K, M, rel_fro(y, want_q))
            want = (x.double() @ W.double().T + bias.double()).numpy()
            assert rel_fro(y, want) < (5e-2 if fp8 else 2e-2)
            # the reference's own criterion (tests/test_int.py:96-97, 342-379) is a mean absolute error below 5e-3 on its
            # data; here the outputs have std 0.3, where that bound is met by INT8 and is the e4m3 rounding itself for FP8
            assert float(np.abs(y - want).mean()) < (1.5e-2 if fp8 else 5e-3)


@pytest.mark.parametrize("fp8", [True, False])
def test_block_quant_wide_tiles(lib, fp8):
    """Enough 128 x 256 tiles for every SM (19 x 8): the 256-column form, two weight blocks per tile with a ragged last
    one (N = 2032), rows ending inside a tile."""
    from gemlite_b200 import helper, quant_utils as qu
    N, K, M = 2032, 1024, 2500
    kind = "fp8" if fp8 else "int8"
    g = torch.Generator().manual_seed(7400)
    W = torch.randn(N, K, generator=g) * 0.05
    W[128:256] *= 30.0                                      # neighbouring weight blocks with very different scales
    bias = (torch.randn(N, generator=g) * 0.5).to(torch.bfloat16)
    wq, sw = oracle.quantize_block_weights(W.numpy(), kind)
    layer = (helper.A8W8_FP8_dynamic if fp8 else helper.A8W8_INT8_dynamic)(device="cuda:0", dtype=torch.bfloat16, block_quant=True).from_weights(
        torch.from_numpy(wq).view(torch.float8_e4m3fn) if fp8 else torch.from_numpy(wq), scales=torch.from_numpy(sw), bias=bias)
    x = (torch.randn(M, K, generator=g) / 10.0).to(torch.bfloat16)
    x[:, 128:256] *= 50.0                                   # ... and activation blocks likewise
    assert _kernel_name(layer, x.cuda(), fp8) == "gl_gemm_tc_kernel"
    y = layer(x.cuda()).float().cpu().numpy()
    xq, sx = qu.scale_activations_per_block(x.cuda(), torch.float8_e4m3fn if fp8 else torch.int8)
    xq = xq.view(torch.uint8).cpu().numpy() if fp8 else xq.cpu().numpy()
    want = oracle.matmul_block_quant(xq, sx.cpu().numpy(), wq, sw, kind, bias=bias.double().numpy())
    assert rel_fro(y, want) < 5e-3, rel_fro(y, want)
    for rows in (slice(0, 1), slice(M - 1, M), slice(2432, M)):                    # first, last, the ragged last row tile
        assert rel_fro(y[rows], want[rows]) < 5e-3
    assert rel_fro(y[:, 1920:], want[:, 1920:]) < 5e-3 and rel_fro(y[:, 128:256], want[:, 128:256]) < 5e-3


def test_block_quant_pre_quantised_weights(lib):
    from gemlite_b200 import helper
    N, K = 256, 512
    g = torch.Generator().manual_seed(7300)
    W = (torch.randn(N, K, generator=g) * 0.05)
    wq, sw = oracle.quantize_block_weights(W.numpy(), "int8")
    layer = helper.A8W8_INT8_dynamic(device="cuda:0", dtype=torch.bfloat16, block_quant=True).from_weights(
        torch.from_numpy(wq), scales=torch.from_numpy(sw))
    x = (torch.randn(4, K, generator=g) / 10.0).to(torch.bfloat16)
    y = layer(x.cuda()).float().cpu().numpy()
    xq, sx = oracle.scale_activations_per_block(x.float().numpy(), "int8")
    assert rel_fro(y, oracle.matmul_block_quant(xq, sx, wq, sw, "int8")) < 5e-3
    with pytest.raises(AssertionError):
        helper.A8W8_INT8_dynamic(device="cuda:0", dtype=torch.bfloat16, block_quant=True).from_weights(torch.from_numpy(wq), scales=torch.from_numpy(sw[:1]))
