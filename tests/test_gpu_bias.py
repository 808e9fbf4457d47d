"""GPU: the bias fused into the matmul epilogues (the reference adds it with a separate torch op,
gemlite/core.py:271-272).  The bias is drawn as large as the outputs and the output dtype is fp32, so a dropped,
doubled or mis-indexed bias cannot hide under a whole-tensor norm:
  * (y with bias) - (y without bias) equals the bias to fp32 rounding, element by element;
  * the last batch row and the last 32-column chunk (ragged edge) agree with the fp64 formula element by element.
Kernels: general streaming kernel (N = 2032 is not a multiple of 32), warp-independent streaming kernel, tcgen05 A16Wn
kernel (M > 16), and the general CUDA-core kernel (kernel_override = 1)."""
import ctypes

import numpy as np
import pytest
import torch

from tests.util import make_a16wn

pytestmark = pytest.mark.gpu


def _layer(W_q, s, z, bias, nbits, gs, dtype):
    from gemlite_b200 import GemLiteLinear, DType
    N, K = W_q.shape
    idt = DType.BF16 if dtype == torch.bfloat16 else DType.FP16
    layer = GemLiteLinear(nbits, gs, K, N, input_dtype=idt, output_dtype=DType.FP32)
    layer.pack(W_q.cuda(), s.cuda(), z.cuda(), bias=None if bias is None else bias.cuda())
    return layer


def _kernel(layer, x):
    from gemlite_b200 import core, _lib
    out = torch.empty((x.shape[0], layer.out_features), dtype=torch.float32, device="cuda")
    a = core._fill_args(x, None, layer.W_q, layer.scales, layer.zeros, None, None, out, layer.get_meta_args(), -1)
    return _lib.lib().gl_matmul_kernel_name(ctypes.byref(a)).decode()


CASES = [  # (N, K, nbits, gs, M, expected kernel, element tolerance in units of rms(y))
    (2032, 3968, 4, 128, 1, "gl_gemv_stream_kernel", 2e-4),
    (2032, 3968, 4, 128, 5, "gl_gemv_stream_kernel", 2e-4),
    (2032, 3968, 2, 64, 16, "gl_gemv_stream_kernel", 2e-4),
    (2048, 4096, 4, 128, 1, "gl_gemv_warp_kernel", 2e-4),
    (2048, 4096, 4, 128, 5, "gl_gemv_warp_kernel", 2e-4),
    (2048, 4096, 2, 64, 16, "gl_gemv_warp_kernel", 2e-4),
    (2048, 4096, 8, 128, 16, "gl_gemv_warp_kernel", 2e-4),
    (2048, 4096, 4, 32, 32, "gl_gemv_warp_kernel", 2e-4),     # groups of 32: two 16-row launches of the streaming kernel
    (2048, 4096, 4, 128, 32, "gl_gemm_tc_kernel", 3e-2),      # operands swapped
    (2032, 3968, 4, 128, 33, "gl_gemm_tc_kernel", 3e-2),      # weights rounded to bf16 after dequantisation, as the reference does
    (2032, 3968, 4, 128, 130, "gl_gemm_tc_kernel", 3e-2),
    (2032, 3968, 2, 64, 130, "gl_gemm_tc_kernel", 3e-2),
]


@pytest.mark.parametrize("N,K,nbits,gs,M,kernel,etol", CASES)
@pytest.mark.parametrize("override", [0, 1])
def test_fused_bias_element_wise(lib, N, K, nbits, gs, M, kernel, etol, override):
    from gemlite_b200 import core
    if override == 1 and M > 33:
        pytest.skip("general kernel: one large case is enough")
    if override == 1:
        etol = max(etol, 3e-2)     # the general kernel dequantises in the scale dtype, like the reference
    dtype = torch.bfloat16
    x, W_q, s, z, _ = make_a16wn(N, K, nbits, gs, dtype, seed=700 + M + nbits, M=M, with_bias=False)
    # the layer stores z' = -(z * s) rounded to the scale dtype (fma mode, gemlite/core.py:673-675): the element-wise
    # truth is the fp64 value of x @ (W_q * s + z') with that stored z'
    zp = (-z.float() * s.float()).to(dtype)
    want0 = (x.double() @ (W_q.double().view(N, -1, gs) * s.double().view(N, -1, 1) + zp.double().view(N, -1, 1)).view(N, K).T).numpy()
    rms = float(np.sqrt((want0 ** 2).mean()))
    g = torch.Generator().manual_seed(5)
    bias = (torch.randn(N, generator=g) * rms).float()                     # as large as the outputs
    with_b, without_b = _layer(W_q, s, z, bias, nbits, gs, dtype), _layer(W_q, s, z, None, nbits, gs, dtype)
    xd = x.cuda()
    if override == 0:
        assert _kernel(with_b, xd) == kernel
    core.set_kernel_override(override)
    try:
        yb = with_b(xd).double().cpu().numpy()
        y0 = without_b(xd).double().cpu().numpy()
    finally:
        core.set_kernel_override(0)
    assert yb.dtype == np.float64 and yb.shape == (M, N)
    # the epilogue adds exactly bias[n] to column n of every row
    diff = (yb - y0) - bias.double().numpy()[None, :]
    assert np.abs(diff).max() <= 4e-6 * np.abs(yb).max(), np.abs(diff).max()
    # element-wise agreement with fp64 on the last row and on the ragged last column chunk
    want = want0 + bias.double().numpy()[None, :]
    assert np.abs(yb[-1] - want[-1]).max() <= etol * rms, np.abs(yb[-1] - want[-1]).max() / rms
    assert np.abs(yb[:, -32:] - want[:, -32:]).max() <= etol * rms
    assert np.abs(yb - want).max() <= 2 * etol * rms
