"""GPU: the other weight formats through GemLiteLinear / the helper processors and the C ABI,
against the oracle: A8W8 FP8 / INT8 dynamic (channel-wise scales), A16W8, MXFP4 / NVFP4 block-scaled
with fused-in-forward activation quantisation, and weight-only MX / NV.  Tolerances: 1e-2 relative
Frobenius for 16-bit paths, 3e-2 for FP8 / FP4 paths (quantisation of the activations is part of the
operator, so the reference point is the oracle fed with the same quantised activations, at 1e-3,
and the unquantised layer at the looser bound)."""
import numpy as np
import pytest
import torch

from oracle import oracle
from tests.util import rel_fro

pytestmark = pytest.mark.gpu


def _lin(seed, N, K, dtype=torch.bfloat16, M=4, wstd=0.02):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g).to(dtype)
    W = (torch.randn(N, K, generator=g) * wstd).to(dtype)
    return x, W


@pytest.mark.parametrize("M", [1, 2, 16, 65, 130])
@pytest.mark.parametrize("fp8", [True, False])
def test_a8w8_dynamic(lib, M, fp8):
    from gemlite_b200 import helper
    N, K = 1024, 2048
    x, W = _lin(50 + M, N, K, M=M)
    proc = helper.A8W8_FP8_dynamic(device="cuda:0", dtype=torch.bfloat16) if fp8 else helper.A8W8_INT8_dynamic(device="cuda:0", dtype=torch.bfloat16)
    lin = torch.nn.Linear(K, N, bias=False, dtype=torch.bfloat16)
    lin.weight.data = W.clone()
    layer = proc.from_linear(lin.cuda())
    assert (layer.W_group_mode, layer.channel_scale_mode) == (0, 3)
    assert layer.scales.dtype == torch.float32 and layer.W_q.shape == (K, N) and layer.W_q.stride() == (1, K)
    y = layer(x.cuda()).float().cpu().numpy()
    # oracle on the same quantised operands
    xq, sx = oracle.scale_activations_per_token(x.float().numpy(), "fp8" if fp8 else "int8")
    Wq = layer.W_q.t().contiguous().cpu()
    if fp8:
        Xd, Wd = oracle.e4m3_decode(xq).astype(np.float64), Wq.float().double().numpy()
    else:
        Xd, Wd = xq.astype(np.float64), Wq.double().numpy()
    want_q = (Xd @ Wd.T) * sx.astype(np.float64) * layer.scales.cpu().double().numpy().reshape(1, -1)
    assert rel_fro(y, want_q) < 5e-3, rel_fro(y, want_q)
    want = (x.double() @ W.double().T).numpy()
    assert rel_fro(y, want) < 5e-2


@pytest.mark.parametrize("fp8", [True, False])
def test_a16w8(lib, fp8):
    from gemlite_b200 import helper
    N, K = 512, 1024
    x, W = _lin(60, N, K, torch.float16, M=3)
    for post_scale in (False, True):
        proc = (helper.A16W8_FP8 if fp8 else helper.A16W8_INT8)(device="cuda:0", dtype=torch.float16, post_scale=post_scale)
        layer = proc.from_weights(W.cuda())
        assert (layer.W_group_mode, layer.channel_scale_mode) == ((0, 1) if post_scale else (2, 0))
        y = layer(x.cuda()).float().cpu().numpy()
        Wd = layer.W_q.t().float().cpu().double() * layer.scales.cpu().double().view(-1, 1)
        assert rel_fro(y, (x.double() @ Wd.T).numpy()) < 1e-2


@pytest.mark.parametrize("fp8", [True, False])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_a16w8_decode_kernel(lib, fp8, dtype):
    """Weight-only INT8 / FP8 with one scale per channel at 1..4 rows runs on the streaming decode kernel of its own
    (the general kernel above that); ragged N and a K that is not a multiple of 512, with and without bias, both scale
    placements, against the fp64 product of the stored operands and against the general kernel."""
    import ctypes
    from gemlite_b200 import core, helper, _lib
    for (N, K) in ((2032, 3968), (4096, 8192)):
        g = torch.Generator().manual_seed(900 + N)
        W = (torch.randn(N, K, generator=g) * 0.05).to(dtype)
        bias = (torch.randn(N, generator=g) * 3.0).to(dtype)
        for post_scale in (False, True):
            proc = (helper.A16W8_FP8 if fp8 else helper.A16W8_INT8)(device="cuda:0", dtype=dtype, post_scale=post_scale)
            layer = proc.from_weights(W.cuda(), bias=bias.cuda() if post_scale else None)
            Wd = layer.W_q.t().float().cpu().double() * layer.scales.cpu().double().view(-1, 1)
            for M in (1, 2, 3, 4, 5):
                x = torch.randn(M, K, generator=g).to(dtype)
                xd = x.cuda()
                out = torch.empty((M, N), dtype=dtype, device="cuda")
                a = core._fill_args(xd, layer.bias, layer.W_q, layer.scales, layer.zeros, None, None, out, layer.get_meta_args(), -1)
                name = _lib.lib().gl_matmul_kernel_name(ctypes.byref(a)).decode()
                assert name == ("gl_w8_gemv_kernel" if M <= 4 else "gl_generic_kernel"), (M, name)
                y = layer(xd)
                assert torch.equal(y, layer(xd))                                   # deterministic
                want = (x.double() @ Wd.T).numpy() + (bias.double().numpy() if post_scale else 0.0)
                yn = y.float().cpu().numpy()
                assert rel_fro(yn, want) < 1e-2, (N, K, M, post_scale, rel_fro(yn, want))
                assert rel_fro(yn[-1], want[-1]) < 1e-2 and rel_fro(yn[:, -40:], want[:, -40:]) < 1e-2     # last row, ragged tail columns
                core.set_kernel_override(1)
                try:
                    yg = layer(xd).float().cpu().numpy()
                finally:
                    core.set_kernel_override(0)
                assert rel_fro(yn, yg) < 1e-2


@pytest.mark.parametrize("which", ["A16W4_MXFP", "A16W4_NVFP", "A16W8_MXFP"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_weight_only_fp4_decode_kernel(lib, which, dtype):
    """Weight-only MXFP4 / NVFP4 / MXFP8 (16-bit activations) at 1..4 rows runs on a streaming decode kernel; checked against the
    general kernel (which decodes every weight and scale individually) and against the unquantised product, on the
    reference's test shape 4224 -> 2048 (K is 132 groups of 32: a ragged last step) and a larger one."""
    import ctypes
    from gemlite_b200 import core, helper, _lib
    for (N, K) in ((2048, 4224), (4096, 8192)):
        g = torch.Generator().manual_seed(950 + N)
        lin = torch.nn.Linear(K, N, bias=True, dtype=dtype)
        lin.weight.data = (torch.randn(N, K, generator=g) / 10.0 / (K ** 0.5) * 8).to(dtype)
        lin.bias.data = torch.randn(N, generator=g).to(dtype) * 0.1
        W, b = lin.weight.data.clone(), lin.bias.data.clone()
        layer = getattr(helper, which)(device="cuda:0", dtype=dtype).from_linear(lin.cuda())
        for M in (1, 2, 4, 5):
            x = torch.randn(M, K, generator=g).to(dtype)
            xd = x.cuda()
            out = torch.empty((M, N), dtype=dtype, device="cuda")
            a = core._fill_args(xd, layer.bias, layer.W_q, layer.scales, layer.zeros, None,
                                layer.meta_scale.reshape(1) if which == "A16W4_NVFP" else None, out, layer.get_meta_args(), -1)
            name = _lib.lib().gl_matmul_kernel_name(ctypes.byref(a)).decode()
            fast = "gl_w8_gemv_kernel" if which == "A16W8_MXFP" else "gl_w4mx_gemv_kernel"
            assert name == (fast if M <= 4 else "gl_generic_kernel"), (M, name)
            y = layer(xd)
            assert torch.equal(y, layer(xd))
            core.set_kernel_override(1)
            try:
                yg = layer(xd).float().cpu().numpy()
            finally:
                core.set_kernel_override(0)
            yn = y.float().cpu().numpy()
            assert rel_fro(yn, yg) < 5e-3, (which, N, K, M, rel_fro(yn, yg))
            assert rel_fro(yn[-1], yg[-1]) < 5e-3 and rel_fro(yn[:, -33:], yg[:, -33:]) < 5e-3
            want = (x.double() @ W.double().T + b.double()).numpy()
            assert rel_fro(yn, want) < (0.2 if "W4" in which else 0.06)


@pytest.mark.parametrize("M", [1, 3, 16, 33, 100, 300, 1300, 3000])   # 1300 rows: 176 tiles of 128 columns, 3000 rows: 192 tiles of 256 columns
def test_a8w8_mxfp8_block_scaled_tensor_core(lib, M):
    """MXFP8 activations x MXFP8 weights with block scales on both sides (A8W8_MXFP_dynamic, post_scale=False; the
    reference's test: tests/test_mxfp.py:73-92) run on the tcgen05 kernel (kind::mxf8f6f4 with e8m0 scale atoms); checked
    against the oracle fed with the identical quantised operands and against the general kernel."""
    import ctypes
    from gemlite_b200 import core, helper, _lib, quant_utils as qu
    N, K = 2048, 4224                                                           # 33 K tiles of 128, 132 scale groups
    g = torch.Generator().manual_seed(970 + M)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    lin = torch.nn.Linear(K, N, bias=False, dtype=torch.bfloat16)
    lin.weight.data = (torch.randn(N, K, generator=g) / 10.0 / (K ** 0.5) * 8).to(torch.bfloat16)
    W = lin.weight.data.clone()
    layer = helper.A8W8_MXFP_dynamic(device="cuda:0", dtype=torch.bfloat16, post_scale=False).from_linear(lin.cuda())
    assert (layer.W_group_mode, layer.channel_scale_mode) == (0, 4)
    xd = x.cuda()
    xq, sx = qu.scale_activations_mxfp8(xd, scale_layout=1)
    out = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    a = core._fill_args(xq.view(M, K), layer.bias, layer.W_q, layer.scales, layer.zeros, sx, None, out, layer.get_meta_args(), -1,
                        core._scale_atoms_of(layer.scales), 1)
    assert _lib.lib().gl_matmul_kernel_name(ctypes.byref(a)).decode() == "gl_gemm_tc_kernel"
    y = layer(xd).float().cpu().numpy()
    xq_o, sx_o = oracle.scale_activations_mxfp8(x.float().numpy())
    wq = layer.W_q.t().contiguous().view(torch.uint8).cpu().numpy()
    sw = layer.scales.contiguous().view(torch.uint8).cpu().numpy()
    want_q = oracle.matmul_mx(xq_o, sx_o, wq, sw, 32, x_is_fp4=False, w_is_fp4=False)
    assert rel_fro(y, want_q) < 5e-3, (M, rel_fro(y, want_q))
    core.set_kernel_override(1)
    try:
        yg = layer(xd).float().cpu().numpy()
    finally:
        core.set_kernel_override(0)
    assert rel_fro(y, yg) < 5e-3
    assert rel_fro(y, (x.double() @ W.double().T).numpy()) < 0.06


@pytest.mark.parametrize("M", [1, 3, 16, 33, 100, 300, 1300, 3000])
def test_a8w8_mxfp8_weights_per_token_activations_tensor_core(lib, M):
    """A8W8_MXFP_dynamic(post_scale=True) (tests/test_mxfp.py:73-79): FP8 activations with one fp32 scale per token,
    MXFP8 weights.  The block-scaled MMA runs with unit activation scale atoms and the epilogue applies the token scale;
    checked against the product of the identical quantised operands and against the general kernel."""
    import ctypes
    from gemlite_b200 import core, helper, _lib, quant_utils as qu
    N, K = 2048, 4224
    g = torch.Generator().manual_seed(990 + M)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    x[M // 2] *= 37.0                                                            # token scales that differ a lot
    lin = torch.nn.Linear(K, N, bias=True, dtype=torch.bfloat16)
    lin.weight.data = (torch.randn(N, K, generator=g) / 10.0 / (K ** 0.5) * 8).to(torch.bfloat16)
    lin.bias.data = (torch.randn(N, generator=g) * 0.5).to(torch.bfloat16)
    W, bias = lin.weight.data.clone(), lin.bias.data.clone()
    layer = helper.A8W8_MXFP_dynamic(device="cuda:0", dtype=torch.bfloat16, post_scale=True).from_linear(lin.cuda())
    assert (layer.W_group_mode, layer.channel_scale_mode) == (0, 2)
    xd = x.cuda()
    xq, sx = qu.scale_activations_per_token(xd, torch.float8_e4m3fn)
    out = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    a = core._fill_args(xq.view(M, K), layer.bias, layer.W_q, layer.scales, layer.zeros, sx, None, out, layer.get_meta_args(), -1,
                        core._scale_atoms_of(layer.scales), 0)
    assert _lib.lib().gl_matmul_kernel_name(ctypes.byref(a)).decode() == "gl_gemm_tc_kernel"
    y = layer(xd).float().cpu().numpy()
    assert core.matmul_status("cuda:0", clear=False) == 0
    wq = layer.W_q.t().contiguous().view(torch.uint8).cpu().numpy()
    sw = layer.scales.contiguous().view(torch.uint8).cpu().numpy()
    Wd = (oracle.e4m3_decode(wq).astype(np.float64).reshape(N, K // 32, 32) * np.exp2(sw[:N].astype(np.float64) - 127.0)[..., None]).reshape(N, K)
    xq_o, sx_o = oracle.scale_activations_per_token(x.float().numpy(), "fp8")
    want_q = (oracle.e4m3_decode(xq_o).astype(np.float64) @ Wd.T) * sx_o.astype(np.float64).reshape(-1, 1) + bias.double().numpy()
    assert rel_fro(y, want_q) < 5e-3, (M, rel_fro(y, want_q))
    assert rel_fro(y[M // 2], want_q[M // 2]) < 5e-3 and rel_fro(y[-1], want_q[-1]) < 5e-3
    core.set_kernel_override(1)
    try:
        yg = layer(xd).float().cpu().numpy()
    finally:
        core.set_kernel_override(0)
    assert rel_fro(y, yg) < 5e-3
    assert rel_fro(y, (x.double() @ W.double().T + bias.double()).numpy()) < 0.06


@pytest.mark.parametrize("fmt", ["mxfp4", "nvfp4"])
@pytest.mark.parametrize("M", [1, 3, 16, 64, 100])
def test_a4w4_block_scaled(lib, fmt, M):
    # tests/test_mxfp.py shape: 4224 -> 2048, weights / 10
    from gemlite_b200 import helper
    N, K = 2048, 4224
    g = torch.Generator().manual_seed(70 + M)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    lin = torch.nn.Linear(K, N, bias=False, dtype=torch.bfloat16)
    lin.weight.data = (torch.randn(N, K, generator=g) / 10.0 / (K ** 0.5) * 8).to(torch.bfloat16)
    W = lin.weight.data.clone()
    proc = (helper.A4W4_MXFP_dynamic if fmt == "mxfp4" else helper.A4W4_NVFP_dynamic)(device="cuda:0", dtype=torch.bfloat16)
    layer = proc.from_linear(lin.cuda())
    gs = 32 if fmt == "mxfp4" else 16
    assert (layer.W_group_mode, layer.channel_scale_mode) == (0, 4)
    assert layer.W_q.numel() * layer.W_q.itemsize == N * K // 2            # tests/test_mxfp.py:96,102
    assert layer.W_q.shape == (K // 2, N) and layer.scales.shape == (N, K // gs) and layer.scales.stride() == (1, N)
    y = layer(x.cuda()).float().cpu().numpy()
    # oracle: same quantised weights (checked against the oracle's quantiser) and activations
    if fmt == "mxfp4":
        codes, sw = oracle.quantize_mxfp4_weights(W.float().numpy())
        xq, sx = oracle.scale_activations_mxfp4(x.float().numpy())
        meta = None
    else:
        mw = np.float32(layer.meta_scale.item())
        assert abs(float(mw) / float(oracle.quantize_nvfp4_weights(W.float().numpy())[2]) - 1.0) < 1e-6
        codes, sw, _ = oracle.quantize_nvfp4_weights(W.float().numpy(), meta=mw)
        xq, sx, mx = oracle.scale_activations_nvfp4(x.float().numpy())
        meta = 1.0 / (float(mw) * float(mx))
    wq = oracle.pack_fp4_codes(codes)
    assert np.array_equal(layer.W_q.t().contiguous().cpu().numpy(), wq)
    assert np.array_equal(layer.scales.contiguous().view(torch.uint8).cpu().numpy(), sw)
    want_q = oracle.matmul_mx(xq, sx, wq, sw, gs, meta_scale=meta)
    assert rel_fro(y, want_q) < 5e-3, rel_fro(y, want_q)
    want = (x.double() @ W.double().T).numpy()
    assert rel_fro(y, want) < 0.25      # fp4 x fp4 quantisation noise itself (reference tolerance is on mean abs error)


@pytest.mark.parametrize("which", ["A16W4_MXFP", "A16W8_MXFP", "A16W4_NVFP", "A8W4_MXFP", "A8W8_MXFP_post", "A8W8_MXFP_mx"])
def test_weight_only_and_mixed_block_scaled(lib, which):
    from gemlite_b200 import helper
    N, K, M = 512, 1024, 5
    x, W = _lin(80, N, K, torch.bfloat16, M=M)
    lin = torch.nn.Linear(K, N, bias=False, dtype=torch.bfloat16)
    lin.weight.data = W.clone()
    if which == "A16W4_MXFP":
        layer = helper.A16W4_MXFP(device="cuda:0", dtype=torch.bfloat16).from_linear(lin.cuda())
    elif which == "A16W8_MXFP":
        layer = helper.A16W8_MXFP(device="cuda:0", dtype=torch.bfloat16).from_linear(lin.cuda())
    elif which == "A16W4_NVFP":
        layer = helper.A16W4_NVFP(device="cuda:0", dtype=torch.bfloat16).from_linear(lin.cuda())
    elif which == "A8W4_MXFP":
        layer = helper.A8W4_MXFP_dynamic(device="cuda:0", dtype=torch.bfloat16, post_scale=False).from_linear(lin.cuda())
    elif which == "A8W8_MXFP_post":
        layer = helper.A8W8_MXFP_dynamic(device="cuda:0", dtype=torch.bfloat16, post_scale=True).from_linear(lin.cuda())
    else:
        layer = helper.A8W8_MXFP_dynamic(device="cuda:0", dtype=torch.bfloat16, post_scale=False).from_linear(lin.cuda())
    y = layer(x.cuda()).float().cpu().numpy()
    want = (x.double() @ W.double().T).numpy()
    tol = 0.2 if "W4" in which else 0.06
    assert rel_fro(y, want) < tol, (which, rel_fro(y, want))
