"""GPU: A16Wn (group-wise integer weights, fp16 / bf16 activations) through GemLiteLinear and the C
ABI, against the fp64 oracle.  Tolerance: relative Frobenius error <= 1e-2 (the bound stated for
fp16 / bf16 outputs); the kernels normally sit near 2e-3, the rounding of a bf16 output."""
import numpy as np
import pytest
import torch

from oracle import oracle
from tests.util import make_a16wn, exact_a16wn, rel_fro

pytestmark = pytest.mark.gpu
TOL = 1e-2


def build_layer(W_q, scales, zeros, bias, nbits, group_size, dtype):
    from gemlite_b200 import helper
    proc = helper.A16Wn_HQQ_INT(device="cuda:0", dtype=dtype, W_nbits=nbits)
    return proc.from_weights(W_q.cuda(), scales.cuda(), zeros.cuda(), bias=None if bias is None else bias.cuda())


@pytest.mark.parametrize("nbits,gs", [(4, 128), (2, 64), (1, 128), (4, 64), (4, 32), (8, 128)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_decode_sizes_match_oracle(lib, nbits, gs, dtype):
    # the reference's own test shape (tests/test_int.py:32, 40-41): N = 2032, K = 3968 = 31 * 128
    N, K = 2032, 3968
    from gemlite_b200 import core
    for M in (1, 3, 5, 16, 30):
        x, W_q, s, z, b = make_a16wn(N, K, nbits, gs, dtype, seed=1000 + M + nbits, M=M)
        layer = build_layer(W_q, s, z, b, nbits, gs, dtype)
        assert (layer.W_group_mode, layer.channel_scale_mode) == (4, 0)
        assert layer.W_q.dtype == torch.int32 and layer.W_q.shape == (K * nbits // 32, N)
        y = layer(x.cuda()).float().cpu().numpy()
        want = exact_a16wn(x, W_q, s, z, b, gs)
        assert y.shape == (M, N)
        assert rel_fro(y, want) < TOL, (M, nbits, rel_fro(y, want))
        # the general kernel and the streaming kernel agree with each other at least as well
        core.set_kernel_override(1)
        try:
            y_gen = layer(x.cuda()).float().cpu().numpy()
        finally:
            core.set_kernel_override(0)
        assert rel_fro(y_gen, want) < TOL
        # every family name is addressable and gives the same result for a decode size
        for fam in ("GEMV", "GEMV_REVSPLITK", "GEMV_SPLITK", "GEMM_SPLITK", "GEMM"):
            yf = layer.forward_manual(x.cuda(), fam).float().cpu().numpy()
            assert rel_fro(yf, want) < TOL, fam


def test_streaming_kernel_is_the_one_that_runs(lib):
    import ctypes
    from gemlite_b200 import core, _lib
    x, W_q, s, z, b = make_a16wn(1024, 1024, 4, 128, torch.bfloat16, seed=5)
    layer = build_layer(W_q, s, z, b, 4, 128, torch.bfloat16)
    xs = x.cuda()
    out = torch.empty((1, 1024), dtype=torch.bfloat16, device="cuda")
    a = core._fill_args(xs, layer.bias, layer.W_q, layer.scales, layer.zeros, None, None, out, layer.get_meta_args(), -1)
    assert lib.gl_matmul_kernel_name(ctypes.byref(a)) in (b"gl_gemv_stream_kernel", b"gl_gemv_warp_kernel")
    assert lib.gl_matmul_workspace_bytes(ctypes.byref(a)) > 0
    # too small a workspace is an error, not a silent fallback
    a.workspace, a.workspace_bytes = None, 0
    assert lib.gl_matmul(ctypes.byref(a), None) == _lib.GL_E_WORKSPACE


def test_deterministic_and_workspace_reuse(lib):
    # split-K partial sums are added in slice order: two runs give identical bits, also when another
    # shape used the same workspace in between.
    x, W_q, s, z, b = make_a16wn(4096, 4096, 4, 128, torch.bfloat16, seed=9, M=4)
    layer = build_layer(W_q, s, z, b, 4, 128, torch.bfloat16)
    x2, W_q2, s2, z2, b2 = make_a16wn(512, 2048, 2, 64, torch.bfloat16, seed=10, M=2)
    layer2 = build_layer(W_q2, s2, z2, b2, 2, 64, torch.bfloat16)
    y1 = layer(x.cuda()).clone()
    _ = layer2(x2.cuda())
    y2 = layer(x.cuda())
    assert torch.equal(y1, y2)


@pytest.mark.parametrize("mode", ["sym", "shift_scalar", "asym_nofma", "channelwise_post", "channelwise_pre", "no_meta"])
def test_mode_matrix(lib, mode):
    # W_group_mode / channel_scale_mode combinations pack() and the helpers select (core.py:646-703,
    # helper.py:260-266), each against the fp64 formula it stands for
    from gemlite_b200 import GemLiteLinear, DType
    N, K, gs, nbits = 512, 1024, 128, 4
    g = torch.Generator().manual_seed(77)
    x = torch.randn(3, K, generator=g).to(torch.float16)
    W_q = torch.randint(0, 15, (N, K), generator=g, dtype=torch.int32).to(torch.uint8)
    s = (torch.randn(N * (K // gs), 1, generator=g).abs() * 0.02).to(torch.float16)
    z = torch.randint(0, 15, (N * (K // gs), 1), generator=g).to(torch.float16)
    Wd, G = W_q.double(), K // gs
    layer = GemLiteLinear(nbits, gs if "channelwise" not in mode else K, K, N, DType.FP16, DType.FP16)
    if mode == "sym":
        layer.pack(W_q.cuda(), s.cuda(), None)
        want_modes, W = (2, 0), (Wd.view(N, G, gs) * s.double().view(N, G, 1)).view(N, K)
    elif mode == "shift_scalar":
        layer.pack(W_q.cuda(), s.cuda(), 7)
        want_modes, W = (3, 0), ((Wd - 7).view(N, G, gs) * s.double().view(N, G, 1)).view(N, K)
    elif mode == "asym_nofma":
        layer.pack(W_q.cuda(), s.cuda(), z.cuda(), fma_mode=False)
        want_modes, W = (3, 0), ((Wd.view(N, G, gs) - z.double().view(N, G, 1)) * s.double().view(N, G, 1)).view(N, K)
    elif mode == "channelwise_post":
        sc, zc = s[:N], z[:N]
        layer.pack(W_q.cuda(), sc.cuda(), zc.cuda())
        want_modes, W = (1, 1), (Wd - zc.double()) * sc.double()
    elif mode == "channelwise_pre":
        sc, zc = s[:N], z[:N]
        layer.pack(W_q.cuda(), sc.cuda(), zc.cuda())
        layer.W_group_mode, layer.channel_scale_mode = 3, 0     # what helper.A16Wn does for post_scale=False
        want_modes, W = (3, 0), (Wd - zc.double()) * sc.double()
    else:
        layer.pack(W_q.cuda(), None, None)
        want_modes, W = (0, 0), Wd
    assert (layer.W_group_mode, layer.channel_scale_mode) == want_modes
    y = layer(x.cuda()).float().cpu().numpy()
    want = (x.double() @ W.T).numpy()
    assert rel_fro(y, want) < TOL, (mode, rel_fro(y, want))


def test_packing_widths_and_fp32_output(lib):
    from gemlite_b200 import GemLiteLinear, DType
    N, K, gs = 256, 512, 64
    x, W_q, s, z, b = make_a16wn(N, K, 4, gs, torch.float16, seed=31, M=2)
    want = exact_a16wn(x, W_q, s, z, b, gs)
    for pb, wdt in ((8, torch.uint8), (16, torch.int16), (32, torch.int32)):
        layer = GemLiteLinear(4, gs, K, N, DType.FP16, DType.FP32)
        layer.pack(W_q.cuda(), s.cuda(), z.cuda(), bias=b.cuda(), packing_bitwidth=pb)
        assert layer.W_q.dtype == wdt
        y = layer(x.cuda())
        assert y.dtype == torch.float32
        assert rel_fro(y.cpu().numpy(), want) < TOL


def test_full_size_linearity(lib):
    # 8192 x 8192 (the benchmark layer), too large for a quick CPU oracle: check linearity in x,
    # y(a*x1 + x2) = a*y(x1) + y(x2) up to output rounding, and a sampled set of columns against fp64.
    N = K = 8192
    x, W_q, s, z, b = make_a16wn(N, K, 4, 128, torch.bfloat16, seed=2, M=2, with_bias=False)
    layer = build_layer(W_q, s, z, None, 4, 128, torch.bfloat16)
    xs = x.cuda()
    y = layer(xs).float()
    x3 = (2.0 * xs[0:1].float() + xs[1:2].float()).to(torch.bfloat16)
    y3 = layer(x3).float()
    # x3 is rounded to bf16, so compare against the layer applied to the rounded input only through linearity in fp64
    cols = torch.arange(0, N, 97)
    Wc = ((W_q[cols].double().view(len(cols), -1, 128) - z.view(N, -1)[cols].double()[..., None]) * s.view(N, -1)[cols].double()[..., None]).view(len(cols), K)
    want = (x.double() @ Wc.T).numpy()
    assert rel_fro(y[:, cols.cuda()].cpu().numpy(), want) < TOL
    want3 = (x3.cpu().double() @ Wc.T).numpy()
    assert rel_fro(y3[:, cols.cuda()].cpu().numpy(), want3) < TOL


def test_input_validation(lib):
    from gemlite_b200 import GemLiteLinear, DType
    with pytest.raises(NotImplementedError):
        GemLiteLinear(3, 64, 128, 128)
    with pytest.raises(NotImplementedError):
        GemLiteLinear(4, 8, 128, 128)
    with pytest.raises(NotImplementedError):
        GemLiteLinear(4, 64, 100, 128)
    layer = GemLiteLinear(4, 64, 128, 64, DType.FP16, DType.FP16)
    with pytest.raises(Exception):
        layer.pack(torch.zeros(64, 128, dtype=torch.int32).cuda(), None, None)    # not a packable dtype
    x, W_q, s, z, b = make_a16wn(64, 128, 4, 64, torch.float16, seed=3)
    layer.pack(W_q.cuda(), s.cuda(), z.cuda())
    with pytest.raises(RuntimeError):
        layer(x)                                                                  # CPU activations: no CPU path
    y = layer(x.cuda().view(1, 1, 128))                                           # N-D input keeps its leading dims
    assert y.shape == (1, 1, 64)
    assert layer(torch.empty(0, 128, dtype=torch.float16, device="cuda")).shape == (0, 64)


@pytest.mark.parametrize("N,K", [(1024, 28672), (8192, 3584), (1280, 8192), (8192, 1024)])
@pytest.mark.parametrize("M", [1, 4, 8, 16])
def test_decode_kernel_covers_llama_shard_shapes(lib, M, N, K):
    """Per-GPU shapes of Llama-70B linears under tensor parallelism.  K = 28672: the staged activations of a whole K
    range no longer fit one CTA for M >= 4, so the planner widens the CTA's column groups / adds cluster slices.
    K = 3584 = 112 iterations: 7 slices of 16 iterations (no power-of-two split fills the machine).  K = 1024: 4 slices."""
    import ctypes
    from gemlite_b200 import core
    x, W_q, s, z, b = make_a16wn(N, K, 4, 128, torch.bfloat16, seed=300 + M, M=M)
    layer = build_layer(W_q, s, z, b, 4, 128, torch.bfloat16)
    xs = x.cuda()
    y = layer(xs).float().cpu().numpy()
    assert rel_fro(y, exact_a16wn(x, W_q, s, z, b, 128)) < TOL
    out = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    a = core._fill_args(xs, layer.bias, layer.W_q, layer.scales, layer.zeros, None, None, out, layer.get_meta_args(), -1)
    # at M = 16, K = 28672 the 16 x 3584 activations of a cluster slice plus the per-group constants exceed one CTA: general kernel
    want_name = (b"gl_gemv_warp_kernel",) if (M <= 8 or K < 28672) else (b"gl_gemv_warp_kernel", b"gl_gemv_stream_kernel")
    assert lib.gl_matmul_kernel_name(ctypes.byref(a)) in want_name


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M", [1, 3, 8, 16])
def test_decode_kernel_packed_8bit(lib, M, dtype):
    """Packed 8-bit group-wise weights (A16W8 HQQ) at decode sizes on the warp-independent kernel: a word holds 4 k, and
    for bf16 (7 mantissa bits) every byte enters the MMA as its low 7 bits and its top bit separately."""
    import ctypes
    from gemlite_b200 import core
    N, K = 2048, 4096
    x, W_q, s, z, b = make_a16wn(N, K, 8, 128, dtype, seed=800 + M, M=M)
    layer = build_layer(W_q, s, z, b, 8, 128, dtype)
    xs = x.cuda()
    y = layer(xs).float().cpu().numpy()
    assert rel_fro(y, exact_a16wn(x, W_q, s, z, b, 128)) < TOL
    out = torch.empty((M, N), dtype=dtype, device="cuda")
    a = core._fill_args(xs, layer.bias, layer.W_q, layer.scales, layer.zeros, None, None, out, layer.get_meta_args(), -1)
    assert lib.gl_matmul_kernel_name(ctypes.byref(a)) == b"gl_gemv_warp_kernel"


@pytest.mark.parametrize("nbits,gs", [(4, 128), (2, 64)])
@pytest.mark.parametrize("M", [1, 3, 12])
def test_decode_bf16_activations_wide_range(lib, nbits, gs, M):
    """bf16 activations far outside the fp16 range in one batch row (up to ~1e6) next to ordinary rows and tiny values
    (1e-30): the decode kernel multiplies in the activation dtype and accumulates in fp32, so every row still agrees
    with fp64 at the usual tolerance (a kernel that went through fp16 would overflow here)."""
    from gemlite_b200 import helper
    N, K = 2048, 4096
    x, W_q, s, z, b = make_a16wn(N, K, nbits, gs, torch.bfloat16, seed=31 + M, M=M)
    x = x.float()
    x[0] *= 3.0e5
    x[0, ::7] = 1e-30
    if M > 1:
        x[1, 100:200] *= 1.0e4          # one K slice of another row
    x = x.to(torch.bfloat16)
    layer = helper.A16Wn_HQQ_INT(device="cuda:0", dtype=torch.bfloat16, W_nbits=nbits).from_weights(W_q.cuda(), s.cuda(), z.cuda(), bias=b.cuda())
    from tests.test_gpu_tc import _kernel_name
    assert _kernel_name(layer, x.cuda()) == "gl_gemv_warp_kernel"
    y = layer(x.cuda()).float().cpu().numpy()
    assert np.isfinite(y).all()
    want = exact_a16wn(x, W_q, s, z, b, gs)
    for m in range(M):                   # row by row: the rows differ by orders of magnitude
        assert rel_fro(y[m], want[m]) < 1e-2, (m, rel_fro(y[m], want[m]))


@pytest.mark.parametrize("nbits,gs", [(4, 32), (4, 128), (2, 64), (8, 128)])
@pytest.mark.parametrize("M", [17, 25, 32])
def test_decode_kernel_up_to_32_rows(lib, nbits, gs, M):
    """17 to 32 batch rows: the tensor-core kernel (operands swapped) where it covers the problem; groups of 32, which it
    does not take, run as two launches of the warp-independent streaming kernel (rows 0..15, then the rest)."""
    from gemlite_b200 import helper
    from tests.test_gpu_tc import _kernel_name
    for N, K in ((2048, 4096), (8192, 1024)):
        x, W_q, s, z, b = make_a16wn(N, K, nbits, gs, torch.bfloat16, seed=800 + M + nbits, M=M)
        layer = helper.A16Wn_HQQ_INT(device="cuda:0", dtype=torch.bfloat16, W_nbits=nbits).from_weights(W_q.cuda(), s.cuda(), z.cuda(), bias=b.cuda())
        assert _kernel_name(layer, x.cuda()) == ("gl_gemv_warp_kernel" if gs == 32 else "gl_gemm_tc_kernel")
        y = layer(x.cuda()).float().cpu().numpy()
        want = exact_a16wn(x, W_q, s, z, b, gs)
        assert rel_fro(y, want) < 1e-2, (N, K, rel_fro(y, want))
        for m in (0, M - 1):
            assert rel_fro(y[m], want[m]) < 1e-2
