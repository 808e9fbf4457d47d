"""GPU: the tcgen05 tensor-core kernels (prefill sizes) through GemLiteLinear and the C ABI, against the
fp64 oracle: A16Wn with in-kernel dequantisation, FP8 / INT8 with channel scales, MXFP4 / NVFP4 block-scaled.
Shapes include the reference's test shapes with ragged tiles (N = 2032, K = 3968; K = 4224 = 16.5 fp4 tiles).
Tolerances: relative Frobenius 1e-2 (16-bit paths) against the fp64 formula, 5e-3 against the oracle fed with
the identical quantised operands (FP8 / FP4 paths)."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import oracle
from tests.util import make_a16wn, exact_a16wn, rel_fro

pytestmark = pytest.mark.gpu


def _kernel_name(layer, x):
    from gemlite_b200 import core, _lib
    out = torch.empty((x.shape[0], layer.out_features), dtype=x.dtype, device="cuda")
    a = core._fill_args(x, layer.bias, layer.W_q, layer.scales, layer.zeros, None, None, out, layer.get_meta_args(), -1)
    return _lib.lib().gl_matmul_kernel_name(ctypes.byref(a)).decode()


def _status_word():
    """Device status word of the workspace: non-zero when a bounded wait in a kernel gave up."""
    from gemlite_b200 import core
    return core.matmul_status("cuda:0", clear=False)


@pytest.mark.parametrize("nbits,gs", [(4, 128), (2, 64), (1, 128), (4, 64), (8, 128)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_a16wn_prefill_ragged(lib, nbits, gs, dtype):
    from gemlite_b200 import helper
    N, K = 2032, 3968
    for M in (33, 64, 65, 130, 250):
        x, W_q, s, z, b = make_a16wn(N, K, nbits, gs, dtype, seed=3000 + M + nbits, M=M)
        layer = helper.A16Wn_HQQ_INT(device="cuda:0", dtype=dtype, W_nbits=nbits).from_weights(W_q.cuda(), s.cuda(), z.cuda(), bias=b.cuda())
        assert _kernel_name(layer, x.cuda()) == "gl_gemm_tc_kernel"
        y = layer(x.cuda()).float().cpu().numpy()
        assert _status_word() == 0
        want = exact_a16wn(x, W_q, s, z, b, gs)
        assert rel_fro(y, want) < 1e-2, (M, nbits, rel_fro(y, want))


@pytest.mark.parametrize("nbits,gs", [(4, 128), (2, 64), (1, 128), (8, 128)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_a16wn_swapped_operands_small_batches(lib, nbits, gs, dtype):
    """At most 64 rows run with the operands swapped (32 or 64 token columns).  The library sends up to 32 rows to the
    streaming kernel, so those sizes are forced onto the tensor-core kernel here (kernel_override = 2)."""
    from gemlite_b200 import core, helper
    core.set_kernel_override(2)
    try:
        for (N, K) in ((2032, 3968), (1024, 8192)):          # ragged channel tile with 31 K tiles; a split-K cluster
            for M in (1, 17, 32, 33, 47, 64):
                x, W_q, s, z, b = make_a16wn(N, K, nbits, gs, dtype, seed=3100 + M + nbits, M=M)
                layer = helper.A16Wn_HQQ_INT(device="cuda:0", dtype=dtype, W_nbits=nbits).from_weights(W_q.cuda(), s.cuda(), z.cuda(), bias=b.cuda())
                assert _kernel_name(layer, x.cuda()) == "gl_gemm_tc_kernel"
                y = layer(x.cuda())
                y2 = layer(x.cuda())
                assert _status_word() == 0
                assert torch.equal(y, y2)
                want = exact_a16wn(x, W_q, s, z, b, gs)
                assert rel_fro(y.float().cpu().numpy(), want) < 1e-2, (N, K, M, nbits, rel_fro(y.float().cpu().numpy(), want))
    finally:
        core.set_kernel_override(0)


@pytest.mark.parametrize("mode", ["sym", "shift_scalar", "asym_nofma", "channelwise_post", "no_meta"])
def test_a16wn_prefill_modes(lib, mode):
    from gemlite_b200 import GemLiteLinear, DType
    N, K, gs, nbits, M = 512, 1024, 128, 4, 96
    g = torch.Generator().manual_seed(78)
    x = torch.randn(M, K, generator=g).to(torch.float16)
    W_q = torch.randint(0, 15, (N, K), generator=g, dtype=torch.int32).to(torch.uint8)
    s = (torch.randn(N * (K // gs), 1, generator=g).abs() * 0.02).to(torch.float16)
    z = torch.randint(0, 15, (N * (K // gs), 1), generator=g).to(torch.float16)
    Wd, G = W_q.double(), K // gs
    layer = GemLiteLinear(nbits, gs if "channelwise" not in mode else K, K, N, DType.FP16, DType.FP16)
    if mode == "sym":
        layer.pack(W_q.cuda(), s.cuda(), None)
        W = (Wd.view(N, G, gs) * s.double().view(N, G, 1)).view(N, K)
    elif mode == "shift_scalar":
        layer.pack(W_q.cuda(), s.cuda(), 7)
        W = ((Wd - 7).view(N, G, gs) * s.double().view(N, G, 1)).view(N, K)
    elif mode == "asym_nofma":
        layer.pack(W_q.cuda(), s.cuda(), z.cuda(), fma_mode=False)
        W = ((Wd.view(N, G, gs) - z.double().view(N, G, 1)) * s.double().view(N, G, 1)).view(N, K)
    elif mode == "channelwise_post":
        layer.pack(W_q.cuda(), s[:N].cuda(), z[:N].cuda())
        W = (Wd - z[:N].double()) * s[:N].double()
    else:
        layer.pack(W_q.cuda(), None, None)
        W = Wd
    assert _kernel_name(layer, x.cuda()) == "gl_gemm_tc_kernel"
    y = layer(x.cuda()).float().cpu().numpy()
    assert _status_word() == 0
    assert rel_fro(y, (x.double() @ W.T).numpy()) < 1e-2, mode


def test_a16w4_full_size_sampled(lib):
    # the benchmark layer at M = 4096: compare 64 sampled output columns with fp64
    from gemlite_b200 import helper
    N = K = 8192
    x, W_q, s, z, b = make_a16wn(N, K, 4, 128, torch.bfloat16, seed=4, M=4096)
    layer = helper.A16W4_HQQ_INT(device="cuda:0", dtype=torch.bfloat16).from_weights(W_q.cuda(), s.cuda(), z.cuda(), bias=b.cuda())
    y = layer(x.cuda()).float()
    assert _status_word() == 0
    cols = torch.arange(5, N, 128)
    Wc = ((W_q[cols].double().view(len(cols), -1, 128) - z.view(N, -1)[cols].double()[..., None]) * s.view(N, -1)[cols].double()[..., None]).view(len(cols), K)
    want = (x.double() @ Wc.T + b[cols].double()).numpy()
    assert rel_fro(y[:, cols.cuda()].cpu().numpy(), want) < 1e-2


@pytest.mark.parametrize("fp8", [True, False])
@pytest.mark.parametrize("M", [1, 16, 65, 130, 300])
def test_a8w8_tensor_core(lib, fp8, M):
    from gemlite_b200 import helper
    N, K = 1000, 2048 + 64            # N not a multiple of the tile, K not a multiple of 128
    g = torch.Generator().manual_seed(90 + M)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    W = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16)
    lin = torch.nn.Linear(K, N, bias=True, dtype=torch.bfloat16)
    lin.weight.data = W.clone()
    bias = lin.bias.data.clone()
    proc = helper.A8W8_FP8_dynamic(device="cuda:0", dtype=torch.bfloat16) if fp8 else helper.A8W8_INT8_dynamic(device="cuda:0", dtype=torch.bfloat16)
    layer = proc.from_linear(lin.cuda())
    y = layer(x.cuda()).float().cpu().numpy()
    assert _status_word() == 0
    xq, sx = oracle.scale_activations_per_token(x.float().numpy(), "fp8" if fp8 else "int8")
    Wq = layer.W_q.t().contiguous().cpu()
    Xd = oracle.e4m3_decode(xq).astype(np.float64) if fp8 else xq.astype(np.float64)
    Wd = Wq.float().double().numpy() if fp8 else Wq.double().numpy()
    want_q = (Xd @ Wd.T) * sx.astype(np.float64) * layer.scales.cpu().double().numpy().reshape(1, -1) + bias.double().numpy()
    assert rel_fro(y, want_q) < 5e-3, rel_fro(y, want_q)


@pytest.mark.parametrize("N", [3976, 3968])
@pytest.mark.parametrize("nbits,gs", [(4, 128), (2, 64)])
def test_a16wn_partial_last_wave_runs_as_half_tiles(lib, N, nbits, gs):
    """11 x 16 = 176 tiles of 256 x 256 on 148 SMs: the 28 tiles of the last wave run as 56 halves of 128 columns in a
    second launch.  N = 3976: the last tile's right half has 8 columns; N = 3968: it has none.  Same bits as the single
    launch ("tail": 0 in the cache entry), and both against the dequantised product."""
    from gemlite_b200 import helper, _lib
    L = _lib.lib()
    if torch.cuda.get_device_properties(0).multi_processor_count != 148:
        pytest.skip("tile counts chosen for 148 SMs")
    K, M = 2048, 2560 + 37
    x, W_q, s, z, b = make_a16wn(N, K, nbits, gs, torch.bfloat16, seed=61, M=M)
    layer = helper.A16Wn_HQQ_INT(device="cuda:0", dtype=torch.bfloat16, W_nbits=nbits).from_weights(W_q.cuda(), s.cuda(), z.cuda(), bias=b.cuda())
    xd = x.cuda()
    y = layer(xd)
    assert _status_word() == 0 and _kernel_name(layer, xd) == "gl_gemm_tc_kernel"
    sig = "(%d, %d, %d, %d, %d, %d)" % (L.gl_get_closest_m(M), N, K, gs, 32 // nbits, 100 + nbits)
    try:
        assert L.gl_cfg_set(b"GEMM", sig.encode(), b'{"tail": 0}') == 0
        y1 = layer(xd)
    finally:
        L.gl_cfg_set(b"GEMM", sig.encode(), b'{"tail": 1}')
    assert torch.equal(y, y1)
    Wd = ((W_q.double().view(N, -1, gs) - z.view(N, -1).double()[..., None]) * s.view(N, -1).double()[..., None]).view(N, K)
    want = (x.double() @ Wd.T + b.double()).numpy()
    got = y.float().cpu().numpy()
    assert rel_fro(got, want) < 1e-2
    assert rel_fro(got[:, 3584:], want[:, 3584:]) < 1e-2 and rel_fro(got[-37:], want[-37:]) < 1e-2      # the half tiles, the ragged rows
    assert rel_fro(got[:, -8:], want[:, -8:]) < 1e-2


@pytest.mark.parametrize("M,cfg", [(2597, b'{}'), (2048, b'{"tail": 0}'), (2597, b'{"tail": 0, "tile_n": 128}')])
def test_a16wn_back_to_back_calls_are_bit_identical(lib, M, cfg):
    """Two accumulators per CTA make the MMAs, not the dequant warps, set the pace: the regime in which a packed-word
    slot handed back to its producer before the tile was unpacked gave wrong scale granules in 10-25 % of the calls.
    48 calls in a row (each overlapping the previous one's tail) must agree bit for bit, and with the dequantised product."""
    from gemlite_b200 import helper, _lib
    L = _lib.lib()
    N, K = 3976, 2048
    x, W_q, s, z, b = make_a16wn(N, K, 4, 128, torch.bfloat16, seed=62, M=M)
    layer = helper.A16W4_HQQ_INT(device="cuda:0", dtype=torch.bfloat16).from_weights(W_q.cuda(), s.cuda(), z.cuda(), bias=b.cuda())
    xd = x.cuda()
    sig = "(%d, %d, %d, 128, 8, 104)" % (L.gl_get_closest_m(M), N, K)
    try:
        assert L.gl_cfg_set(b"GEMM", sig.encode(), cfg) == 0
        outs = [layer(xd).clone() for _ in range(48)]
        torch.cuda.synchronize()
    finally:
        L.gl_cfg_set(b"GEMM", sig.encode(), b'{}')
    assert _status_word() == 0
    differing = [i for i, o in enumerate(outs) if not torch.equal(o, outs[0])]
    assert differing == [], differing
    Wd = ((W_q.double().view(N, -1, 128) - z.view(N, -1).double()[..., None]) * s.view(N, -1).double()[..., None]).view(N, K)
    want = (x.double() @ Wd.T + b.double()).numpy()
    got = outs[-1].float().cpu().numpy()
    assert rel_fro(got, want) < 1e-2
    # no 32-column block of any 256-row tile may stand out either (a wrong scale granule is invisible in the whole-matrix norm)
    err = np.abs(got - want)
    blk = err[: (M // 256) * 256, : (N // 32) * 32].reshape(M // 256, 256, N // 32, 32).mean(axis=(1, 3))
    assert blk.max() < 4 * np.median(blk) + 1e-3, (float(blk.max()), float(np.median(blk)))


@pytest.mark.parametrize("kind", ["fp8", "a16w4"])
def test_banded_tile_order_for_large_activations(lib, kind):
    """Activations of 64 MB and more switch the tile numbering to bands of 2048 rows (the last band short, the last row
    tile ragged): every band's rows and the last columns against the product of the identical operands."""
    from gemlite_b200 import helper, quant_utils as qu
    g = torch.Generator(device="cuda").manual_seed(97)
    if kind == "fp8":
        N, K, M = 520, 8192, 8192 + 2048 + 77              # 81 row tiles: five bands of 16 and one of 1
        x = torch.randn(M, K, generator=g, device="cuda", dtype=torch.bfloat16)
        lin = torch.nn.Linear(K, N, bias=False, dtype=torch.bfloat16, device="cuda")
        lin.weight.data.normal_(0, 0.02, generator=g)
        layer = helper.A8W8_FP8_dynamic(device="cuda:0", dtype=torch.bfloat16).from_linear(lin)
        y = layer(x).float()
        xq, sx = qu.scale_activations_per_token(x, torch.float8_e4m3fn)
        rows = torch.cat([torch.arange(0, M, 509, device="cuda"), torch.arange(M - 80, M, device="cuda")])
        want = (xq[rows].float() @ layer.W_q.float()) * sx[rows].view(-1, 1) * layer.scales.float().view(1, -1)
    else:
        N, K, M = 1024, 8192, 4096 + 300                    # 256-row tiles (two accumulators): bands of 8, 18 row tiles
        x0, W_q, s, z, b = make_a16wn(N, K, 4, 128, torch.bfloat16, seed=98, M=1)
        x = torch.randn(M, K, generator=g, device="cuda", dtype=torch.bfloat16)
        layer = helper.A16W4_HQQ_INT(device="cuda:0", dtype=torch.bfloat16).from_weights(W_q.cuda(), s.cuda(), z.cuda(), bias=b.cuda())
        y = layer(x).float()
        rows = torch.cat([torch.arange(0, M, 211, device="cuda"), torch.arange(M - 80, M, device="cuda")])
        Wd = ((W_q.double().view(N, -1, 128) - z.view(N, -1).double()[..., None]) * s.view(N, -1).double()[..., None]).view(N, K).float().cuda()
        want = x[rows].float() @ Wd.T + b.float().cuda()
    assert _status_word() == 0
    got = y[rows]
    assert float((got - want).norm() / want.norm()) < (5e-3 if kind == "fp8" else 1e-2)
    assert float((got[:, -40:] - want[:, -40:]).norm() / want[:, -40:].norm()) < 1e-2
    assert float((got[-1] - want[-1]).norm() / want[-1].norm()) < 1e-2


@pytest.mark.parametrize("fmt", ["mxfp4", "nvfp4"])
@pytest.mark.parametrize("M", [1, 16, 100, 300])
@pytest.mark.parametrize("N,K", [(2048, 4224), (384, 1024)])
def test_a4w4_tensor_core(lib, fmt, M, N, K):
    from gemlite_b200 import helper
    g = torch.Generator().manual_seed(170 + M)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    lin = torch.nn.Linear(K, N, bias=False, dtype=torch.bfloat16)
    lin.weight.data = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16)
    W = lin.weight.data.clone()
    proc = (helper.A4W4_MXFP_dynamic if fmt == "mxfp4" else helper.A4W4_NVFP_dynamic)(device="cuda:0", dtype=torch.bfloat16)
    layer = proc.from_linear(lin.cuda())
    gs = 32 if fmt == "mxfp4" else 16
    y = layer(x.cuda()).float().cpu().numpy()
    assert _status_word() == 0
    wq = layer.W_q.t().contiguous().cpu().numpy()
    sw = layer.scales.contiguous().view(torch.uint8).cpu().numpy()
    if fmt == "mxfp4":
        xq, sx = oracle.scale_activations_mxfp4(x.float().numpy())
        meta = None
    else:
        xq, sx, mx = oracle.scale_activations_nvfp4(x.float().numpy())
        meta = 1.0 / (float(layer.meta_scale.item()) * float(mx))
    want_q = oracle.matmul_mx(xq, sx, wq, sw, gs, meta_scale=meta)
    assert rel_fro(y, want_q) < 5e-3, rel_fro(y, want_q)
    # the general kernel gives the same result from the row-major scale layout
    from gemlite_b200 import core
    core.set_kernel_override(1)
    try:
        y2 = layer(x.cuda()).float().cpu().numpy()
    finally:
        core.set_kernel_override(0)
    assert rel_fro(y2, want_q) < 5e-3


def test_scale_atom_layout_matches_reference_shuffle(lib):
    # activation scales written as atoms == the reference's 5-D pre-shuffle of the row layout
    from gemlite_b200 import quant_utils as qu
    x = torch.randn(200, 1024, dtype=torch.bfloat16, device="cuda")
    q0, s0 = qu.scale_activations_mxfp4(x, scale_layout=0)
    q1, s1 = qu.scale_activations_mxfp4(x, scale_layout=1)
    assert torch.equal(q0, q1)
    rows = torch.full((256, 32), 127, dtype=torch.uint8, device="cuda")
    rows[:224] = s0
    want = rows.view(2, 4, 32, 8, 4).permute(0, 3, 2, 1, 4).reshape(2, 8, 512)
    assert torch.equal(s1, want)


def test_a16wn_split_k_is_deterministic_and_sized(lib):
    """Few-tile problems split K over the CTAs of a cluster; each CTA adds its share of the partial tiles in split
    order out of the cluster's shared memories, so two runs give identical bits and no workspace beyond the counter
    block is needed."""
    import ctypes
    from gemlite_b200 import core, helper
    N, K, M = 1024, 4096, 48
    x, W_q, s, z, b = make_a16wn(N, K, 4, 128, torch.bfloat16, seed=77, M=M)
    layer = helper.A16W4_HQQ_INT(device="cuda:0", dtype=torch.bfloat16).from_weights(W_q.cuda(), s.cuda(), z.cuda(), bias=b.cuda())
    xs = x.cuda()
    y1 = layer(xs).clone()
    y2 = layer(xs).clone()
    assert torch.equal(y1, y2)
    assert _status_word() == 0
    want = exact_a16wn(x, W_q, s, z, b, 128)
    assert rel_fro(y1.float().cpu().numpy(), want) < 1e-2
    out = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    a = core._fill_args(xs, layer.bias, layer.W_q, layer.scales, layer.zeros, None, None, out, layer.get_meta_args(), -1)
    assert lib.gl_matmul_kernel_name(ctypes.byref(a)) == b"gl_gemm_tc_kernel"
    need = lib.gl_matmul_workspace_bytes(ctypes.byref(a))
    assert need == lib.gl_matmul_counter_bytes()
    a.workspace, a.workspace_bytes = core._workspace(torch.device("cuda", 0), int(need)).data_ptr(), int(need) - 16
    from gemlite_b200 import _lib
    assert lib.gl_matmul(ctypes.byref(a), torch.cuda.current_stream().cuda_stream) == _lib.GL_E_WORKSPACE   # too small: an error, no fallback


@pytest.mark.parametrize("fmt", ["mxfp4", "nvfp4"])
def test_a4w4_256_column_tiles_with_replicated_scale_atoms(lib, fmt):
    """Enough tiles for the 256-column configuration: scale atoms arrive through the stride-0 tensor maps and are copied
    to TMEM two at a time; K ends in the middle of a K tile (missing atoms read as zero).  Compared with the general
    kernel (itself pinned to the oracle above) and, on sampled rows, with the oracle."""
    from gemlite_b200 import core, helper
    M, N, K = 1024, 3072, 1408
    g = torch.Generator().manual_seed(911)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    lin = torch.nn.Linear(K, N, bias=False, dtype=torch.bfloat16)
    lin.weight.data = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16)
    proc = (helper.A4W4_MXFP_dynamic if fmt == "mxfp4" else helper.A4W4_NVFP_dynamic)(device="cuda:0", dtype=torch.bfloat16)
    layer = proc.from_linear(lin.cuda())
    y = layer(x.cuda()).float()
    assert _status_word() == 0
    core.set_kernel_override(1)
    try:
        y_gen = layer(x.cuda()).float()
    finally:
        core.set_kernel_override(0)
    assert rel_fro(y.cpu().numpy(), y_gen.cpu().numpy()) < 2e-3
    rows = [0, 127, 128, 517, 1023]
    gs = 32 if fmt == "mxfp4" else 16
    wq = layer.W_q.t().contiguous().cpu().numpy()
    sw = layer.scales.contiguous().view(torch.uint8).cpu().numpy()
    if fmt == "mxfp4":
        xq, sx = oracle.scale_activations_mxfp4(x.float().numpy())
        meta = None
    else:
        xq, sx, mx = oracle.scale_activations_nvfp4(x.float().numpy())
        meta = 1.0 / (float(layer.meta_scale.item()) * float(mx))
    want = oracle.matmul_mx(xq[rows], sx[rows], wq, sw, gs, meta_scale=meta)
    assert rel_fro(y.cpu().numpy()[rows], want) < 5e-3
