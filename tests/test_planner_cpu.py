"""CPU: kernel selection and workspace sizing are host-only code in the library (no device call, pointers are never
dereferenced), so the planner can be swept over shapes without a GPU: it must not fail on any of them, and the shapes
of the benchmark configurations must land on the kernels built for them."""
import ctypes
import itertools

from gemlite_b200 import _lib
from gemlite_b200.dtypes import DType

FAKE = 0x7F0000000000        # 16-byte aligned, never dereferenced


def _args(M, N, K, nbits, gs, dtype=DType.BF16):
    a = _lib.GLMatmulArgs()
    for f in ("x", "w", "scales", "zeros", "out", "workspace"):
        setattr(a, f, FAKE)
    a.workspace_bytes = 1 << 30
    a.M, a.N, a.K, a.W_nbits, a.group_size, a.elements_per_sample = M, N, K, nbits, gs, 32 // nbits
    a.input_dtype = a.x_dtype = a.out_dtype = a.meta_dtype = a.zeros_dtype = dtype.value
    a.w_dtype = DType.INT32.value
    a.W_group_mode, a.channel_scale_mode, a.matmul_type = 4, 0, -1
    a.w_stride_k, a.w_stride_n, a.s_stride_g, a.s_stride_n = N, 1, N, 1
    return a


def _plan(*shape):
    L = _lib.lib()
    a = _args(*shape)
    return L.gl_matmul_kernel_name(ctypes.byref(a)).decode(), int(L.gl_matmul_workspace_bytes(ctypes.byref(a)))


def test_planner_survives_a_sweep_of_shapes():
    L = _lib.lib()
    counter = int(L.gl_matmul_counter_bytes())
    names = set()
    for M, (N, K), (nbits, gs) in itertools.product(
            (1, 2, 3, 4, 8, 9, 16, 17, 32, 33, 64, 200, 4096),
            ((8192, 8192), (2032, 3968), (1024, 28672), (8192, 3584), (1280, 8192), (8192, 1024), (32, 256), (4096, 128)),
            ((8, 128), (4, 128), (4, 64), (4, 32), (2, 64), (1, 128))):
        if K % gs:
            continue
        name, ws = _plan(M, N, K, nbits, gs)
        assert name.startswith("gl_"), (M, N, K, nbits, gs, name)
        assert ws >= counter or name == "gl_generic_kernel"      # the general kernel needs no workspace
        names.add(name)
    assert {"gl_gemv_warp_kernel", "gl_gemv_stream_kernel", "gl_gemm_tc_kernel"} <= names


def test_benchmark_shapes_land_on_their_kernels():
    for M in (1, 2, 4, 8, 16):
        assert _plan(M, 8192, 8192, 4, 128)[0] == "gl_gemv_warp_kernel"
        assert _plan(M, 8192, 8192, 2, 64)[0] == "gl_gemv_warp_kernel"
        assert _plan(M, 8192, 8192, 8, 128)[0] == "gl_gemv_warp_kernel"
    for M in (17, 32, 33, 64, 256, 1024, 4096, 8192):
        assert _plan(M, 8192, 8192, 4, 128)[0] == "gl_gemm_tc_kernel"
    # Llama-70B shard shapes at decode size
    for N, K in ((8192, 3584), (1280, 8192), (8192, 1024), (7168, 8192)):
        assert _plan(1, N, K, 4, 128)[0] == "gl_gemv_warp_kernel"
    # the tensor-core kernels need the counter block only: K splits are summed inside a cluster, not through a workspace
    counter = int(_lib.lib().gl_matmul_counter_bytes())
    assert _plan(64, 8192, 8192, 4, 128)[1] == counter
    assert _plan(4096, 8192, 8192, 4, 128)[1] == counter


def test_weight_only_decode_kernels_are_selected():
    """Unpacked 8-bit weights with one scale per channel and weight-only block-scaled fp4 / fp8 at 1..4 rows go to the
    streaming decode kernels of their own; more rows stay on the general kernel."""
    L = _lib.lib()

    def name(M, N, K, w_dtype, nbits, e, gs, input_dtype, wgm, csm, w_stride_n):
        a = _args(M, N, K, 4, 128)
        a.W_nbits, a.elements_per_sample, a.group_size = nbits, e, gs
        a.w_dtype, a.input_dtype = w_dtype.value, input_dtype.value
        a.W_group_mode, a.channel_scale_mode = wgm, csm
        a.w_stride_k, a.w_stride_n = 1, w_stride_n
        a.meta_dtype = DType.FP32.value
        return L.gl_matmul_kernel_name(ctypes.byref(a)).decode()

    for M, want8, want4 in ((1, "gl_w8_gemv_kernel", "gl_w4mx_gemv_kernel"), (4, "gl_w8_gemv_kernel", "gl_w4mx_gemv_kernel"),
                            (5, "gl_generic_kernel", "gl_generic_kernel")):
        assert name(M, 8192, 8192, DType.INT8, 8, 1, 8192, DType.BF16, 2, 0, 8192) == want8          # A16W8_INT8, scale on the weights
        assert name(M, 2032, 3968, DType.FP8, 8, 1, 3968, DType.BF16, 0, 1, 3968) == want8           # A16W8_FP8, scale on the sums
        assert name(M, 4096, 8192, DType.FP8, 8, 1, 32, DType.MXBF16, 0, 0, 8192) == want8           # A16W8_MXFP
        assert name(M, 4096, 8192, DType.UINT8, 4, 2, 32, DType.MXBF16, 0, 0, 4096) == want4         # A16W4_MXFP
        assert name(M, 4096, 8192, DType.UINT8, 4, 2, 16, DType.NVFP4, 0, 0, 4096) == want4          # A16W4_NVFP
    # grouped zeros or a K that is not a multiple of 16 bytes are not what these kernels take
    assert name(1, 8192, 8192, DType.INT8, 8, 1, 128, DType.BF16, 4, 0, 8192) == "gl_generic_kernel"
    assert name(1, 512, 1000, DType.INT8, 8, 1, 1000, DType.BF16, 2, 0, 1000) == "gl_generic_kernel"


def test_quantised_activation_paths_are_selected():
    """FP8 / INT8 with channel scales or 128 x 128 block scales, and MXFP8 weights with block-scaled or per-token
    activations, go to the tensor-core kernels at every batch size; what they cannot take stays on the general kernel."""
    L = _lib.lib()

    def name(M, N, K, dt, csm, input_dtype=None, group=None, atoms=True, sx_layout=0, meta=DType.FP32):
        a = _args(M, N, K, 8, K if group is None else group)
        a.elements_per_sample = 1
        a.w_dtype = a.x_dtype = dt.value
        a.input_dtype = (dt if input_dtype is None else input_dtype).value
        a.W_group_mode, a.channel_scale_mode = 0, csm
        a.w_stride_k, a.w_stride_n = 1, K
        a.meta_dtype = meta.value
        a.scales_x = FAKE
        a.sx_layout = sx_layout
        a.w_scales_atoms = FAKE if atoms else None
        a.s_stride_g, a.s_stride_n = (N + 127) // 128, 1
        return L.gl_matmul_kernel_name(ctypes.byref(a)).decode()

    for M in (1, 16, 17, 64, 300, 4096):
        for dt in (DType.FP8, DType.INT8):
            assert name(M, 14336, 4096, dt, 3) == "gl_gemm_tc_kernel"                    # per-token x per-channel scales
            assert name(M, 8192, 8192, dt, 5) == "gl_gemm_tc_kernel"                     # 128 x 128 block scales
        assert name(M, 8192, 8192, DType.FP8, 4, DType.MXFP8, 32, sx_layout=1) == "gl_gemm_tc_kernel"   # MXFP8 x MXFP8
        assert name(M, 8192, 8192, DType.FP8, 2, DType.MXFP8, 32) == "gl_gemm_tc_kernel"                # MXFP8 weights, per-token x
    # block scales that are not fp32, a K that is not a multiple of 128, MXFP8 without the scale atoms
    assert name(64, 8192, 8192, DType.FP8, 5, meta=DType.BF16) == "gl_generic_kernel"
    assert name(64, 8192, 4160, DType.FP8, 5) == "gl_generic_kernel"
    assert name(64, 8192, 8192, DType.FP8, 2, DType.MXFP8, 32, atoms=False) == "gl_generic_kernel"
