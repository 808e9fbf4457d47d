"""GPU: the layer configurations that the reference's own layer tests build by hand (tests/test_int.py:99-340), on its
shape (N = 2032, K = 3968 = 31 groups of 128), its batch sizes and all five matmul families through `forward_manual`,
with its criterion: mean absolute error against the torch product below the tolerance written beside each case
(tests/test_int.py:96-97), and its assertions on the modes `pack()` derives.  Data recipe as there: codes 0..14, scales
0.001, zeros chosen so that the dequantised weights are e4m3-representable."""
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
N, K, NBITS, GS = 2032, 3968, 4, 128
BATCHES = [1, 3, 5, 16, 30, 65, 100, 250]
FAMILIES = ["GEMV_REVSPLITK", "GEMV", "GEMV_SPLITK", "GEMM_SPLITK", "GEMM"]
CD = torch.bfloat16
FP8 = torch.float8_e4m3fn


@pytest.fixture(scope="module")
def data(lib):
    g = torch.Generator(device=DEV).manual_seed(0)
    W_q = torch.randint(0, 2 ** NBITS - 1, (N, K), generator=g, device=DEV).to(torch.uint8)
    n_groups = W_q.numel() // GS
    scales = torch.full((n_groups, 1), 0.001, device=DEV, dtype=CD)
    z0 = torch.zeros((n_groups, 1), device=DEV, dtype=CD)
    W = ((W_q.reshape(-1, GS) - z0) * scales).to(FP8).to(CD)
    zeros = torch.mean(W_q.reshape(-1, GS).float() - (W / scales).float(), dim=1, keepdim=True).to(CD)
    W = ((W_q.reshape(-1, GS).to(CD) - zeros) * scales).reshape(N, K)
    xs = {}
    for M in BATCHES:
        gx = torch.Generator(device=DEV).manual_seed(M)
        xs[M] = torch.randn((M, K), generator=gx, dtype=CD, device=DEV) / 10.0
    return W, W_q, scales, zeros, xs


def _check(layer, ref_fn, tol, inputs):
    for M in BATCHES:
        x = inputs(M)
        want = ref_fn(x).float()
        for fam in FAMILIES:
            if M > 4 and "GEMV" in fam:
                continue
            got = layer.forward_manual(x, matmul_type=fam).float()
            assert got.shape == want.shape
            err = (want - got).abs().mean().item()
            assert err < tol, (fam, M, err, tol)
        got = layer(x).float()                                  # the automatic choice too
        assert (want - got).abs().mean().item() < tol, ("auto", M)


def _layer(nbits, gs, input_dtype, output_dtype, scaled):
    from gemlite_b200 import GemLiteLinear
    return GemLiteLinear(nbits, group_size=gs, in_features=K, out_features=N, input_dtype=input_dtype,
                         output_dtype=output_dtype, scaled_activations=scaled)


def test_fp16_weights(lib, data):                               # tests/test_int.py:99-118
    from gemlite_b200.dtypes import DType, TORCH_TO_DTYPE
    W, _, _, _, xs = data
    layer = _layer(16, None, TORCH_TO_DTYPE[CD], TORCH_TO_DTYPE[CD], False)
    layer.pack(W, None, None, None)
    assert layer.W_group_mode == 0 and layer.channel_scale_mode == 0
    _check(layer, lambda x: x @ W.T, 2.5e-3, lambda M: xs[M])


def test_16bit_times_packed_asymmetric(lib, data):              # tests/test_int.py:120-144
    from gemlite_b200.dtypes import TORCH_TO_DTYPE
    W, W_q, scales, zeros, xs = data
    layer = _layer(NBITS, GS, TORCH_TO_DTYPE[CD], TORCH_TO_DTYPE[CD], False)
    layer.pack(W_q, scales, zeros, None)
    assert layer.W_group_mode in (3, 4) and layer.channel_scale_mode == 0
    _check(layer, lambda x: x @ W.T, 2.5e-3, lambda M: xs[M])


def test_int8_times_packed_shift_only(lib, data):               # tests/test_int.py:146-171
    from gemlite_b200 import DType
    _, W_q, _, _, _ = data
    layer = _layer(NBITS, GS, DType.INT8, DType.FP32, False)
    g = torch.Generator(device=DEV).manual_seed(11)
    s = torch.randn((N, 1), generator=g, dtype=CD, device=DEV) * 1e-4
    layer.pack(W_q, scales=s, zeros=7, bias=None)
    assert layer.W_group_mode == 1 and layer.channel_scale_mode == 1

    def inputs(M):
        gx = torch.Generator(device=DEV).manual_seed(100 + M)
        return torch.randint(-10, 10, (M, K), generator=gx, device=DEV).to(torch.int8)

    _check(layer, lambda x: x.to(CD) @ ((W_q.to(CD) - 7) * s).T, 1e-3, inputs)


def test_int8_times_packed_scaled_activations(lib, data):       # tests/test_int.py:173-199
    from gemlite_b200 import DType
    from gemlite_b200.quant_utils import scale_activations_per_token_torch
    _, W_q, _, _, _ = data
    layer = _layer(NBITS, GS, DType.INT8, DType.FP32, True)
    layer.pack(W_q, scales=None, zeros=7, bias=None)
    layer.meta_dtype = DType.FP32
    assert layer.W_group_mode == 1 and layer.channel_scale_mode == 2

    def inputs(M):
        gx = torch.Generator(device=DEV).manual_seed(200 + M)
        return torch.randn((M, K), generator=gx, dtype=torch.float16, device=DEV) / 20.0

    def ref(x):
        xq, sx = scale_activations_per_token_torch(x, w_dtype=torch.int8)
        return (xq.to(torch.float16) @ (W_q.to(torch.float16) - 7).T) * sx

    _check(layer, ref, 7e-3, inputs)


def test_int8_codes_scaled_weights_and_activations(lib, data):  # tests/test_int.py:201-224
    from gemlite_b200 import DType
    from gemlite_b200.quant_utils import scale_activations_per_token_torch
    _, W_q, _, _, xs = data
    layer = _layer(8, K, DType.INT8, DType.FP32, True)
    g = torch.Generator(device=DEV).manual_seed(12)
    s = torch.randn((N, 1), generator=g, dtype=CD, device=DEV) * 1e-4
    layer.pack(W_q, scales=s, zeros=7, bias=None)
    assert layer.W_group_mode == 1 and layer.channel_scale_mode == 3

    def ref(x):
        xq, sx = scale_activations_per_token_torch(x, w_dtype=torch.int8)
        return (xq.to(CD) @ ((W_q.to(CD) - 7) * s).T) * sx

    _check(layer, ref, 1e-3, lambda M: xs[M])


def test_fp8_times_fp8_unscaled(lib, data):                     # tests/test_int.py:227-252
    from gemlite_b200.dtypes import TORCH_TO_DTYPE
    W, _, _, _, _ = data
    layer = _layer(8, None, TORCH_TO_DTYPE[FP8], TORCH_TO_DTYPE[CD], False)
    layer.pack(W.to(FP8), None, None, None)
    assert layer.W_group_mode == 0 and layer.channel_scale_mode == 0

    def inputs(M):
        gx = torch.Generator(device=DEV).manual_seed(300 + M)
        return (torch.randn((M, K), generator=gx, dtype=CD, device=DEV) / 10.0).to(FP8)

    _check(layer, lambda x: x.to(CD) @ W.T, 5e-3, inputs)


def test_fp8_times_fp8_scaled_weights_and_activations(lib, data):   # tests/test_int.py:254-278
    from gemlite_b200.dtypes import TORCH_TO_DTYPE
    from gemlite_b200.quant_utils import scale_activations_per_token_torch
    W, _, _, _, xs = data
    layer = _layer(8, K, TORCH_TO_DTYPE[FP8], TORCH_TO_DTYPE[CD], True)
    g = torch.Generator(device=DEV).manual_seed(13)
    s = torch.randn((1, N), generator=g, dtype=CD, device=DEV) * 1e-4
    layer.pack(W.to(FP8), scales=s, zeros=None, bias=None)
    assert layer.W_group_mode == 0 and layer.channel_scale_mode == 3

    def ref(x):
        xq, sx = scale_activations_per_token_torch(x, w_dtype=FP8)
        return (xq.to(CD) @ W.T) * (s * sx)

    _check(layer, ref, 5e-3, lambda M: xs[M])


def test_fp8_times_packed_scaled_activations(lib, data):        # tests/test_int.py:280-309
    from gemlite_b200.dtypes import TORCH_TO_DTYPE
    from gemlite_b200.quant_utils import scale_activations_per_token_torch
    W, W_q, scales, zeros, _ = data
    layer = _layer(NBITS, GS, TORCH_TO_DTYPE[FP8], TORCH_TO_DTYPE[CD], True)
    layer.pack(W_q, scales, zeros, None)
    assert layer.W_group_mode in (3, 4) and layer.channel_scale_mode == 2

    def inputs(M):
        gx = torch.Generator(device=DEV).manual_seed(400 + M)
        return (torch.randn((M, K), generator=gx, dtype=CD, device=DEV) / 10.0).to(FP8).to(CD)

    def ref(x):
        xq, sx = scale_activations_per_token_torch(x, w_dtype=FP8)
        return (xq.to(CD) @ W.T) * sx

    _check(layer, ref, 5e-3, inputs)


def test_fp8_times_packed_unscaled(lib, data):                  # tests/test_int.py:312-340
    from gemlite_b200.dtypes import TORCH_TO_DTYPE
    W, W_q, scales, zeros, _ = data
    layer = _layer(NBITS, GS, TORCH_TO_DTYPE[FP8], TORCH_TO_DTYPE[CD], False)
    layer.pack(W_q, scales, zeros, None)
    assert layer.W_group_mode in (3, 4) and layer.channel_scale_mode == 0

    def inputs(M):
        gx = torch.Generator(device=DEV).manual_seed(500 + M)
        return (torch.randn((M, K), generator=gx, dtype=CD, device=DEV) / 10.0).to(FP8)

    _check(layer, lambda x: x.to(CD) @ W.T, 5e-3, inputs)


def test_processor_fp8_activations_packed_codes(lib, data):     # helper.py:712-870 (A8W4_HQQ_INT_dynamic)
    from gemlite_b200 import helper
    from gemlite_b200.quant_utils import scale_activations_per_token_torch
    W, W_q, scales, zeros, xs = data
    layer = helper.A8W4_HQQ_INT_dynamic(device=DEV, dtype=CD).from_weights(W_q, scales, zeros)
    assert (layer.W_group_mode, layer.channel_scale_mode, layer.scaled_activations) == (3, 2, True)

    def ref(x):
        xq, sx = scale_activations_per_token_torch(x, w_dtype=FP8)
        return (xq.to(CD) @ W.T) * sx

    _check(layer, ref, 5e-3, lambda M: xs[M])
    # one group per row with the weight scale folded into the epilogue
    g = torch.Generator(device=DEV).manual_seed(21)
    s_row = (torch.rand((N, 1), generator=g, device=DEV) * 1e-3 + 5e-4).to(CD)
    z_row = torch.full((N, 1), 7.0, device=DEV, dtype=CD)
    Wr = (W_q.to(torch.float32) - 7.0) * s_row.float()
    for post_scale, modes in ((True, (1, 3)), (False, (3, 2))):
        lyr = helper.A8W4_HQQ_INT_dynamic(device=DEV, dtype=CD, post_scale=post_scale).from_weights(W_q, s_row, z_row)
        assert (lyr.W_group_mode, lyr.channel_scale_mode) == modes
        _check(lyr, lambda x: ((scale_activations_per_token_torch(x, w_dtype=FP8)[0].float() @ Wr.T)
                               * scale_activations_per_token_torch(x, w_dtype=FP8)[1]), 5e-3, lambda M: xs[M])


@pytest.mark.parametrize("dynamic", [False, True])
def test_processor_ternary_weights(lib, data, dynamic):         # helper.py:1208-1320 (A16W158_INT, A8W158_INT_dynamic)
    from gemlite_b200 import helper
    from gemlite_b200.quant_utils import scale_activations_per_token_torch
    _, _, _, _, xs = data
    g = torch.Generator(device=DEV).manual_seed(22)
    w = (torch.randint(0, 3, (N, K), generator=g, device=DEV) - 1).to(CD)
    bias = (torch.randn(N, generator=g, device=DEV) * 0.1).to(CD)
    w_scale = torch.tensor(0.0123, device=DEV)
    proc = (helper.A8W158_INT_dynamic if dynamic else helper.A16W158_INT)(device=DEV, dtype=CD)
    layer = proc.from_weights(w, w_scale, bias=bias)
    assert layer.W_nbits == 2 and layer.W_group_mode == 1 and layer.channel_scale_mode == (3 if dynamic else 1)

    def ref(x):
        if dynamic:
            xq, sx = scale_activations_per_token_torch(x, w_dtype=torch.int8)
            return (xq.float() @ w.float().T) * sx * 0.0123 + bias.float()
        return (x.float() @ w.float().T) * 0.0123 + bias.float()

    _check(layer, ref, 5e-3, lambda M: xs[M])


# ---- the block-scaled processors on the reference's MX test (tests/test_mxfp.py:30-103): Linear(4224 -> 2048) with its
# weights divided by 10, bf16, against the unquantised layer; tolerances as written there per processor
MX_CASES = [  # (processor, keyword arguments, packed bytes per weight, tolerance)
    ("A8W8_MXFP_dynamic", {"post_scale": True}, 1.0, 2e-4),
    ("A8W8_MXFP_dynamic", {"post_scale": False}, 1.0, 2e-4),
    ("A8W4_MXFP_dynamic", {}, 0.5, 7e-4),
    ("A4W4_MXFP_dynamic", {}, 0.5, 1e-3),
    ("A4W4_NVFP_dynamic", {}, 0.5, 2e-3),
    ("A16W8_MXFP", {}, 1.0, 2e-4),          # (commented out there, same criterion)
    ("A16W4_MXFP", {}, 0.5, 7e-4),
]


@pytest.mark.parametrize("name,kw,bytes_per_weight,tol", MX_CASES)
def test_block_scaled_processors_on_the_reference_mx_case(lib, name, kw, bytes_per_weight, tol):
    from gemlite_b200 import helper
    Kmx, Nmx = 4224, 2048
    torch.manual_seed(0)
    lin = torch.nn.Linear(Kmx, Nmx, device=DEV, dtype=CD, bias=False)
    lin.weight.data /= 10.0
    lin.weight.requires_grad = False
    layer = getattr(helper, name)(device=DEV, dtype=CD, **kw).from_linear(lin, del_orig=False)
    assert layer.W_q.numel() * layer.W_q.itemsize == int(Kmx * Nmx * bytes_per_weight)
    assert layer.scaled_activations == (not name.startswith("A16"))
    for M in [1, 3, 16, 30, 32, 60, 100, 128]:
        g = torch.Generator(device=DEV).manual_seed(M)
        x = torch.randn((M, Kmx), generator=g, dtype=CD, device=DEV) / 10.0
        want = lin(x).float()
        for fam in ("GEMM", "GEMM_SPLITK"):
            got = layer.forward_manual(x, matmul_type=fam).float()
            err = (want - got).abs().mean().item()
            assert err < tol, (name, kw, fam, M, err, tol)
