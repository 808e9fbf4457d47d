"""GPU: the persistent tensor-core kernel with MORE OUTPUT TILES THAN SMs, so that a CTA walks several tiles: the
shared-memory ring runs across tile boundaries, the accumulator buffers alternate and their barrier phases flip.
FP8, INT8, MXFP4 and NVFP4, each with a ragged last tile and a K that ends in the middle of a K tile.  The whole
output is compared with a plain torch fp32 product of the same quantised operands (2e-3) and sampled rows with the
CPU oracle (5e-3)."""
import numpy as np
import pytest
import torch

from oracle import oracle
from tests.util import rel_fro, torch_decode_fp4, sample_index
from tests.test_gpu_tc import _status_word

pytestmark = pytest.mark.gpu


def _tiles(M, N, bn):
    return ((M + 127) // 128) * ((N + bn - 1) // bn)


@pytest.mark.parametrize("fp8", [True, False])
@pytest.mark.parametrize("M,N,K", [(2048, 4096, 1536), (2100, 4000, 1472), (1152, 8200, 640)])
def test_a8w8_more_tiles_than_sms(lib, fp8, M, N, K):
    from gemlite_b200 import helper, quant_utils as qu
    assert _tiles(M, N, 256) > 148                        # more 128 x 256 tiles than SMs: CTAs walk several tiles
    g = torch.Generator(device="cuda").manual_seed(31 + M)
    x = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    lin = torch.nn.Linear(K, N, bias=True, dtype=torch.bfloat16, device="cuda")
    lin.weight.data = (torch.randn(N, K, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    lin.bias.data = torch.randn(N, generator=g, device="cuda").to(torch.bfloat16)      # as large as the outputs
    bias = lin.bias.data.clone()
    proc = (helper.A8W8_FP8_dynamic if fp8 else helper.A8W8_INT8_dynamic)(device="cuda:0", dtype=torch.bfloat16)
    layer = proc.from_linear(lin)
    y = layer(x).float()
    assert _status_word() == 0
    xq, sx = qu.scale_activations_per_token(x, torch.float8_e4m3fn if fp8 else torch.int8)
    Wq = layer.W_q.t()                                    # [N, K]
    ref = (xq.float() @ Wq.float().T) * sx.view(-1, 1) * layer.scales.float().view(1, -1) + bias.float()
    assert rel_fro(y.cpu().numpy(), ref.cpu().numpy()) < 2e-3
    # element-wise: a wrong tile / a stale accumulator shows as a block of large errors, not as a small norm
    tol = 2e-2 * float(ref.abs().mean()) + 1e-2 * ref.abs()
    assert bool(((y - ref).abs() <= tol).all()), float(((y - ref).abs() - tol).max())
    rows = sample_index(M, 6, seed=M)
    xo, so = oracle.scale_activations_per_token(x[rows].float().cpu().numpy(), "fp8" if fp8 else "int8")
    Xd = oracle.e4m3_decode(xo).astype(np.float64) if fp8 else xo.astype(np.float64)
    Wd = Wq.float().double().cpu().numpy()
    want = (Xd @ Wd.T) * so.astype(np.float64) * layer.scales.cpu().double().numpy().reshape(1, -1) + bias.double().cpu().numpy()
    assert rel_fro(y[rows].cpu().numpy(), want) < 5e-3


@pytest.mark.parametrize("fmt", ["mxfp4", "nvfp4"])
@pytest.mark.parametrize("M,N,K", [(2048, 4096, 1536), (2100, 4224, 1408), (1152, 8320, 768)])
def test_a4w4_more_tiles_than_sms(lib, fmt, M, N, K):
    from gemlite_b200 import helper, quant_utils as qu
    assert _tiles(M, N, 256) > 148
    g = torch.Generator(device="cuda").manual_seed(57 + M)
    x = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    lin = torch.nn.Linear(K, N, bias=False, dtype=torch.bfloat16, device="cuda")
    lin.weight.data = (torch.randn(N, K, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    proc = (helper.A4W4_MXFP_dynamic if fmt == "mxfp4" else helper.A4W4_NVFP_dynamic)(device="cuda:0", dtype=torch.bfloat16)
    layer = proc.from_linear(lin)
    y = layer(x).float()
    assert _status_word() == 0
    gs = 32 if fmt == "mxfp4" else 16
    wq = layer.W_q.t().contiguous()                       # [N, K/2] bytes
    sw = layer.scales.contiguous().view(torch.uint8)      # [N, G]
    if fmt == "mxfp4":
        xq, sx = qu.scale_activations_mxfp4(x, scale_layout=0)
        meta = 1.0
    else:
        xq, sx, mx = qu.scale_activations_nvfp4(x, scale_layout=0)
        meta = 1.0 / (float(layer.meta_scale.item()) * float(mx.item()))
    ref = (torch_decode_fp4(xq, sx, gs, fmt == "mxfp4") @ torch_decode_fp4(wq, sw, gs, fmt == "mxfp4").T) * meta
    assert rel_fro(y.cpu().numpy(), ref.cpu().numpy()) < 3e-3
    tol = 3e-2 * float(ref.abs().mean()) + 1e-2 * ref.abs()
    assert bool(((y - ref).abs() <= tol).all()), float(((y - ref).abs() - tol).max())
    rows = sample_index(M, 5, seed=M + 1)
    xr = x[rows].float().cpu().numpy()
    if fmt == "mxfp4":
        xo, so = oracle.scale_activations_mxfp4(xr)
        want = oracle.matmul_mx(xo, so, wq.cpu().numpy(), sw.cpu().numpy(), gs, meta_scale=None)
    else:
        # the tensor-wide scale comes from the whole activation matrix: quantise the sampled rows with that scale
        xo, so, _ = oracle.scale_activations_nvfp4(xr, meta_scale=float(mx.item()))
        want = oracle.matmul_mx(xo, so, wq.cpu().numpy(), sw.cpu().numpy(), gs, meta_scale=meta)
    assert rel_fro(y[rows].cpu().numpy(), want) < 5e-3
