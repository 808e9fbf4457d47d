"""GPU: the benchmark configurations at their own sizes.  The CPU oracle cannot finish these in seconds, so the
checker is a plain torch fp32 product on the GPU of the same quantised operands (no library matmul involved), on the
whole output, plus sampled output columns against the fp64 formula / the CPU oracle.

  cfg2  A16W4 gs128 / A16W2 gs64, bf16, 8192 x 8192, M in {1, 2, 4, 8, 16, 64, 256, 1024, 4096, 8192}
  cfg3  A8W8 FP8 dynamic, 4096 -> 14336 and 14336 -> 4096, M in {1, 16, 128, 1024, 4096}
  cfg4  MXFP4 / NVFP4 dynamic, 16384 x 16384, M in {1, 64, 512, 4096}
Tolerances: 1e-2 relative Frobenius for the 16-bit path; for FP8 / FP4 5e-3 against the product of the identical
quantised operands (what the reference's kernels compute), and a loose bound against the unquantised layer (the
quantisation error itself: about 3.7e-2 for e4m3 x e4m3, 0.13 for e2m1 x e2m1)."""
import numpy as np
import pytest
import torch

from oracle import oracle
from tests.util import rel_fro, torch_ref_a16wn, torch_decode_fp4, sample_index

pytestmark = pytest.mark.gpu


def _rel(y, ref):
    return float((y.double() - ref.double()).norm() / ref.double().norm())


@pytest.mark.parametrize("nbits,gs", [(4, 128), (2, 64)])
def test_cfg2_a16wn_8192(lib, nbits, gs):
    from gemlite_b200 import helper
    N = K = 8192
    g = torch.Generator(device="cuda").manual_seed(2000 + nbits)
    W_q = torch.randint(0, 2 ** nbits, (N, K), generator=g, device="cuda", dtype=torch.int32).to(torch.uint8)
    s = (torch.randn(N * K // gs, 1, generator=g, device="cuda").abs() * 0.02).to(torch.bfloat16)
    z = (torch.rand(N * K // gs, 1, generator=g, device="cuda") * (2 ** nbits - 1)).to(torch.bfloat16)
    b = (torch.randn(N, generator=g, device="cuda") * 0.01).to(torch.bfloat16)
    layer = helper.A16Wn_HQQ_INT(device="cuda:0", dtype=torch.bfloat16, W_nbits=nbits).from_weights(W_q, s, z, bias=b)
    cols = sample_index(N, 48, seed=nbits)
    Wc = ((W_q[cols].double().view(len(cols), -1, gs) - z.view(N, -1)[cols].double()[..., None]) * s.view(N, -1)[cols].double()[..., None]).view(len(cols), K)
    for M in (1, 2, 4, 8, 16, 64, 256, 1024, 4096, 8192):
        x = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
        y = layer(x).float()
        ref = torch_ref_a16wn(x, W_q, s, z, b, gs)
        assert _rel(y, ref) < 1e-2, (M, _rel(y, ref))
        want = x.double() @ Wc.T + b[cols].double()
        assert _rel(y[:, cols], want) < 1e-2, (M, "fp64 columns")
        del x, y, ref


@pytest.mark.parametrize("K,N", [(4096, 14336), (14336, 4096)])
def test_cfg3_fp8_llama_mlp(lib, K, N):
    from gemlite_b200 import helper, quant_utils as qu
    g = torch.Generator(device="cuda").manual_seed(3000 + K)
    lin = torch.nn.Linear(K, N, bias=False, dtype=torch.bfloat16, device="cuda")
    lin.weight.data = (torch.randn(N, K, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    W = lin.weight.data.clone()
    layer = helper.A8W8_FP8_dynamic(device="cuda:0", dtype=torch.bfloat16).from_linear(lin)
    Wq = layer.W_q.t().float()
    for M in (1, 16, 128, 1024, 4096):
        x = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
        y = layer(x).float()
        xq, sx = qu.scale_activations_per_token(x, torch.float8_e4m3fn)
        ref = (xq.float() @ Wq.T) * sx.view(-1, 1) * layer.scales.float().view(1, -1)
        assert _rel(y, ref) < 5e-3, (M, _rel(y, ref))
        assert _rel(y, x.float() @ W.float().T) < 6e-2, (M, "unquantised")   # e4m3 on both operands: about 3.7e-2
        # sampled rows through the CPU oracle's quantiser and an fp64 product
        rows = sample_index(M, 3, seed=M)
        xo, so = oracle.scale_activations_per_token(x[rows].float().cpu().numpy(), "fp8")
        want = (oracle.e4m3_decode(xo).astype(np.float64) @ Wq.double().cpu().numpy().T) * so.astype(np.float64) * layer.scales.cpu().double().numpy().reshape(1, -1)
        assert rel_fro(y[rows].cpu().numpy(), want) < 5e-3, (M, "oracle rows")
        del x, y, ref


@pytest.mark.parametrize("fmt", ["mxfp4", "nvfp4"])
def test_cfg4_fp4_16384(lib, fmt):
    from gemlite_b200 import helper, quant_utils as qu
    N = K = 16384
    g = torch.Generator(device="cuda").manual_seed(4000)
    lin = torch.nn.Linear(K, N, bias=False, dtype=torch.bfloat16, device="cuda")
    lin.weight.data = (torch.randn(N, K, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    W = lin.weight.data.clone()
    proc = (helper.A4W4_MXFP_dynamic if fmt == "mxfp4" else helper.A4W4_NVFP_dynamic)(device="cuda:0", dtype=torch.bfloat16)
    layer = proc.from_linear(lin)
    gs, e8 = (32, True) if fmt == "mxfp4" else (16, False)
    wq = layer.W_q.t().contiguous()
    sw = layer.scales.contiguous().view(torch.uint8)
    Wd = torch_decode_fp4(wq, sw, gs, e8)
    for M in (1, 64, 512, 4096):
        x = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
        y = layer(x).float()
        if fmt == "mxfp4":
            xq, sx = qu.scale_activations_mxfp4(x, scale_layout=0)
            meta = 1.0
        else:
            xq, sx, mx = qu.scale_activations_nvfp4(x, scale_layout=0)
            meta = 1.0 / (float(layer.meta_scale.item()) * float(mx.item()))
        ref = (torch_decode_fp4(xq, sx, gs, e8) @ Wd.T) * meta
        assert _rel(y, ref) < 5e-3, (M, _rel(y, ref))
        # against the unquantised layer: 4-bit operands on both sides (about 0.13 relative at these distributions)
        assert _rel(y, x.float() @ W.float().T) < 0.2, (M, "unquantised")
        del x, y, ref
