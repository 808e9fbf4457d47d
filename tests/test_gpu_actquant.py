"""GPU: dynamic activation quantisation kernels, through the C ABI, bit-exact against the oracle
(integer / byte outputs and fp32 scales), for ragged M, padded scale rows and zero inputs."""
import numpy as np
import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu


def _x(seed, M, K, dtype, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(M, K, generator=g) * scale).to(dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("M,K", [(1, 4096), (5, 14336), (33, 256), (128, 3968)])
def test_per_token_fp8_and_int8(lib, dtype, M, K):
    from gemlite_b200 import quant_utils as qu
    x = _x(M * 7 + K, M, K, dtype, 1.5)
    xf = x.float().numpy()
    q, s = qu.scale_activations_per_token(x.cuda(), torch.float8_e4m3fn)
    oq, os_ = oracle.scale_activations_per_token(xf, "fp8")
    assert s.shape == (M, 1) and s.dtype == torch.float32
    assert np.array_equal(s.cpu().numpy(), os_)
    assert np.array_equal(q.view(torch.uint8).cpu().numpy(), oq)
    q, s = qu.scale_activations_per_token(x.cuda(), torch.int8)
    oq, os_ = oracle.scale_activations_per_token(xf, "int8")
    assert np.array_equal(s.cpu().numpy(), os_) and np.array_equal(q.cpu().numpy(), oq)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,K", [(1, 16384), (3, 4224), (32, 128), (65, 2048)])
def test_mxfp4_mxfp8(lib, dtype, M, K):
    from gemlite_b200 import quant_utils as qu
    x = _x(M + K, M, K, dtype)
    x[0, :32] = 0                      # an all-zero group: scale clamps to 2^-30, codes 0
    xf = x.float().numpy()
    q, s = qu.scale_activations_mxfp4(x.cuda())
    oq, os_ = oracle.scale_activations_mxfp4(xf)
    assert q.shape == (M, K // 2) and s.shape == ((M + 31) // 32 * 32, K // 32) and s.dtype == torch.uint8
    assert np.array_equal(s.cpu().numpy(), os_)
    assert np.array_equal(q.cpu().numpy(), oq)
    q, s = qu.scale_activations_mxfp8(x.cuda())
    oq, os_ = oracle.scale_activations_mxfp8(xf)
    assert np.array_equal(s.cpu().numpy(), os_)
    assert np.array_equal(q.view(torch.uint8).cpu().numpy(), oq)


@pytest.mark.parametrize("M,K", [(1, 16384), (3, 4224), (16, 64), (70, 2048)])
def test_nvfp4_dynamic_and_static(lib, M, K):
    from gemlite_b200 import quant_utils as qu
    x = _x(3 * M + K, M, K, torch.bfloat16, 2.0)
    xf = x.float().numpy()
    for _ in range(2):                 # second call re-uses the amax scratch
        q, s, meta = qu.scale_activations_nvfp4(x.cuda())
        oq, os_, ometa = oracle.scale_activations_nvfp4(xf)
        assert s.shape == ((M + 15) // 16 * 16, K // 16) and s.dtype == torch.float8_e4m3fn
        assert np.float32(meta.item()) == ometa
        assert np.array_equal(s.view(torch.uint8).cpu().numpy(), os_)
        assert np.array_equal(q.cpu().numpy(), oq)
    static = torch.tensor([448.0], device="cuda")
    q, s, meta = qu.scale_activations_nvfp4(x.cuda(), meta_scale=static)
    oq, os_, _ = oracle.scale_activations_nvfp4(xf, meta_scale=448.0)
    assert meta.item() == 448.0
    assert np.array_equal(s.view(torch.uint8).cpu().numpy(), os_) and np.array_equal(q.cpu().numpy(), oq)


def test_full_size_properties(lib):
    # 4096 x 16384 bf16 (the largest benchmark activation that the oracle would take minutes on):
    # decoded values never exceed the group amax by more than the format allows, scales are powers of two
    # that avoid clipping, and quantising the dequantised tensor again is the identity (idempotence).
    from gemlite_b200 import quant_utils as qu
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(4096, 16384, generator=g, device="cuda", dtype=torch.bfloat16)
    q, s = qu.scale_activations_mxfp4(x)
    lut = torch.tensor(oracle.FP4_VALUES, device="cuda")
    vals = torch.stack([lut[(q & 15).long()], lut[(q >> 4).long()]], dim=-1).view(4096, 16384)
    scale = torch.pow(2.0, s[:4096].float() - 127.0)
    deq = (vals.view(4096, -1, 32) * scale[..., None]).view(4096, 16384)
    amax = x.float().abs().view(4096, -1, 32).amax(-1)
    assert bool((6.0 * scale >= amax).all()) and bool((3.0 * scale < amax).all())
    assert bool(((deq - x.float()).abs().view(4096, -1, 32).amax(-1) <= scale).all())
    q2, s2 = qu.scale_activations_mxfp4(deq.to(torch.bfloat16))
    vals2 = torch.stack([lut[(q2 & 15).long()], lut[(q2 >> 4).long()]], dim=-1).view(4096, 16384)
    deq2 = (vals2.view(4096, -1, 32) * torch.pow(2.0, s2[:4096].float() - 127.0)[..., None]).view(4096, 16384)
    assert torch.equal(deq2, deq)


def test_rejects_bad_inputs(lib):
    from gemlite_b200 import quant_utils as qu
    with pytest.raises(ValueError):
        qu.scale_activations_mxfp4(torch.zeros(2, 48, dtype=torch.bfloat16, device="cuda"))   # K % 32 != 0
    with pytest.raises(RuntimeError):
        qu.scale_activations_mxfp4(torch.zeros(2, 64, dtype=torch.bfloat16))                  # CPU tensor
    q, s = qu.scale_activations_mxfp4(torch.zeros(0, 64, dtype=torch.bfloat16, device="cuda"))
    assert q.shape == (0, 32) and s.shape == (0, 2)
