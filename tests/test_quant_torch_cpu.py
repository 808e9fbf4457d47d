"""CPU: the plain-torch restatements of the activation quantisers that the package keeps beside its kernels
(`scale_activations_*_torch`, the reference's comparison points: gemlite/quant_utils.py:261-283, 712-747, 1131-1224,
2503-2522) against the oracle, bit for bit, on seeded inputs with tiny groups, a zero group and padded rows."""
import numpy as np
import pytest
import torch

from oracle import oracle


def _x(seed, M, K, dtype):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g) * 1.5
    x[0, :32] *= 1e-12                       # a group whose scale hits the 2^-30 floor
    if M > 2:
        x[2, 32:64] = 0.0                    # an all-zero group
    return x.to(dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("M,K", [(1, 4096), (5, 4224), (33, 2048)])
def test_block_scaled_restatements_match_the_oracle(M, K, dtype):
    from gemlite_b200 import quant_utils as qu
    x = _x(M * 7 + K, M, K, dtype)
    xf = x.float().numpy()
    q, s = qu.scale_activations_mxfp8_torch(x)
    oq, os_ = oracle.scale_activations_mxfp8(xf)
    assert q.shape == x.shape and np.array_equal(q.view(torch.uint8).numpy(), oq) and np.array_equal(s.numpy(), os_)
    q, s = qu.scale_activations_mxfp4_torch(x)
    oq, os_ = oracle.scale_activations_mxfp4(xf)
    assert np.array_equal(q.numpy(), oq) and np.array_equal(s.numpy(), os_)
    for meta in (None, 448.0):
        q, s, m = qu.scale_activations_nvfp4_torch(x, meta_scale=meta)
        oq, os_, om = oracle.scale_activations_nvfp4(xf, meta_scale=meta)
        assert np.array_equal(q.numpy(), oq) and np.array_equal(s.view(torch.uint8).numpy(), os_)
        assert np.float32(m.item()) == om and m.shape == (1,)


@pytest.mark.parametrize("kind,dt", [("fp8", torch.float8_e4m3fn), ("int8", torch.int8)])
def test_per_token_and_per_block_restatements_match_the_oracle(kind, dt):
    from gemlite_b200 import quant_utils as qu
    x = _x(5, 9, 1024, torch.bfloat16)
    q, s = qu.scale_activations_per_token_torch(x, dt)
    oq, os_ = oracle.scale_activations_per_token(x.float().numpy(), kind)
    got = q.view(torch.uint8).numpy() if kind == "fp8" else q.numpy()
    assert np.array_equal(got, oq) and np.array_equal(s.numpy().reshape(-1), np.asarray(os_).reshape(-1))
    q, s = qu.scale_activations_per_block_torch(x, dt)
    oq, os_ = oracle.scale_activations_per_block(x.float().numpy(), kind)
    got = q.view(torch.uint8).numpy() if kind == "fp8" else q.numpy()
    assert np.array_equal(got, oq) and np.array_equal(s.numpy(), os_)
