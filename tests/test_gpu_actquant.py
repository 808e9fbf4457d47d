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


def _midpoint_groups(scale, group):
    """Rows of groups whose scaled values sit on and next to every e2m1 midpoint, both signs, with signed zeros: the
    group's largest magnitude is 6 * scale, so the group scale is exactly `scale` (a power of two)."""
    mids = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)
    vals = []
    for m in mids:
        for d in (0, 1, -1):                                  # the midpoint, one fp32 ulp above it, one below
            f = np.nextafter(m, np.float32(np.inf if d > 0 else -np.inf)) if d else m
            vals += [f, -f]
    vals += [0.0, -0.0, 1e-30, -1e-30, 0.1, -0.1, 6.0, -6.0, 7.5, 5.5, -5.5, 0.5, 1.0, -3.0]
    vals = np.array(vals, dtype=np.float32)
    n_groups = -(-len(vals) // (group - 1))
    out = np.zeros((n_groups, group), dtype=np.float32)
    for g in range(n_groups):
        chunk = vals[g * (group - 1):(g + 1) * (group - 1)]
        out[g, :len(chunk)] = chunk
        out[g, group - 1] = 6.0                               # pins the group's amax (7.5 is clipped below)
    out = np.clip(out, -6.0, 6.0)
    return (out * np.float32(scale)).astype(np.float32)


def test_fp4_codes_on_and_around_the_midpoints(lib):
    """The codes come from the hardware conversion plus corrections (ties go to the smaller magnitude, -0.0 is +0): values
    exactly on a midpoint, one ulp either side, signed zeros and saturation, against the oracle's thresholds."""
    from gemlite_b200 import quant_utils as qu
    # NVFP4 with a given tensor scale of 1: group scale = e4m3(amax / 6) = 0.5, so x / 0.5 is exact
    g16 = _midpoint_groups(0.5, 16)
    x = torch.from_numpy(g16.reshape(1, -1).copy())
    x = torch.cat([x, torch.zeros(1, (-x.shape[1]) % 64)], dim=1) if x.shape[1] % 64 else x
    q, s, meta = qu.scale_activations_nvfp4(x.cuda(), meta_scale=torch.tensor([1.0], device="cuda"))
    oq, os_, _ = oracle.scale_activations_nvfp4(x.numpy(), meta_scale=1.0)
    assert np.array_equal(s.view(torch.uint8).cpu().numpy(), os_) and np.array_equal(q.cpu().numpy(), oq)
    # MXFP4: fp32 activations (exact form) and bf16 activations (nudged form; the ulp neighbours round to the midpoints in bf16)
    g32 = _midpoint_groups(0.25, 32)
    x32 = torch.from_numpy(g32.reshape(1, -1).copy())
    x32 = torch.cat([x32, torch.zeros(1, (-x32.shape[1]) % 128)], dim=1) if x32.shape[1] % 128 else x32
    for xin in (x32, x32.to(torch.bfloat16), x32.to(torch.float16)):
        q, s = qu.scale_activations_mxfp4(xin.cuda())
        oq, os_ = oracle.scale_activations_mxfp4(xin.float().numpy())
        assert np.array_equal(s.cpu().numpy(), os_) and np.array_equal(q.cpu().numpy(), oq), xin.dtype


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_kernels_match_the_torch_restatements_on_the_device(lib, dtype):
    """The block-scaled `scale_activations_*_torch` run on the GPU as plain torch ops: same codes and scale bytes as the
    kernels.  (The per-token one is not compared here: torch divides by a scalar on the GPU by multiplying with its
    reciprocal, one ulp off the kernel's IEEE division; kernel and restatement each match the oracle on their own.)"""
    from gemlite_b200 import quant_utils as qu
    x = _x(77, 37, 4224, dtype, 2.0).cuda()
    q, s = qu.scale_activations_mxfp8(x)
    qt, st = qu.scale_activations_mxfp8_torch(x)
    assert torch.equal(q.view(torch.uint8), qt.view(torch.uint8)) and torch.equal(s, st)
    q, s = qu.scale_activations_mxfp4(x)
    qt, st = qu.scale_activations_mxfp4_torch(x)
    assert torch.equal(q, qt) and torch.equal(s, st)
    q, s, m = qu.scale_activations_nvfp4(x)
    qt, st, mt = qu.scale_activations_nvfp4_torch(x)
    assert torch.equal(m.reshape(-1), mt.reshape(-1)) and torch.equal(q, qt) and torch.equal(s.view(torch.uint8), st.view(torch.uint8))


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
