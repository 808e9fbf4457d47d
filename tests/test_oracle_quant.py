"""CPU: the oracle's activation / weight quantisers against independent restatements of the
reference's torch functions (gemlite/quant_utils.py:261-283, 1131-1224, 130-219) on seeded inputs,
and internal properties (scales are the smallest that avoid clipping, codes decode back within half a
step)."""
import numpy as np
import torch

from oracle import oracle


def _x(seed, M, K, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(M, K, generator=g) * scale).to(torch.bfloat16).float().numpy()


def test_per_token_fp8_matches_torch_formula():
    x = _x(1, 5, 256)
    q, s = oracle.scale_activations_per_token(x, "fp8")
    t = torch.from_numpy(x)
    s_ref = (t.abs().amax(1, keepdim=True) / 448.0).clamp_(min=1e-6)
    q_ref = (t / s_ref).clamp_(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(s, s_ref.numpy()) and np.array_equal(q, q_ref)


def test_per_token_int8_rounds_half_away():
    x = np.array([[0.5, 1.5, -0.5, -1.5, 127.0, -64.0, 2.5, 0.0]], dtype=np.float32)
    q, s = oracle.scale_activations_per_token(x, "int8")
    assert s[0, 0] == np.float32(1.0)
    assert q.tolist() == [[1, 2, -1, -2, 127, -64, 3, 0]]


def test_mxfp4_matches_torch_reference_values():
    # torch reference: scales = 2^ceil(log2(amax/6)); codes by nearest value (argmin), ties to the lower
    # magnitude.  Decoded values must agree with the threshold rounding everywhere.
    x = _x(2, 7, 128)
    q, sc = oracle.scale_activations_mxfp4(x)
    assert sc.shape == (32, 4) and (sc[7:] == 127).all()
    t = torch.from_numpy(x).view(-1, 32)
    s_ref = (2 ** torch.ceil(torch.log2(t.abs().amax(1, keepdim=True) / 6.0))).clamp_(2.0 ** -30)
    assert np.array_equal(oracle.e8m0_decode(sc[:7]).reshape(-1, 1), s_ref.numpy())
    vals = torch.tensor(oracle.FP4_VALUES)
    idx = ((t / s_ref).reshape(-1, 1) - vals.view(1, -1)).abs().argmin(1)
    assert np.array_equal(oracle.unpack_fp4(q).reshape(-1), vals[idx].numpy())


def test_nvfp4_dynamic_and_static():
    x = _x(3, 3, 64, 2.0)
    q, sc, meta = oracle.scale_activations_nvfp4(x)
    assert sc.shape == (16, 4) and (sc[3:] == 0x38).all()
    assert meta == np.float32(2688.0) / np.abs(x).max()
    # reconstruction error bounded by half an fp4 step of the group scale (+ e4m3 scale rounding)
    rec = oracle.unpack_fp4(q).reshape(3, 4, 16) * (oracle.e4m3_decode(sc[:3]) / meta)[..., None]
    assert np.abs(rec.reshape(3, 64) - x).max() <= np.abs(x).max() * 0.25
    q2, sc2, meta2 = oracle.scale_activations_nvfp4(x, meta_scale=float(meta))
    assert np.array_equal(q, q2) and np.array_equal(sc, sc2)


def test_weight_quantisers_match_torch_reference():
    from gemlite_b200.quant_utils import WeightQuantizerMXFP
    g = torch.Generator().manual_seed(4)
    W = (torch.randn(16, 128, generator=g) * 0.02).to(torch.bfloat16)
    wq = WeightQuantizerMXFP(compute_dtype=torch.bfloat16, device="cpu")
    c, s = wq.quantize_mxfp4(W, index=True)
    oc, os_ = oracle.quantize_mxfp4_weights(W.float().numpy())
    assert np.array_equal(c.view(16, 128).numpy(), oc)
    assert np.array_equal(s.view(torch.uint8).view(16, 4).numpy(), os_)
    c, s, m = wq.quantize_nvfp4(W, index=True)
    oc, os_, om = oracle.quantize_nvfp4_weights(W.float().numpy())
    assert np.array_equal(c.view(16, 128).numpy(), oc)
    assert np.array_equal(s.view(torch.uint8).view(16, 8).numpy(), os_)
    assert np.float32(m.item()) == om
    deq = wq.dequantize(c.view(16, 128), s.view(16, 8), shape=(16, 128), dtype=torch.float32, meta_scales=1.0 / m)
    assert (deq - W.float()).abs().max() < W.float().abs().max() * 0.3


def test_matmul_int_modes_agree_with_plain_formula():
    g = torch.Generator().manual_seed(5)
    K, N, gs = 256, 24, 64
    Wq = torch.randint(0, 16, (N, K), generator=g)
    s = (torch.randn(N, K // gs, generator=g).abs() * 0.02).to(torch.bfloat16)
    z = (torch.rand(N, K // gs, generator=g) * 15).to(torch.bfloat16)
    x = torch.randn(3, K, generator=g).to(torch.bfloat16)
    W = ((Wq.view(N, -1, gs).double() - z.double()[..., None]) * s.double()[..., None]).view(N, K)
    want = (x.double() @ W.T).numpy()
    y3 = oracle.matmul_int(x, Wq.t(), s.t(), z.t(), 3, 0, gs, exact=True).numpy()
    assert oracle.rel_frobenius(y3, want) < 1e-12
    zp = (-z.float() * s.float()).to(torch.bfloat16)           # what pack() stores for fma mode
    y4 = oracle.matmul_int(x, Wq.t(), s.t(), zp.t(), 4, 0, gs).numpy()
    assert oracle.rel_frobenius(y4, want) < 1e-2
