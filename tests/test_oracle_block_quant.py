"""CPU: the oracle's restatement of 128 x 128 block quantisation (channel_scale_mode 5).  The per-block activation
quantiser is pinned to the output of the reference's own torch function (tests/golden/block_quant_golden.npz); the
reference's int8 torch path rounds half to even where its active Triton kernel (and the oracle) round half away from
zero, so int8 codes are compared with a tie allowance.  The matmul is checked against the defining formula."""
import numpy as np
import torch

from oracle import oracle
from tests import golden_inputs as gi


def test_per_block_quantiser_matches_reference_torch_function():
    gold = np.load(gi.GOLDEN_BLOCK_QUANT)
    for seed, M, K in gi.BLOCK_QUANT_CASES:
        x = gi.block_quant_input(seed, M, K)
        assert abs(float(x.double().sum()) - float(gold["x_sum_s%d" % seed][0])) < 1e-6
        xf = x.float().numpy()
        q, s = oracle.scale_activations_per_block(xf, "fp8")
        assert s.shape == (M, K // 128) and np.array_equal(s, gold["s_fp8_s%d" % seed])
        assert np.array_equal(q, gold["q_fp8_s%d" % seed])
        q, s = oracle.scale_activations_per_block(xf, "int8")
        assert np.array_equal(s, gold["s_int8_s%d" % seed])
        ref = gold["q_int8_s%d" % seed]
        diff = q.astype(np.int32) - ref.astype(np.int32)
        assert np.abs(diff).max() <= 1 and (diff != 0).mean() < 2e-3          # exact ties only
        assert float(s.min()) == np.float32(1e-6) or seed != 7001               # the floored block of case 7001


def test_block_quant_matmul_formula_and_weight_quantiser():
    g = torch.Generator().manual_seed(7100)
    N, K, M = 200, 384, 3                                                        # ragged N: 2 block rows, the last one partial
    W = (torch.randn(N, K, generator=g) * 0.05).numpy()
    x = (torch.randn(M, K, generator=g) * 0.3).numpy()
    for kind in ("fp8", "int8"):
        wq, sw = oracle.quantize_block_weights(W, kind)
        assert wq.shape == (N, K) and sw.shape == (2, 3)
        xq, sx = oracle.scale_activations_per_block(x, kind)
        y = oracle.matmul_block_quant(xq, sx, wq, sw, kind)
        # the same thing written out: dequantise both operands element-wise, then one product
        Wd = (oracle.e4m3_decode(wq) if kind == "fp8" else wq).astype(np.float64) * np.repeat(np.repeat(sw, 128, 0)[:N], 128, 1)
        Xd = (oracle.e4m3_decode(xq) if kind == "fp8" else xq).astype(np.float64) * np.repeat(sx, 128, 1)
        assert np.allclose(y, Xd @ Wd.T, rtol=1e-10, atol=1e-12)
        assert np.linalg.norm(y - x.astype(np.float64) @ W.astype(np.float64).T) / np.linalg.norm(x @ W.T) < (0.05 if kind == "fp8" else 0.02)
