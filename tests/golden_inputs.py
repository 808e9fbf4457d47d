"""Regenerates, from their seeds, the inputs that tests/golden/make_golden_triton.py fed to the reference
(same generator calls in the same order), and verifies them against the checksums in the fixture."""
import os

import numpy as np
import torch

from tests.util import make_a16wn

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "triton_golden.npz")
A16_CASES = [  # (seed, N, K, nbits, group_size, dtype, Ms) -- as in make_golden_triton.py
    (2001, 2032, 3968, 4, 128, torch.bfloat16, (1, 3, 16, 65)),
    (2002, 2032, 3968, 2, 64, torch.bfloat16, (1, 4, 30)),
    (2003, 1024, 2048, 4, 64, torch.float16, (1, 5, 100)),
    (2004, 512, 1024, 8, 128, torch.float16, (2, 16)),
]
LIN_CASES = (("fp8", 1024, 2048, (1, 16, 130)), ("int8", 1024, 2048, (2, 65)),
             ("mxfp4", 2048, 4224, (1, 16, 100)), ("nvfp4", 2048, 4224, (1, 16, 100)))


def load():
    return np.load(GOLDEN)


def a16_inputs(seed, N, K, nbits, gs, dtype, M):
    return make_a16wn(N, K, nbits, gs, dtype, seed + M, M=M, with_bias=False)


def quant_inputs(gold):
    """[(M, K, x bf16)], W bf16 [256, 1024] of the quantiser cases."""
    g = torch.Generator().manual_seed(3001)
    xs = []
    for M, K in ((1, 4096), (5, 4224), (33, 2048)):
        x = (torch.randn(M, K, generator=g) * 1.5).to(torch.bfloat16)
        assert abs(float(x.double().sum()) - float(gold["xq_M%d_K%d_x_sum" % (M, K)][0])) < 1e-6
        xs.append((M, K, x))
    W = (torch.randn(256, 1024, generator=g) * 0.02).to(torch.bfloat16)
    assert abs(float(W.double().sum()) - float(gold["wq_W_sum"][0])) < 1e-6
    return xs, W


def lin_inputs(gold, name):
    """W bf16 [N, K] and {M: x bf16} of one linear-layer case."""
    for nm, N, K, Ms in LIN_CASES:
        if nm != name:
            continue
        gg = torch.Generator().manual_seed(4000 + N)
        W = (torch.randn(N, K, generator=gg) * 0.02).to(torch.bfloat16)
        xs = {}
        for M in Ms:
            xs[M] = torch.randn(M, K, generator=gg).to(torch.bfloat16)
            assert abs(float(xs[M].double().sum()) - float(gold["lin_%s_M%d_x_sum" % (name, M)][0])) < 1e-6
        return W, xs
    raise KeyError(name)


# ---- the benchmark configurations at their own sizes (tests/golden/triton_golden_baseline.npz) ----
GOLDEN_BASELINE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "triton_golden_baseline.npz")
# (tag, kind, N, K, nbits, group size, {M: reference kernel families})
BASELINE_CASES = [
    ("cfg2_a16w4", "a16", 8192, 8192, 4, 128, {1: ("GEMV_REVSPLITK", "GEMM_SPLITK"), 64: ("GEMM_SPLITK", "GEMM"), 256: ("GEMM",)}),
    ("cfg2_a16w2", "a16", 8192, 8192, 2, 64, {1: ("GEMV_REVSPLITK",), 64: ("GEMM",)}),
    ("cfg3_fp8_up", "fp8", 14336, 4096, 8, 0, {1: ("GEMM_SPLITK",), 64: ("GEMM",)}),
    ("cfg3_fp8_down", "fp8", 4096, 14336, 8, 0, {1: ("GEMM_SPLITK",), 64: ("GEMM",)}),
    ("cfg4_mxfp4", "mxfp4", 16384, 16384, 4, 32, {1: ("GEMM_SPLITK",), 64: ("GEMM",)}),
]


def kept_rows(M):
    """Rows of an [M, N] output the fixture keeps: the first two, the middle one, the last two."""
    return sorted(set(r for r in (0, 1, M // 2, M - 2, M - 1) if 0 <= r < M))


def kept_cols(N):
    """Columns the fixture keeps: every 16th, shifted by 5 so that no tile boundary is favoured."""
    return list(range(5, N, 16))


def baseline_inputs(tag, M):
    """The operands of one baseline case, regenerated from its seed: a16 -> (x, W_q, scales, zeros); fp8 / mxfp4 -> (x, W bf16)."""
    idx = [c[0] for c in BASELINE_CASES].index(tag)
    _, kind, N, K, nbits, gs, _ = BASELINE_CASES[idx]
    if kind == "a16":
        x, W_q, s, z, _ = make_a16wn(N, K, nbits, gs, torch.bfloat16, 5000 + 10 * idx + 1, M=1, with_bias=False)
        g = torch.Generator().manual_seed(5500 + 10 * idx + M)
        return torch.randn(M, K, generator=g).to(torch.bfloat16), W_q, s, z
    g = torch.Generator().manual_seed(6000 + idx)
    W = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16)
    gx = torch.Generator().manual_seed(6500 + 10 * idx + M)
    return torch.randn(M, K, generator=gx).to(torch.bfloat16), W


# ---- per-block activation quantiser (tests/golden/block_quant_golden.npz) ----
GOLDEN_BLOCK_QUANT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "block_quant_golden.npz")
BLOCK_QUANT_CASES = [(7001, 1, 256), (7002, 5, 512), (7003, 33, 1024)]     # (seed, M, K)


def block_quant_input(seed, M, K):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g) * 1.5
    x[0, :128] *= 1e-8                      # a block whose scale hits the 1e-6 floor
    return x.to(torch.bfloat16)
