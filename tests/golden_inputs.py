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
