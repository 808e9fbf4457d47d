"""GPU: seeded random layers (packed 8/4/2/1-bit with random group sizes and ragged N, FP8 / INT8 with channel or block
scales, MXFP8 with block or per-token activation scales, MXFP4, NVFP4) at random batch sizes from every dispatch range:
the kernel the library picks against the general CUDA-core kernel (`kernel_override = 1`, itself pinned to the oracle by
the other tests) at 1e-2, a second call bit-identical, the status word zero."""
import random

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _rel(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-30))


def _check(tag, layer, K, rnd):
    from gemlite_b200 import core
    for M in sorted({1, rnd.randint(2, 16), rnd.randint(17, 64), rnd.randint(65, 300), rnd.randint(301, 1500)}):
        x = torch.randn(M, K, dtype=torch.bfloat16, device=DEV)
        y, y2 = layer(x), layer(x)
        core.set_kernel_override(1)
        try:
            yg = layer(x)
        finally:
            core.set_kernel_override(0)
        assert core.matmul_status(DEV, clear=True) == 0, (tag, M)
        assert torch.equal(y, y2), (tag, M)
        assert bool(torch.isfinite(y.float()).all()) and _rel(y, yg) < 1e-2, (tag, M, _rel(y, yg))


@pytest.mark.parametrize("seed", [11, 12, 13])
def test_packed_layers(lib, seed):
    from gemlite_b200 import helper
    rnd = random.Random(seed)
    torch.manual_seed(seed)
    for it in range(8):
        nbits, gs = rnd.choice([4, 4, 2, 8, 1]), rnd.choice([64, 128, 256])
        N, K = rnd.choice([8, 16, 32]) * rnd.randint(4, 180), gs * rnd.randint(2, 40)
        g = torch.Generator(device=DEV).manual_seed(seed * 100 + it)
        W_q = torch.randint(0, 2 ** nbits, (N, K), generator=g, device=DEV, dtype=torch.int32).to(torch.uint8)
        s = (torch.randn(N * K // gs, 1, generator=g, device=DEV).abs() * 0.02 + 1e-3).to(torch.bfloat16)
        z = (torch.rand(N * K // gs, 1, generator=g, device=DEV) * (2 ** nbits - 1)).to(torch.bfloat16)
        b = (torch.randn(N, generator=g, device=DEV) * 0.5).to(torch.bfloat16) if it % 2 else None
        layer = helper.A16Wn_HQQ_INT(device=DEV, dtype=torch.bfloat16, W_nbits=nbits).from_weights(W_q, s, z, bias=b)
        _check("A16W%d gs%d N%d K%d" % (nbits, gs, N, K), layer, K, rnd)


@pytest.mark.parametrize("kind", ["fp8", "int8", "fp8_block", "int8_block", "mxfp8", "mxfp8_per_token", "mxfp4", "nvfp4"])
def test_quantised_activation_layers(lib, kind):
    from gemlite_b200 import helper
    rnd = random.Random(len(kind) * 7 + ord(kind[0]))
    torch.manual_seed(len(kind))
    kw = dict(device=DEV, dtype=torch.bfloat16)
    make = {"fp8": lambda: helper.A8W8_FP8_dynamic(**kw), "int8": lambda: helper.A8W8_INT8_dynamic(**kw),
            "fp8_block": lambda: helper.A8W8_FP8_dynamic(block_quant=True, **kw),
            "int8_block": lambda: helper.A8W8_INT8_dynamic(block_quant=True, **kw),
            "mxfp8": lambda: helper.A8W8_MXFP_dynamic(post_scale=False, **kw),
            "mxfp8_per_token": lambda: helper.A8W8_MXFP_dynamic(post_scale=True, **kw),
            "mxfp4": lambda: helper.A4W4_MXFP_dynamic(**kw), "nvfp4": lambda: helper.A4W4_NVFP_dynamic(**kw)}[kind]
    for it in range(3):
        N, K = 8 * rnd.randint(8, 700), 128 * rnd.randint(2, 48)
        if kind.startswith(("mx", "nv")):
            N = 128 * max(1, N // 128)
        lin = torch.nn.Linear(K, N, bias=bool(it % 2), dtype=torch.bfloat16, device=DEV)
        lin.weight.data.normal_(0, 0.03)
        _check("%s N%d K%d" % (kind, N, K), make().from_linear(lin), K, rnd)
