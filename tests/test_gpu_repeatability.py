"""GPU: every kernel family, called many times back to back on the same operands (each call overlapping the tail of the
one before: programmatic dependent launch), returns the same bits every time and leaves the status word at zero.  A race
in a pipeline shows up here long before it moves a whole-matrix error norm."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _linear(K, N):
    lin = torch.nn.Linear(K, N, bias=False, dtype=torch.bfloat16, device=DEV)
    lin.weight.data.normal_(0, 0.02)
    return lin


def _packed(N, K, nbits, gs):
    from gemlite_b200 import helper
    g = torch.Generator(device=DEV).manual_seed(nbits)
    W_q = torch.randint(0, 2 ** nbits, (N, K), generator=g, device=DEV, dtype=torch.int32).to(torch.uint8)
    s = (torch.randn(N * K // gs, 1, generator=g, device=DEV).abs() * 0.02).to(torch.bfloat16)
    z = (torch.rand(N * K // gs, 1, generator=g, device=DEV) * (2 ** nbits - 1)).to(torch.bfloat16)
    return helper.A16Wn_HQQ_INT(device=DEV, dtype=torch.bfloat16, W_nbits=nbits).from_weights(W_q, s, z)


def _make(name):
    from gemlite_b200 import helper
    kw = dict(device=DEV, dtype=torch.bfloat16)
    if name == "a16w4":
        return _packed(4096, 4096, 4, 128), 4096
    if name == "a16w2":
        return _packed(4096, 4096, 2, 64), 4096
    if name == "a16w8":
        return _packed(2048, 4096, 8, 128), 4096
    if name == "fp8":
        return helper.A8W8_FP8_dynamic(**kw).from_linear(_linear(4096, 4096)), 4096
    if name == "int8":
        return helper.A8W8_INT8_dynamic(**kw).from_linear(_linear(4096, 4096)), 4096
    if name == "fp8_block":
        return helper.A8W8_FP8_dynamic(block_quant=True, **kw).from_linear(_linear(4096, 4096)), 4096
    if name == "mxfp8":
        return helper.A8W8_MXFP_dynamic(post_scale=False, **kw).from_linear(_linear(4096, 4096)), 4096
    if name == "mxfp4":
        return helper.A4W4_MXFP_dynamic(**kw).from_linear(_linear(4096, 4096)), 4096
    if name == "nvfp4":
        return helper.A4W4_NVFP_dynamic(**kw).from_linear(_linear(4096, 4096)), 4096
    if name == "a16w8_channel":
        return helper.A16W8_INT8(**kw).from_linear(_linear(4096, 2048)), 4096
    if name == "a16w4_mx":
        return helper.A16W4_MXFP(**kw).from_linear(_linear(4096, 2048)), 4096
    raise KeyError(name)


@pytest.mark.parametrize("name,Ms", [
    ("a16w4", (1, 8, 32, 64, 200, 600, 2304)), ("a16w2", (1, 16, 64, 2304)), ("a16w8", (1, 64, 600)),
    ("fp8", (1, 32, 600, 4096)), ("int8", (1, 600)), ("fp8_block", (1, 64, 2304)), ("mxfp8", (1, 600)),
    ("mxfp4", (1, 64, 2304)), ("nvfp4", (1, 64, 2304)), ("a16w8_channel", (1, 4, 9)), ("a16w4_mx", (1, 4, 9))])
def test_repeated_calls_agree_bit_for_bit(lib, name, Ms):
    from gemlite_b200 import core
    torch.manual_seed(len(name))
    layer, K = _make(name)
    for M in Ms:
        x = torch.randn(M, K, dtype=torch.bfloat16, device=DEV)
        outs = [layer(x).clone() for _ in range(24)]
        torch.cuda.synchronize()
        differing = [i for i, o in enumerate(outs) if not torch.equal(o, outs[0])]
        assert differing == [], (name, M, differing)
        assert bool(torch.isfinite(outs[0].float()).all())
    assert core.matmul_status(DEV, clear=False) == 0
