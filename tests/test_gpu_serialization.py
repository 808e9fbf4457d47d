"""GPU: checkpoint schema and round trips of GemLiteLinear (the cases of the reference's
tests/test_serialization.py: direct and through a parent module, bias presence, fresh-module keys,
W_q dtype per packing width, helper mode overrides surviving a reload)."""
import pytest
import torch

from tests.util import make_a16wn

pytestmark = pytest.mark.gpu
KEYS = {"W_q", "scales", "zeros", "metadata", "orig_shape", "meta_scale"}


def _layer(bias=True, pb=32):
    from gemlite_b200 import GemLiteLinear, DType
    x, W_q, s, z, b = make_a16wn(256, 512, 4, 64, torch.float16, seed=1, M=3)
    layer = GemLiteLinear(4, 64, 512, 256, DType.FP16, DType.FP16)
    layer.pack(W_q.cuda(), s.cuda(), z.cuda(), bias=b.cuda() if bias else None, packing_bitwidth=pb)
    return layer, x.cuda()


def test_fresh_module_advertises_schema(lib):
    from gemlite_b200 import GemLiteLinear
    sd = GemLiteLinear(4, 64, 512, 256).state_dict()
    assert set(sd) == KEYS and sd["W_q"].numel() == 0 and sd["meta_scale"].dim() == 0


@pytest.mark.parametrize("bias", [True, False])
def test_direct_roundtrip(lib, bias):
    from gemlite_b200 import GemLiteLinear
    layer, x = _layer(bias)
    sd = layer.state_dict()
    assert set(sd) == (KEYS | {"bias"} if bias else KEYS)
    assert sd["metadata"].dtype == torch.int32 and sd["metadata"].numel() == 12
    assert sd["orig_shape"].tolist() == [256, 512]
    fresh = GemLiteLinear(4, 64, 512, 256)
    fresh.load_state_dict({k: v.clone() for k, v in sd.items()})
    assert torch.equal(fresh(x), layer(x))
    assert fresh.get_meta_args() == layer.get_meta_args()
    sd2 = fresh.state_dict()
    assert set(sd2) == set(sd) and all(torch.equal(sd2[k], sd[k]) for k in sd)


def test_parent_module_roundtrip_and_mode_override(lib):
    from gemlite_b200 import GemLiteLinear
    layer, x = _layer(True)
    layer.W_group_mode = 3                       # a helper-style override after pack()
    layer.zeros.data = (-layer.zeros.data / layer.scales.data).to(layer.zeros.dtype)
    parent = torch.nn.Sequential(layer)
    sd = parent.state_dict()
    assert sd["0.metadata"].tolist()[10] == 3    # metadata is rebuilt from the live attributes on save
    fresh = torch.nn.Sequential(GemLiteLinear(4, 64, 512, 256))
    fresh.load_state_dict(sd, strict=True, assign=True)
    assert fresh[0].W_group_mode == 3
    assert torch.equal(fresh(x), parent(x))


@pytest.mark.parametrize("pb,dt", [(8, torch.uint8), (16, torch.int16), (32, torch.int32)])
def test_packing_width_dtypes(lib, pb, dt):
    layer, x = _layer(False, pb)
    assert layer.W_q.dtype == dt and layer.elements_per_sample == pb // 4
    assert layer.W_q.shape == (512 * 4 // pb, 256) and layer.W_q.is_contiguous()


def test_missing_keys_raise(lib):
    from gemlite_b200 import GemLiteLinear
    layer, _ = _layer()
    sd = layer.state_dict()
    del sd["metadata"]
    with pytest.raises(RuntimeError):
        GemLiteLinear(4, 64, 512, 256).load_state_dict(dict(sd))


def test_nvfp4_legacy_default_and_5d_scales(lib):
    from gemlite_b200 import helper, GemLiteLinear
    lin = torch.nn.Linear(512, 256, bias=False, dtype=torch.bfloat16).cuda()
    layer = helper.A4W4_NVFP_dynamic(device="cuda:0", dtype=torch.bfloat16).from_linear(lin)
    x = torch.randn(4, 512, dtype=torch.bfloat16, device="cuda")
    sd = {k: v.clone() for k, v in layer.state_dict().items()}
    # a checkpoint written with the reference's 5-D pre-shuffled scales loads to the same layer
    s2d = sd["scales"].contiguous()
    N, G = s2d.shape
    sd5 = dict(sd)
    sd5["scales"] = s2d.view(torch.uint8).reshape(N // 128, 4, 32, G // 4, 4).permute(0, 3, 2, 1, 4).reshape(1, N // 128, G // 4, 2, 256).contiguous().view(torch.float8_e4m3fn)
    a, b = GemLiteLinear(4, 16, 512, 256), GemLiteLinear(4, 16, 512, 256)
    a.load_state_dict(dict(sd))
    b.load_state_dict(sd5)
    assert torch.equal(a(x), layer(x)) and torch.equal(b(x), layer(x))
    legacy = dict(sd)
    del legacy["meta_scale"]
    c = GemLiteLinear(4, 16, 512, 256)
    c.load_state_dict(legacy)
    assert abs(c.meta_scale.item() - 0.05) < 1e-7
