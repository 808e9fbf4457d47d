"""GPU: the save / load cases of the reference's tests/test_serialization.py on its shapes, with its criteria: a
default-constructed layer loaded from a file written by `torch.save(state_dict)` reports the same 12 meta arguments,
bit-equal tensors and the same outputs (mean absolute difference below 1e-7) as the layer that was saved
(tests/test_serialization.py:28-56), directly and through a parent module, strict and with `assign=True`."""
import os
import tempfile

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV, CD = "cuda:0", torch.bfloat16


def _int_layer(K=4096, N=2048, bias=False, pb=None):
    from gemlite_b200 import GemLiteLinear
    from gemlite_b200.dtypes import TORCH_TO_DTYPE
    g = torch.Generator(device=DEV).manual_seed(K + N)
    W_q = torch.randint(0, 15, (N, K), generator=g, device=DEV).to(torch.uint8)
    n_groups = W_q.numel() // 128
    scales = torch.full((n_groups, 1), 0.001, device=DEV, dtype=CD)
    zeros = torch.full((n_groups, 1), 7.0, device=DEV, dtype=CD)
    b = (torch.randn(N, generator=g, device=DEV) * 0.01).to(CD) if bias else None
    layer = GemLiteLinear(4, group_size=128, in_features=K, out_features=N, input_dtype=TORCH_TO_DTYPE[CD], output_dtype=TORCH_TO_DTYPE[CD])
    layer.pack(W_q, scales, zeros, b, packing_bitwidth=pb)
    return layer


def _through_file(state):
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "layer.pt")
        torch.save(state, path)
        return torch.load(path)


def _same_outputs(a, b, K, family="GEMM", M=32):
    x = torch.randn(M, K, dtype=CD, device=DEV) / 10.0
    assert (a.forward_manual(x, matmul_type=family) - b.forward_manual(x, matmul_type=family)).abs().mean().item() < 1e-7


def _check_round_trip(layer, family="GEMM", M=32):
    from gemlite_b200 import GemLiteLinear
    loaded = GemLiteLinear()
    loaded.load_state_dict(_through_file(layer.state_dict()))
    assert list(loaded.get_meta_args()) == list(layer.get_meta_args())
    for t0, t1 in zip(layer.get_tensor_args(), loaded.get_tensor_args()):
        if t0 is not None and t0.numel() > 0:
            assert (t0.float() - t1.float()).abs().mean().item() == 0
    _same_outputs(layer, loaded, layer.in_features, family, M)
    return loaded


def test_packed_int_layer(lib):                                   # :62-79
    _check_round_trip(_int_layer())


def test_fp8_layer_with_channel_scales(lib):                      # :82-100
    from gemlite_b200 import GemLiteLinear
    from gemlite_b200.dtypes import TORCH_TO_DTYPE
    K, N = 4096, 2048
    g = torch.Generator(device=DEV).manual_seed(5)
    W = torch.randn((N, K), generator=g, dtype=CD, device=DEV) / 10.0
    s = torch.rand((1, N), generator=g, dtype=CD, device=DEV) * 1e-4
    layer = GemLiteLinear(W_nbits=8, group_size=K, in_features=K, out_features=N, input_dtype=TORCH_TO_DTYPE[torch.float8_e4m3fn],
                          output_dtype=TORCH_TO_DTYPE[CD], scaled_activations=True)
    layer.pack(W.to(torch.float8_e4m3fn), scales=s, zeros=None, bias=None)
    _check_round_trip(layer)


def _patched(processor_name):
    from gemlite_b200 import helper
    torch.manual_seed(42)
    model = torch.nn.Sequential(torch.nn.Linear(4224, 2048, dtype=CD, device=DEV, bias=False))
    model.requires_grad_(False)
    model[0].weight.data /= 10.0
    helper.patch_model(model, device=DEV, processor=getattr(helper, processor_name)(dtype=CD))
    return model


@pytest.mark.parametrize("processor", ["A4W4_MXFP_dynamic", "A4W4_NVFP_dynamic"])
def test_block_scaled_layers(lib, processor):                     # :123-131, 485-491
    from gemlite_b200 import GemLiteLinear
    model = _patched(processor)
    _check_round_trip(model[0], "GEMM")
    _check_round_trip(model[0], "GEMM_SPLITK", M=2)
    # through a parent module, strict: what the helper changed after pack() (meta_scale, channel mode 4) comes back
    loaded = torch.nn.Sequential(GemLiteLinear()).to(DEV)
    loaded.load_state_dict(_through_file(model.state_dict()), strict=True)
    assert loaded[0].meta_scale.dtype == model[0].meta_scale.dtype and torch.equal(loaded[0].meta_scale, model[0].meta_scale)
    assert loaded[0].channel_scale_mode == model[0].channel_scale_mode == 4
    _same_outputs(model[0], loaded[0], 4224, "GEMM")
    _same_outputs(model[0], loaded[0], 4224, "GEMM_SPLITK", M=2)


def test_saved_again_after_a_load(lib):                           # :138-177
    from gemlite_b200 import GemLiteLinear
    orig = _int_layer()
    first = GemLiteLinear()
    first.load_state_dict(_through_file(orig.state_dict()))
    assert len(list(first.parameters())) > 0
    sd2 = _through_file(first.state_dict())
    assert "W_q" in sd2 and "scales" in sd2
    second = GemLiteLinear()
    second.load_state_dict(sd2)
    _same_outputs(orig, second, 4096)


def test_fresh_module_placeholders(lib):                          # :250-272
    from gemlite_b200 import GemLiteLinear
    sd = GemLiteLinear().state_dict()
    assert {"W_q", "scales", "zeros", "metadata", "orig_shape", "meta_scale"} <= set(sd) and "bias" not in sd
    assert all(sd[k].numel() == 0 for k in ("W_q", "scales", "zeros", "metadata", "orig_shape")) and sd["meta_scale"].dim() == 0


@pytest.mark.parametrize("strict,assign", [(False, False), (True, False), (True, True)])
def test_parent_module_loads(lib, strict, assign):                # :299-331, 428-441
    from gemlite_b200 import GemLiteLinear
    ref = torch.nn.Sequential(_int_layer(2048, 1024)).to(DEV)
    loaded = torch.nn.Sequential(GemLiteLinear()).to(DEV)
    res = loaded.load_state_dict(_through_file(ref.state_dict()), strict=strict, assign=assign)
    assert list(res.missing_keys) == [] and list(res.unexpected_keys) == []
    _same_outputs(ref[0], loaded[0], 2048)


@pytest.mark.parametrize("pb,dt", [(8, torch.uint8), (16, torch.int16), (32, torch.int32)])
def test_packing_widths_round_trip(lib, pb, dt):                  # :334-358
    layer = _int_layer(2048, 1024, pb=pb)
    assert layer.W_q.dtype == dt
    assert _check_round_trip(layer).W_q.dtype == dt


def test_bias_round_trips(lib):                                   # :380-408
    from gemlite_b200 import GemLiteLinear
    layer = _int_layer(2048, 1024, bias=True)
    assert "bias" in layer.state_dict()
    _check_round_trip(layer)
    ref = torch.nn.Sequential(layer).to(DEV)
    loaded = torch.nn.Sequential(GemLiteLinear()).to(DEV)
    loaded.load_state_dict(_through_file(ref.state_dict()), strict=True)
    assert loaded[0].bias is not None and torch.equal(ref[0].bias, loaded[0].bias)
    _same_outputs(ref[0], loaded[0], 2048)
