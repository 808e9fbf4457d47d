"""Layer processors: turn ``nn.Linear`` / pre-quantised tensors / HQQ layers into packed
``GemLiteLinear`` modules.  Class names, constructor arguments, ``from_weights`` /
``from_linear`` / ``from_packed_weights`` / ``from_hqqlinear`` signatures and the post-pack
mode overrides follow gemlite/helper.py (A16W8 :89-171, A16Wn :174-333, A16Wn_MXFP :384-421,
A16W4_NVFP :423-504, A8W8_dynamic :509-707, A8Wn_MXFP_dynamic :950-1040, A4W4_MXFP_dynamic
:1042-1114, A4W4_NVFP_dynamic :1116-1203, patch_model :35-87, warmup :1326-1376).
Weight quantisation here is offline torch code; the packed layer runs on the CUDA library.
"""
import gc

import torch

from .core import GemLiteLinear, GEMLITE_NVFP4_INPUT_SCALES
from .dtypes import DType, TORCH_TO_DTYPE
from .quant_utils import WeightQuantizerMXFP

default_fp8 = torch.float8_e4m3fn
default_post_scale = False
_FLOAT_DTYPES = (torch.float16, torch.bfloat16, torch.float32)


def cleanup_linear(linear_layer, del_orig=True):
    if del_orig:
        for attr in ["weight", "bias", "weight_scale", "W_q", "meta"]:
            val = getattr(linear_layer, attr, None)
            if val is not None and hasattr(val, "__len__") and len(val) > 0:
                setattr(linear_layer, attr, None)
    if torch.cuda.is_available():
        torch.cuda.empty_cache()


def _data(t):
    return t.data if isinstance(t, torch.nn.Parameter) else t


def _quantize_channelwise(weight, w_dtype, device):
    """Symmetric per-output-channel 8-bit quantisation: s = max(amax/qmax, 1e-6), q = clamp(W/s)."""
    info = torch.finfo(w_dtype) if w_dtype.is_floating_point else torch.iinfo(w_dtype)
    w = weight.to(dtype=torch.float32, device=device)
    scales = (w.abs().amax(axis=1, keepdim=True) / info.max).clamp_(min=1e-6)
    q = (w / scales).clamp_(min=info.min, max=info.max)
    q = q.to(w_dtype) if w_dtype.is_floating_point else q.round_().to(w_dtype)
    return q, scales


def patch_model(model, device, processor, skip_modules=["lm_head", "vision", "visual"], group_size=64):
    """Replace every ``nn.Linear`` (not matched by ``skip_modules``) by ``processor.from_linear`` /
    ``from_hqqlinear``.  ``group_size`` only matters for HQQ with W_nbits <= 4."""
    use_hqq = hasattr(processor, "from_hqqlinear")
    if use_hqq:
        from hqq.core.quantize import HQQLinear, BaseQuantizeConfig   # optional dependency
    else:
        class HQQLinear:  # placeholder type that nothing is an instance of
            pass
    for name, module in model.named_modules():
        module.name = name

    def convert(layer):
        layer = layer.to(device=device, non_blocking=True)
        if any(s in layer.name for s in skip_modules):
            return layer
        if use_hqq:
            if isinstance(layer, torch.nn.Linear):
                nb = processor.W_nbits
                cfg = BaseQuantizeConfig(nbits=nb, group_size=group_size if nb <= 4 else None)
                layer = HQQLinear(layer, quant_config=cfg, compute_dtype=layer.weight.dtype, device=device)
            return processor.from_hqqlinear(layer)
        return processor.from_linear(layer)

    def walk(parent):
        for name, child in parent.named_children():
            if isinstance(child, (torch.nn.Linear, HQQLinear)):
                setattr(parent, name, convert(child))
            else:
                walk(child)

    walk(model)
    model = model.to(device=device)
    torch.cuda.empty_cache()
    gc.collect()
    return model


# ---------------------------------------------------------------------------------------------
# 16-bit activations, 8-bit channel-wise weights
# ---------------------------------------------------------------------------------------------
class A16W8:
    def __init__(self, device="cuda:0", dtype=None, fp8=None, fp32_scale=True, post_scale=False):
        self.device, self.dtype, self.fp8 = device, dtype, fp8
        self.fp32_scale, self.post_scale = fp32_scale, post_scale

    def from_weights(self, weight, bias=None, scales=None):
        weight, bias = _data(weight), _data(bias)
        in_features, out_features = weight.shape[::-1]
        if scales is None:
            dtype = weight.dtype if self.dtype is None else self.dtype
            assert dtype in _FLOAT_DTYPES, f"Invalid weight dtype, should be floating point, got {dtype}"
            W_q, scales = _quantize_channelwise(weight, self.fp8 if self.fp8 else torch.int8, self.device)
        else:
            assert weight.itemsize == 1, f"Invalid weight.dtype, should be 8-bit (INT8 or FP8), got {weight.dtype}"
            dtype = self.dtype if self.dtype is not None else (scales.dtype if scales.dtype in (torch.float16, torch.bfloat16) else torch.float16)
            W_q, scales = weight.to(device=self.device), scales.to(device=self.device)
        bias = bias.to(device=self.device, dtype=dtype) if bias is not None else None
        gl_dtype = TORCH_TO_DTYPE[dtype]
        layer = GemLiteLinear(8, group_size=in_features, in_features=in_features, out_features=out_features,
                              input_dtype=gl_dtype, output_dtype=gl_dtype)
        layer.pack(W_q, scales, zeros=None, bias=bias)
        if self.post_scale:   # scale the accumulator per output channel
            layer.W_group_mode, layer.channel_scale_mode = 0, 1
        else:                 # scale the weights before the product
            layer.W_group_mode, layer.channel_scale_mode = 2, 0
        return layer

    def from_linear(self, linear_layer, del_orig=True):
        out = self.from_weights(weight=linear_layer.weight, bias=linear_layer.bias)
        cleanup_linear(linear_layer, del_orig)
        return out


class A16W8_INT8(A16W8):
    def __init__(self, device="cuda:0", dtype=None, fp32_scale=True, post_scale=False):
        super().__init__(device=device, dtype=dtype, fp8=None, fp32_scale=fp32_scale, post_scale=post_scale)


class A16W8_FP8(A16W8):
    def __init__(self, device="cuda:0", dtype=None, fp8=default_fp8, fp32_scale=True, post_scale=False):
        super().__init__(device=device, dtype=dtype, fp8=fp8, fp32_scale=fp32_scale, post_scale=post_scale)


# ---------------------------------------------------------------------------------------------
# 16-bit activations, n-bit grouped integer weights (HQQ style) or MXFP weights
# ---------------------------------------------------------------------------------------------
class A16Wn:
    def __init__(self, device="cuda:0", dtype=None, packing_bitwidth=None, post_scale=default_post_scale):
        self.post_scale, self.device, self.dtype = post_scale, device, dtype
        self.packing_bitwidth = packing_bitwidth
        self.quantizer_mx = None
        self.mx_fp8_dtype = default_fp8

    def from_packed_weights(self, W_q, scales, zeros, W_nbits, group_size, bias=None, quant_type="INT"):
        return self.from_weights_(W_q, scales, zeros, W_nbits, group_size, bias, quant_type, packed=True)

    def from_weights(self, W_q, scales, zeros, W_nbits, group_size, bias=None, quant_type="INT"):
        return self.from_weights_(W_q, scales, zeros, W_nbits, group_size, bias, quant_type)

    def from_weights_(self, W_q, scales, zeros, W_nbits, group_size, bias=None, quant_type="INT", packed=False):
        assert quant_type in ["INT", "MXFP"], f"Invalid quant_type. Got {quant_type}, valid values are INT, MXFP."
        W_q, bias = _data(W_q), _data(bias)
        if quant_type == "INT":
            dtype = scales.dtype if self.dtype is None else self.dtype
            assert dtype in _FLOAT_DTYPES, "Invalid scales.dtype, should floating point."
            gl_dtype = TORCH_TO_DTYPE[dtype]
            scales, zeros = scales.to(dtype), zeros.to(dtype)
        else:
            assert W_nbits in [8, 4], "Unsupported W_nbit for MXFP quant_dtype."
            assert group_size == 32, "group_size should 32 for MXFP."
            if W_nbits == 8:
                assert W_q.dtype in [self.mx_fp8_dtype], f"Unsupported dtype of W_q. got {W_q.dtype}"
            else:
                assert W_q.dtype in [torch.uint8], f"Unsupported dtype of W_q. got {W_q.dtype}"
            dtype = torch.float16 if self.dtype is None else self.dtype
            if dtype == torch.float16:
                gl_dtype = DType.MXFP16
            elif dtype == torch.bfloat16:
                gl_dtype = DType.MXBF16
            else:
                raise Exception(f"Unsupported dtype for MXFP. Got {dtype}, supported [torch.float16, torch.bfloat16]")
            self.post_scale = False
            N, Kp = W_q.shape
            scales = scales.view(N, -1)
        in_features, out_features = W_q.shape[::-1]
        if packed:
            in_features = in_features * (8 // W_nbits) if quant_type == "MXFP" else scales.numel() * group_size // out_features
        W_q = W_q.to(self.device)
        scales = scales.to(device=self.device) if scales is not None else None
        zeros = zeros.to(device=self.device) if zeros is not None else None
        bias = bias.to(device=self.device, dtype=dtype) if bias is not None else None
        layer = GemLiteLinear(W_nbits, group_size=group_size, in_features=in_features, out_features=out_features,
                              input_dtype=gl_dtype, output_dtype=TORCH_TO_DTYPE[dtype] if quant_type == "MXFP" else gl_dtype,
                              scaled_activations=False)
        layer.pack(W_q, scales, zeros, bias=bias, packing_bitwidth=self.packing_bitwidth, packed=packed)
        if group_size == in_features and quant_type == "INT":
            if self.post_scale:
                layer.W_group_mode, layer.channel_scale_mode = 1, 1
            else:
                layer.W_group_mode, layer.channel_scale_mode = 3, 0
        return layer

    def from_hqqlinear(self, hqq_layer, del_orig=True):
        assert hqq_layer.meta["axis"] == 1, "Only axis==1 is supported."
        self.device = hqq_layer.W_q.device
        W_nbits, group_size = hqq_layer.meta["nbits"], hqq_layer.meta["group_size"]
        if group_size is None:
            group_size = hqq_layer.in_features
        W_q = hqq_layer.unpack(dtype=torch.uint8).view(hqq_layer.meta["shape"])   # uint8 codes
        scales, zeros = hqq_layer.meta["scale"].clone(), hqq_layer.meta["zero"].clone()
        bias = hqq_layer.bias.clone() if hqq_layer.bias is not None else None
        cleanup_linear(hqq_layer, del_orig)
        out = self.from_weights_(W_q=W_q, scales=scales, zeros=zeros, W_nbits=W_nbits, group_size=group_size, bias=bias, quant_type="INT")
        del W_q
        torch.cuda.empty_cache()
        return out

    def mxfp_from_linear(self, linear_layer, W_nbits, del_orig=True):
        if self.quantizer_mx is None:
            self.quantizer_mx = WeightQuantizerMXFP(device=self.device, compute_dtype=linear_layer.weight.dtype)
        W = linear_layer.weight.data
        bias = linear_layer.bias.clone() if linear_layer.bias is not None else None
        N, K = W.shape
        if W_nbits == 8:
            W_q, scales = self.quantizer_mx.quantize_mxfp8(W, index=True, mx_fp8_dtype=self.mx_fp8_dtype)
        else:
            W_q, scales = self.quantizer_mx.quantize_mxfp4(W, index=True)
        W_q, scales = W_q.view([N, K]), scales.view(N, K // 32)
        cleanup_linear(linear_layer, del_orig)
        return self.from_weights_(W_q=W_q, scales=scales, zeros=None, W_nbits=W_nbits, group_size=32, bias=bias, quant_type="MXFP")


class A16Wn_HQQ_INT(A16Wn):
    def __init__(self, device="cuda:0", dtype=None, W_nbits=None):
        super().__init__(device=device, dtype=dtype)
        self.W_nbits = W_nbits

    def from_packed_weights(self, W_q_packed, scales, zeros, bias=None):
        group_size = W_q_packed.numel() * (self.W_nbits // 4) // scales.numel()
        return super().from_packed_weights(W_q_packed, scales, zeros, self.W_nbits, group_size, bias=bias)

    def from_weights(self, W_q, scales, zeros, bias=None):
        group_size = W_q.numel() // scales.numel()
        return super().from_weights(W_q=W_q, scales=scales, zeros=zeros, W_nbits=self.W_nbits, group_size=group_size, bias=bias, quant_type="INT")


class A16W8_HQQ_INT(A16Wn_HQQ_INT):
    def __init__(self, device="cuda:0", dtype=None):
        super().__init__(device=device, dtype=dtype, W_nbits=8)


class A16W4_HQQ_INT(A16Wn_HQQ_INT):
    def __init__(self, device="cuda:0", dtype=None):
        super().__init__(device=device, dtype=dtype, W_nbits=4)


class A16W2_HQQ_INT(A16Wn_HQQ_INT):
    def __init__(self, device="cuda:0", dtype=None):
        super().__init__(device=device, dtype=dtype, W_nbits=2)


class A16W1_HQQ_INT(A16Wn_HQQ_INT):
    def __init__(self, device="cuda:0", dtype=None):
        super().__init__(device=device, dtype=dtype, W_nbits=1)


class A16Wn_MXFP(A16Wn):
    def __init__(self, device="cuda:0", dtype=None, W_nbits=None):
        super().__init__(device=device, dtype=dtype)
        self.W_nbits = W_nbits

    def from_packed_weights(self, W_q_packed, scales, bias=None):
        group_size = W_q_packed.numel() * (self.W_nbits // 4) // scales.numel()
        return A16Wn.from_packed_weights(self, W_q_packed, scales, zeros=None, W_nbits=self.W_nbits, group_size=group_size, bias=bias, quant_type="MXFP")

    def from_weights(self, W_q, scales, bias=None):
        group_size = W_q.numel() // scales.numel()
        return A16Wn.from_weights(self, W_q=W_q, scales=scales, zeros=None, W_nbits=self.W_nbits, group_size=group_size, bias=bias, quant_type="MXFP")

    def from_linear(self, linear_layer, del_orig=True):
        return self.mxfp_from_linear(linear_layer=linear_layer, W_nbits=self.W_nbits, del_orig=del_orig)


class A16W8_MXFP(A16Wn_MXFP):
    def __init__(self, device="cuda:0", dtype=None):
        super().__init__(device=device, dtype=dtype, W_nbits=8)


class A16W4_MXFP(A16Wn_MXFP):
    def __init__(self, device="cuda:0", dtype=None):
        super().__init__(device=device, dtype=dtype, W_nbits=4)


# ---------------------------------------------------------------------------------------------
# Block-scaled fp4 processors share everything but the numbers below
# ---------------------------------------------------------------------------------------------
class _FP4Processor:
    W_nbits = 4
    group_size = None           # 32 (MX) / 16 (NV)
    input_dtype = None
    scaled_activations = True
    scale_dtypes = ()

    def __init__(self, device="cuda:0", dtype=None):
        self.device, self.dtype = device, dtype
        self.quantizer_mx = None

    def _build(self, weight, bias, scales, packed):
        weight, bias = _data(weight), _data(bias)
        in_features, out_features = weight.shape[::-1]
        if packed:
            in_features *= 2   # packed bytes hold two codes
        assert scales is not None, "Scales parameter cannot be None. Use from_linear() call to pre-quantize the weights."
        assert weight.dtype in [torch.uint8], f"Invalid weight.dtype, should be uint8 fp4 codes, got {weight.dtype}."
        assert scales.dtype in self.scale_dtypes, f"Invalid scales.dtype {scales.dtype}, expected one of {self.scale_dtypes}."
        assert self.dtype is not None, "Input dtype should be either torch.float16 or torch.bfloat16, not None."
        W_q, scales = weight.to(device=self.device), scales.to(device=self.device)
        if self.group_size == 16 and scales.dtype == torch.uint8:
            scales = scales.view(torch.float8_e4m3fn)
        bias = bias.to(device=self.device, dtype=self.dtype) if bias is not None else None
        layer = GemLiteLinear(self.W_nbits, group_size=self.group_size, in_features=in_features, out_features=out_features,
                              input_dtype=self.input_dtype, output_dtype=TORCH_TO_DTYPE[self.dtype],
                              scaled_activations=self.scaled_activations)
        layer.pack(W_q, scales, zeros=None, bias=bias, packed=packed)
        return layer

    def _quantize(self, linear_layer):
        if self.dtype is None:
            self.dtype = linear_layer.weight.dtype
        if self.quantizer_mx is None:
            self.quantizer_mx = WeightQuantizerMXFP(device=self.device, compute_dtype=linear_layer.weight.dtype)
        W = linear_layer.weight.data
        bias = linear_layer.bias.clone() if linear_layer.bias is not None else None
        return W, bias


class A4W4_MXFP_dynamic(_FP4Processor):
    group_size, input_dtype = 32, DType.MXFP4
    scale_dtypes = (torch.float8_e8m0fnu, torch.uint8)

    def from_packed_weights(self, weight_packed, bias=None, scales=None):
        return self.from_weights(weight_packed, bias=bias, scales=scales, packed=True)

    def from_weights(self, weight, bias=None, scales=None, packed=False):
        layer = self._build(weight, bias, scales, packed)
        layer.W_group_mode, layer.channel_scale_mode = 0, 4
        return layer

    def from_linear(self, linear_layer, del_orig=True):
        W, bias = self._quantize(linear_layer)
        N, K = W.shape
        W_q, scales = self.quantizer_mx.quantize_mxfp4(W, index=True)
        cleanup_linear(linear_layer, del_orig)
        return self.from_weights(weight=W_q.view([N, K]), scales=scales.view(N, K // self.group_size), bias=bias)


class A4W4_NVFP_dynamic(_FP4Processor):
    group_size, input_dtype = 16, DType.NVFP4
    scale_dtypes = (torch.float8_e4m3fn, torch.uint8)

    def from_packed_weights(self, weight_packed, bias=None, scales=None, meta_scale=None, input_scale=None):
        return self.from_weights(weight_packed, bias=bias, scales=scales, meta_scale=meta_scale, input_scale=input_scale, packed=True)

    def from_weights(self, weight, bias=None, scales=None, meta_scale=None, input_scale=None, packed=False):
        layer = self._build(weight, bias, scales, packed)
        layer.W_group_mode, layer.channel_scale_mode = 0, 4
        dev = layer.W_q.device
        if meta_scale is not None:   # weight tensor scale 448*6/amax(W); forward multiplies by 1/(meta_w*meta_x)
            layer.meta_scale = torch.nn.Parameter(meta_scale.to(dtype=torch.float32, device=dev).reshape(()), requires_grad=False)
        if input_scale is not None:  # calibrated amax(x)/(448*6): skip the dynamic amax pass
            GEMLITE_NVFP4_INPUT_SCALES[layer.W_q.data_ptr()] = (1.0 / input_scale.to(dtype=torch.float32, device=dev).reshape(1)).contiguous()
        return layer

    def from_linear(self, linear_layer, del_orig=True):
        W, bias = self._quantize(linear_layer)
        N, K = W.shape
        W_q, scales, meta = self.quantizer_mx.quantize_nvfp4(W, index=True)
        cleanup_linear(linear_layer, del_orig)
        return self.from_weights(weight=W_q.view([N, K]), scales=scales.view(N, K // self.group_size), bias=bias, meta_scale=meta)


class A16W4_NVFP(_FP4Processor):
    """Weight-only NVFP4: fp16 / bf16 activations, e2m1 weights, e4m3 scale per 16 and a tensor scale."""
    group_size, input_dtype, scaled_activations = 16, DType.NVFP4, False
    scale_dtypes = (torch.float8_e4m3fn, torch.uint8)

    def from_packed_weights(self, weight_packed, bias=None, scales=None, meta_scale=None):
        return self.from_weights(weight_packed, bias=bias, scales=scales, meta_scale=meta_scale, packed=True)

    def from_weights(self, weight, bias=None, scales=None, meta_scale=None, packed=False):
        layer = self._build(weight, bias, scales, packed)
        if meta_scale is not None:   # W ~ code * scale / meta: the kernel multiplies by the stored 1/meta
            layer.meta_scale = torch.nn.Parameter((1.0 / meta_scale).to(dtype=torch.float32, device=layer.W_q.device).reshape(()), requires_grad=False)
        return layer

    def from_linear(self, linear_layer, del_orig=True):
        W, bias = self._quantize(linear_layer)
        N, K = W.shape
        W_q, scales, meta = self.quantizer_mx.quantize_nvfp4(W, index=True)
        cleanup_linear(linear_layer, del_orig)
        return self.from_weights(weight=W_q.view([N, K]), scales=scales.view(N, K // self.group_size), bias=bias, meta_scale=meta)


# ---------------------------------------------------------------------------------------------
# 8-bit dynamic activations
# ---------------------------------------------------------------------------------------------
class A8W8_dynamic:
    def __init__(self, device="cuda:0", dtype=None, fp8=False, fp32_scale=True, block_quant=False):
        self.device, self.dtype, self.fp8 = device, dtype, fp8
        self.fp32_scale, self.block_quant = fp32_scale, block_quant

    def from_weights(self, weight, bias=None, scales=None):
        weight, bias = _data(weight), _data(bias)
        if self.block_quant:
            return self._from_weights_block_quant(weight, bias=bias, scales=scales)
        w_dtype = self.fp8 if self.fp8 else torch.int8
        input_dtype = TORCH_TO_DTYPE[self.fp8] if self.fp8 else DType.INT8
        in_features, out_features = weight.shape[::-1]
        if scales is None:
            dtype = weight.dtype if self.dtype is None else self.dtype
            assert dtype in _FLOAT_DTYPES, "Invalid weight dtype, should be floating point."
            W_q, scales = _quantize_channelwise(weight, w_dtype, self.device)
        else:
            assert weight.dtype.itemsize == 1, "Invalid weight.dtype, should be 8-bit."
            dtype = self.dtype if self.dtype is not None else (scales.dtype if scales.dtype in (torch.float16, torch.bfloat16) else torch.float16)
            W_q, scales = weight.to(device=self.device), scales.to(device=self.device)
        scales = scales.to(torch.float32 if self.fp32_scale else dtype)
        bias = bias.to(device=self.device, dtype=dtype) if bias is not None else None
        layer = GemLiteLinear(8, group_size=in_features, in_features=in_features, out_features=out_features,
                              input_dtype=input_dtype, output_dtype=TORCH_TO_DTYPE[dtype], scaled_activations=True)
        layer.pack(W_q, scales, zeros=None, bias=bias)
        layer.W_group_mode, layer.channel_scale_mode = 0, 3   # acc * s_x[m] * s_w[n]
        return layer

    def _from_weights_block_quant(self, weight, bias=None, scales=None):
        """128 x 128 block quantisation of the weights with one fp32 scale per block, activations quantised per row and
        per 128 k in the forward (channel_scale_mode 5; gemlite/helper.py:517-617).  `scales` given: `weight` is already
        8-bit and `scales` is [ceil(N/128), ceil(K/128)]."""
        B = 128
        w_dtype = self.fp8 if self.fp8 else torch.int8
        input_dtype = TORCH_TO_DTYPE[self.fp8] if self.fp8 else DType.INT8
        info = torch.finfo(w_dtype) if w_dtype.is_floating_point else torch.iinfo(w_dtype)
        in_features, out_features = weight.shape[::-1]
        nb, kb = (out_features + B - 1) // B, (in_features + B - 1) // B
        if scales is not None:
            assert weight.dtype == w_dtype, f"Pre-quantized weight must be {w_dtype}, got {weight.dtype}"
            assert tuple(scales.shape) == (nb, kb), f"Pre-quantized scales must have shape {(nb, kb)}, got {tuple(scales.shape)}"
            W_q = weight.contiguous().to(device=self.device)
            scales = scales.to(device=self.device, dtype=torch.float32)
            dtype = self.dtype if self.dtype is not None else torch.bfloat16
        else:
            dtype = weight.dtype if self.dtype is None else self.dtype
            assert dtype in _FLOAT_DTYPES, "Invalid weight dtype, should be floating point."
            w = torch.zeros((nb * B, kb * B), dtype=torch.float32, device=self.device)
            w[:out_features, :in_features] = weight.to(dtype=torch.float32, device=self.device)
            blocks = w.view(nb, B, kb, B)
            scales = (blocks.abs().amax(dim=(1, 3)) / info.max).clamp_(min=1e-6)             # [N/B, K/B]
            W_q = (blocks / scales[:, None, :, None]).clamp_(min=info.min, max=info.max)
            W_q = W_q.to(w_dtype) if w_dtype.is_floating_point else W_q.round_().to(w_dtype)
            W_q = W_q.view(nb * B, kb * B)[:out_features, :in_features].contiguous()
        bias = bias.to(device=self.device, dtype=dtype) if bias is not None else None
        layer = GemLiteLinear(8, group_size=in_features, in_features=in_features, out_features=out_features,
                              input_dtype=input_dtype, output_dtype=TORCH_TO_DTYPE[dtype], acc_dtype=DType.FP32, scaled_activations=True)
        layer.pack(W_q, torch.ones((out_features, 1), dtype=torch.float32, device=self.device), zeros=None, bias=bias)
        # the block scales replace the placeholder: [K/B, N/B] fp32, block row of k first
        layer.scales = torch.nn.Parameter(scales.t().contiguous(), requires_grad=False)
        layer.meta_dtype = DType.FP32
        layer.W_group_mode, layer.channel_scale_mode = 0, 5
        return layer

    def from_linear(self, linear_layer, del_orig=True):
        out = self.from_weights(weight=linear_layer.weight, bias=linear_layer.bias)
        cleanup_linear(linear_layer, del_orig)
        return out


class A8W8_int8_dynamic(A8W8_dynamic):
    def __init__(self, device="cuda:0", dtype=None, block_quant=False):
        super().__init__(device=device, dtype=dtype, fp8=False, block_quant=block_quant)


class A8W8_fp8_dynamic(A8W8_dynamic):
    def __init__(self, device="cuda:0", dtype=None, fp8=default_fp8, block_quant=False):
        super().__init__(device=device, dtype=dtype, fp8=fp8, block_quant=block_quant)


A8W8_INT8_dynamic = A8W8_int8_dynamic
A8W8_FP8_dynamic = A8W8_fp8_dynamic


class A8Wn_MXFP_dynamic:
    """MXFP8 activations (dynamic) x MXFP8 / MXFP4 weights."""

    def __init__(self, device="cuda:0", dtype=None, post_scale=True, fp8=default_fp8, W_nbits=None):
        assert W_nbits is not None, "W_nbits argument should be either 8 or 4, not None."
        self.device, self.dtype, self.mx_fp8_dtype = device, dtype, fp8
        self.quantizer_mx, self.post_scale, self.W_nbits = None, post_scale, W_nbits

    def from_packed_weights(self, weight_packed, bias=None, scales=None):
        return self.from_weights(weight_packed, bias=bias, scales=scales, packed=True)

    def from_weights(self, weight, bias=None, scales=None, packed=False):
        weight, bias = _data(weight), _data(bias)
        in_features, out_features = weight.shape[::-1]
        if packed and self.W_nbits == 4:
            in_features *= 2
        assert scales is not None, "Scales parameter cannot be None. Use from_linear() call to pre-quantize the weights."
        if self.W_nbits == 8:
            assert weight.is_floating_point() and weight.itemsize == 1, f"Invalid weight.dtype, should be an fp8 dtype, got {weight.dtype}."
        else:
            assert weight.dtype in [torch.uint8], f"Invalid weight.dtype, should be uint8 fp4 codes, got {weight.dtype}."
        assert scales.dtype in [torch.float8_e8m0fnu, torch.uint8], f"Invalid scales.dtype, should be e8m0 / view(uint8), got {scales.dtype}."
        assert self.dtype is not None, "Input dtype should be either torch.float16 or torch.bfloat16, not None."
        W_q, scales = weight.to(device=self.device), scales.to(device=self.device)
        bias = bias.to(device=self.device, dtype=self.dtype) if bias is not None else None
        layer = GemLiteLinear(self.W_nbits, group_size=32, in_features=in_features, out_features=out_features,
                              input_dtype=DType.MXFP8, output_dtype=TORCH_TO_DTYPE[self.dtype], scaled_activations=True)
        layer.pack(W_q, scales, zeros=None, bias=bias, packed=packed)
        layer.W_group_mode = 0
        layer.channel_scale_mode = 2 if self.post_scale else 4   # per-token post-scale or MX micro-scales
        return layer

    def from_linear(self, linear_layer, del_orig=True):
        if self.dtype is None:
            self.dtype = linear_layer.weight.dtype
        if self.quantizer_mx is None:
            self.quantizer_mx = WeightQuantizerMXFP(device=self.device, compute_dtype=linear_layer.weight.dtype)
        W = linear_layer.weight.data
        bias = linear_layer.bias.clone() if linear_layer.bias is not None else None
        N, K = W.shape
        if self.W_nbits == 8:
            W_q, scales = self.quantizer_mx.quantize_mxfp8(W, index=True, mx_fp8_dtype=self.mx_fp8_dtype)
        else:
            W_q, scales = self.quantizer_mx.quantize_mxfp4(W, index=True)
        cleanup_linear(linear_layer, del_orig)
        return self.from_weights(weight=W_q.view([N, K]), scales=scales.view(N, K // 32), bias=bias)


class A8W8_MXFP_dynamic(A8Wn_MXFP_dynamic):
    def __init__(self, device="cuda:0", dtype=None, post_scale=True, fp8=default_fp8):
        super().__init__(device=device, dtype=dtype, post_scale=post_scale, fp8=fp8, W_nbits=8)


class A8W4_MXFP_dynamic(A8Wn_MXFP_dynamic):
    def __init__(self, device="cuda:0", dtype=None, post_scale=True, fp8=default_fp8):
        super().__init__(device=device, dtype=dtype, post_scale=post_scale, fp8=fp8, W_nbits=4)


# ---------------------------------------------------------------------------------------------
# the M buckets of get_closest_m, largest first
class A8Wn_HQQ_INT_dynamic(A16Wn):
    """FP8 activations quantised per token in the forward x packed 8/4/2-bit codes with group-wise scales and zeros
    (gemlite/helper.py:712-830): `pack(..., fma_mode=False)`, so grouped layers run mode 3 `(q - z) * s` with the
    activation scale on the finished sums (channel mode 2); one group per row folds the weight scale into the epilogue
    when `post_scale` is set (modes 1 / 3)."""

    def __init__(self, device="cuda:0", packing_bitwidth=None, dtype=None, post_scale=default_post_scale, fp8=default_fp8,
                 fp32_scale=False, W_nbits=None):
        assert W_nbits is not None, "W_nbits argument should be either 8, 4 or 2, not None."
        super().__init__(device=device, dtype=dtype, packing_bitwidth=packing_bitwidth, post_scale=post_scale)
        self.fp8, self.fp32_scale, self.W_nbits = fp8, fp32_scale, W_nbits

    def from_packed_weights(self, W_q_packed, scales, zeros, bias=None):
        group_size = W_q_packed.numel() * (self.W_nbits // 4) // scales.numel()
        return self.from_weights_(W_q_packed, scales, zeros, self.W_nbits, group_size, bias=bias, packed=True)

    def from_weights(self, W_q, scales, zeros, bias=None):
        return self.from_weights_(W_q, scales, zeros, self.W_nbits, W_q.numel() // scales.numel(), bias=bias)

    def from_weights_(self, W_q, scales, zeros, W_nbits, group_size, bias=None, quant_type="INT", packed=False):
        assert quant_type == "INT", "dynamic FP8 activations take integer codes"
        W_q, bias = _data(W_q), _data(bias)
        dtype = self.dtype if self.dtype is not None else (scales.dtype if scales.dtype in (torch.float16, torch.bfloat16) else torch.float16)
        assert dtype in _FLOAT_DTYPES, "Invalid scales.dtype, should be floating point."
        in_features, out_features = W_q.shape[::-1]
        if packed:
            in_features = scales.numel() * group_size // out_features
        layer = GemLiteLinear(W_nbits, group_size=group_size, in_features=in_features, out_features=out_features,
                              input_dtype=TORCH_TO_DTYPE[self.fp8], output_dtype=TORCH_TO_DTYPE[dtype], scaled_activations=True)
        layer.pack(W_q.to(self.device),
                   scales.to(device=self.device, dtype=torch.float32 if self.fp32_scale else dtype) if scales is not None else None,
                   zeros.to(device=self.device, dtype=dtype) if zeros is not None else None,
                   bias=bias.to(device=self.device, dtype=dtype) if bias is not None else None,
                   packing_bitwidth=self.packing_bitwidth, fma_mode=False, packed=packed)
        if group_size == in_features:
            layer.W_group_mode, layer.channel_scale_mode = (1, 3) if self.post_scale else (3, 2)
        return layer


class A8W4_HQQ_INT_dynamic(A8Wn_HQQ_INT_dynamic):
    def __init__(self, device="cuda:0", packing_bitwidth=None, dtype=None, post_scale=default_post_scale, fp8=default_fp8, fp32_scale=False):
        super().__init__(device, packing_bitwidth, dtype, post_scale, fp8, fp32_scale, W_nbits=4)


class A8W2_HQQ_INT_dynamic(A8Wn_HQQ_INT_dynamic):
    def __init__(self, device="cuda:0", packing_bitwidth=None, dtype=None, post_scale=default_post_scale, fp8=default_fp8, fp32_scale=False):
        super().__init__(device, packing_bitwidth, dtype, post_scale, fp8, fp32_scale, W_nbits=2)


class _Ternary:
    """BitNet layers (gemlite/helper.py:1208-1320): weights in {-1, 0, 1} stored as 2-bit codes w + 1 with the scalar
    zero 1 (mode 1, shift only) and one tensor-wide weight scale applied to the finished sums."""
    input_int8 = False

    def __init__(self, device="cuda:0", dtype=None, fp32_scale=True):
        self.device, self.dtype, self.fp32_scale = device, dtype, fp32_scale

    def from_weights(self, weight, weight_scale, bias=None):
        weight, bias = _data(weight), _data(bias)
        dtype = weight.dtype if self.dtype is None else self.dtype
        assert dtype in _FLOAT_DTYPES, "Invalid weight.dtype, should be floating point."
        codes = (weight.to(device=self.device, dtype=dtype) + 1).to(torch.uint8)
        out_features, in_features = codes.shape
        scales = torch.full((out_features, 1), float(weight_scale.item() if hasattr(weight_scale, "item") else weight_scale),
                            dtype=torch.float32 if self.fp32_scale else dtype, device=self.device)
        layer = GemLiteLinear(2, group_size=in_features, in_features=in_features, out_features=out_features,
                              input_dtype=DType.INT8 if self.input_int8 else TORCH_TO_DTYPE[dtype],
                              output_dtype=TORCH_TO_DTYPE[dtype], scaled_activations=self.input_int8)
        layer.pack(codes, scales=scales, zeros=1, bias=bias.to(device=self.device, dtype=dtype) if bias is not None else None)
        layer.W_group_mode = 1                                   # shift only
        layer.channel_scale_mode = 3 if self.input_int8 else 1   # activation and weight scales / weight scale, after the sum
        return layer

    def from_bitlinear(self, linear_layer, del_orig=True):
        out = self.from_weights(linear_layer.weight, linear_layer.weight_scale, bias=linear_layer.bias)
        cleanup_linear(linear_layer, del_orig)
        return out


class A16W158_INT(_Ternary):
    input_int8 = False


class A8W158_INT_dynamic(_Ternary):
    input_int8 = True


default_batch_sizes = [4096, 3072, 2048, 1536, 1024, 768, 512, 384, 256, 192, 128, 96, 64, 48, 32, 24, 16, 8, 4, 2, 1]


def warmup(processor, shapes, batch_sizes=default_batch_sizes, group_size=64, dtype=torch.float16):
    """Run every (shape, batch size) once so that workspaces exist and kernels are loaded before
    CUDA-graph capture.  There is nothing to autotune; this takes milliseconds."""
    device = torch.device(torch.cuda.current_device())
    for out_features, in_features in shapes:
        linear = torch.nn.Linear(in_features=in_features, out_features=out_features, bias=False, dtype=dtype, device=device)
        if hasattr(processor, "from_hqqlinear"):
            from hqq.core.quantize import HQQLinear, BaseQuantizeConfig   # optional dependency
            cfg = BaseQuantizeConfig(nbits=processor.W_nbits, group_size=group_size, axis=1)
            layer = processor.from_hqqlinear(HQQLinear(linear, quant_config=cfg, compute_dtype=dtype, device=device))
        else:
            layer = processor.from_linear(linear)
        for bs in batch_sizes:
            layer(torch.randn((bs, in_features), dtype=dtype, device=device) / 100.0)
        torch.cuda.synchronize()
        del layer
        torch.cuda.empty_cache()
        gc.collect()
