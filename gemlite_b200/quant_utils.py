"""Activation quantisation front ends and the offline MX / NV weight quantiser.

``scale_activations_*`` keep the reference's names and return values
(gemlite/quant_utils.py:2680-2684) and run as CUDA kernels through the C ABI.
``WeightQuantizerMXFP`` is offline torch code (it prepares weights once, it is not on the
matmul path) with the arithmetic of gemlite/quant_utils.py:75-232; it works on any device.
"""
from typing import Tuple

import torch
from torch import Tensor

from . import _lib
from .dtypes import TORCH_TO_DTYPE, DType

_FP4_POS = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
_FP4_THRESHOLDS = [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0]  # midpoints between representable magnitudes
_FP4_VALUES = _FP4_POS + [-v for v in _FP4_POS]             # code -> value, sign in bit 3


def get_dtype_range(compute_dtype: torch.dtype):
    info = torch.finfo(compute_dtype) if compute_dtype.is_floating_point else torch.iinfo(compute_dtype)
    return info.min, info.max


# ------------------------------------------------------------------------------------------
# Offline weight quantiser (gemlite/quant_utils.py:75-232)
# ------------------------------------------------------------------------------------------
class WeightQuantizerMXFP:
    def __init__(self, compute_dtype=torch.bfloat16, device="cuda:0"):
        self.compute_dtype = compute_dtype
        self.device = device

    @staticmethod
    def round_to_closest_fp4(tensor):
        """Nearest E2M1 magnitude, ties to the smaller one (left bisect on the midpoints)."""
        thr = torch.tensor(_FP4_THRESHOLDS, dtype=tensor.dtype, device=tensor.device)
        pos = torch.tensor(_FP4_POS, dtype=tensor.dtype, device=tensor.device)
        out = pos[torch.searchsorted(thr, tensor.abs().contiguous())]
        return out * tensor.sign()

    @staticmethod
    def to_index(W_q):
        """E2M1 codes of fp4-valued floats; -0.0 maps to code 0 like +0.0 (first match)."""
        assert W_q.is_floating_point(), "Input should be floating point fp4 values."
        vals = torch.tensor(_FP4_VALUES, dtype=W_q.dtype, device=W_q.device)
        return (W_q.reshape(-1, 1) == vals.view(1, -1)).to(torch.uint8).argmax(dim=1).to(torch.uint8).view(W_q.shape)

    def quantize_mxfp8(self, W, index=False, mx_fp8_dtype=torch.float8_e4m3fn):
        group_size, eps = 32, 2.0 ** -30
        min_val, max_val = get_dtype_range(mx_fp8_dtype)
        W_flat = W.reshape(-1, group_size).float()
        ideal = W_flat.abs().amax(dim=1, keepdim=True) / max_val
        scales = (2 ** torch.ceil(torch.log2(ideal))).clamp_(min=eps)
        W_q = (W_flat / scales).clamp_(min=min_val, max=max_val).to(mx_fp8_dtype)
        if not index:
            W_q = W_q.to(W_flat.dtype)
        return W_q, scales.to(torch.float8_e8m0fnu)

    def quantize_mxfp4(self, W, window_size: int = 0, index=False):
        group_size, eps, max_val = 32, 2.0 ** -30, 6
        W_flat = W.reshape(-1, group_size).float()
        ideal = W_flat.abs().amax(dim=1, keepdim=True) / max_val
        log2s = torch.ceil(torch.log2(ideal))
        if window_size == 0:
            scales = 2 ** log2s
        else:
            offs = torch.arange(-window_size, window_size + 1, device=W.device, dtype=log2s.dtype).view(1, -1)
            cand = torch.pow(2, log2s + offs)
            cand[cand < eps] = eps
            W_r = self.round_to_closest_fp4(W_flat.unsqueeze(1) / cand.unsqueeze(-1)) * cand.unsqueeze(-1)
            err = (W_flat.unsqueeze(1) - W_r).abs().mean(dim=-1)
            scales = torch.gather(cand, 1, torch.argmin(err, dim=1, keepdim=True))
        scales = scales.clamp_(eps)
        W_q = self.round_to_closest_fp4(W_flat / scales)
        if index:
            W_q = self.to_index(W_q)
        return W_q, scales.to(torch.float8_e8m0fnu)

    def quantize_nvfp4(self, W, window_size: int = 0, index=False):
        group_size, eps, max_val = 16, 1e-6, 6
        fp8_dtype = torch.float8_e4m3fn
        max_fp8 = torch.finfo(fp8_dtype).max  # 448
        W_flat = W.reshape(-1, group_size).float()
        ideal = W_flat.abs().amax(dim=1, keepdim=True) / max_val
        meta_scales = (max_fp8 / ideal.max().clamp_(min=eps)).float()
        ideal = (ideal * meta_scales).clamp_(max=max_fp8).to(fp8_dtype)
        if window_size == 0:
            scales = ideal
        else:
            offs = torch.arange(-window_size, window_size + 1, device=W.device, dtype=torch.int).view(1, -1)
            cand = (ideal.view(torch.int8) + offs).clamp_(-128, 127).to(torch.int8)
            cand[cand == -1] = 1   # 0xFF and 0x7F are the e4m3 NaN patterns
            cand[cand == 127] = 1
            cand = cand.view(fp8_dtype).float()
            cand[cand < eps] = eps
            W_r = self.round_to_closest_fp4(W_flat.unsqueeze(1) * (meta_scales / cand).unsqueeze(-1)) * (cand / meta_scales).unsqueeze(-1)
            err = (W_flat.unsqueeze(1) - W_r).abs().mean(dim=-1)
            scales = torch.gather(cand, 1, torch.argmin(err, dim=1, keepdim=True)).to(fp8_dtype)
        scales_full = (scales.to(W_flat.dtype) / meta_scales).clamp_(min=eps)
        W_q = self.round_to_closest_fp4(W_flat / scales_full)
        if index:
            W_q = self.to_index(W_q)
        return W_q, scales, meta_scales

    def dequantize(self, W_q, scales, shape=None, dtype=None, meta_scales=None):
        if W_q.dtype == torch.uint8:
            W_q = torch.tensor(_FP4_VALUES, dtype=torch.float32, device=W_q.device)[W_q.int()]
        group_size = W_q.numel() // scales.numel()
        out = W_q.reshape(-1, group_size).float() * scales.float().reshape(-1, 1)
        if meta_scales is not None:
            out = out * meta_scales
        if shape is not None:
            out = out.view(shape)
        return out.to(self.compute_dtype if dtype is None else dtype)


# ------------------------------------------------------------------------------------------
# Dynamic activation quantisation (CUDA, via the C ABI)
# ------------------------------------------------------------------------------------------
def _as_2d(tensor):
    _lib.require_cuda(tensor, "activations")
    shape = tensor.shape
    t = tensor.contiguous().view(-1, shape[-1])
    if t.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        raise NotImplementedError("activation dtype %s is not supported" % t.dtype)
    return t, shape


def scale_activations_per_token(tensor: Tensor, w_dtype: torch.dtype, fp32_scale: bool = True) -> Tuple[Tensor, Tensor]:
    """Per-row symmetric quantisation to fp8 e4m3 / int8: returns (q like tensor, scales fp32 [M, 1]).

    Replaces scale_activations_per_token_triton_v3 (gemlite/quant_utils.py:510-539)."""
    if w_dtype not in (torch.float8_e4m3fn, torch.int8):
        raise NotImplementedError("per-token activation quantisation supports float8_e4m3fn and int8, got %s" % w_dtype)
    x, shape = _as_2d(tensor)
    M, K = x.shape
    q = torch.empty((M, K), dtype=w_dtype, device=x.device)
    scales = torch.empty((M, 1), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().gl_scale_activations_per_token(
            x.data_ptr(), q.data_ptr(), scales.data_ptr(), M, K, TORCH_TO_DTYPE[x.dtype].value,
            DType.INT8.value if w_dtype == torch.int8 else DType.FP8.value, _lib.current_stream_ptr(x.device)))
    if not fp32_scale:
        scales = scales.to(tensor.dtype)
    return q.view(shape), scales


def scale_activations_per_token_torch(tensor: Tensor, w_dtype: torch.dtype, fp32_scale: bool = True) -> Tuple[Tensor, Tensor]:
    """The same quantiser in plain torch ops (gemlite/quant_utils.py:261-283): callers and tests of the reference use
    it as the comparison point for the kernel.  Rows are scaled by amax / qmax (at least 1e-6), clamped, and rounded
    for integer targets."""
    lo, hi = get_dtype_range(w_dtype)
    t = tensor.to(torch.float32) if fp32_scale else tensor
    rows = t.reshape(-1, t.shape[-1])
    scales = rows.abs().amax(dim=1, keepdim=True).div(hi).clamp(min=1e-6)
    q = (rows / scales).clamp(lo, hi)
    if not w_dtype.is_floating_point:
        q = q.round()
    return q.to(w_dtype).view(tensor.shape), scales


def _scale_buffer(M, G, pad, scale_layout, dtype, device):
    """Row layout [ceil_pad(M), G] (what the reference returns) or, for scale_layout=1, the 128x4 scale
    atoms the block-scaled tensor-core kernel reads: [ceil128(M)/128, G/4, 512] bytes."""
    if scale_layout == 0:
        return torch.empty(((M + pad - 1) // pad * pad, G), dtype=dtype, device=device)
    return torch.empty(((M + 127) // 128, G // 4, 512), dtype=dtype, device=device)


def scale_activations_mxfp8(tensor: Tensor, w_dtype: torch.dtype = torch.float8_e4m3fn, scale_layout: int = 0) -> Tuple[Tensor, Tensor]:
    """MXFP8: (q e4m3 like tensor, e8m0 scale bytes uint8 [ceil32(M), K/32]).  quant_utils.py:1095-1124."""
    if w_dtype != torch.float8_e4m3fn:
        raise NotImplementedError("MXFP8 activations are e4m3 only")
    x, shape = _as_2d(tensor)
    M, K = x.shape
    q = torch.empty((M, K), dtype=w_dtype, device=x.device)
    scales = _scale_buffer(M, K // 32, 32, scale_layout, torch.uint8, x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().gl_scale_activations_mxfp8(x.data_ptr(), q.data_ptr(), scales.data_ptr(), M, K,
                                                        TORCH_TO_DTYPE[x.dtype].value, scale_layout, _lib.current_stream_ptr(x.device)))
    return q.view(shape), scales


def scale_activations_mxfp4(tensor: Tensor, scale_layout: int = 0) -> Tuple[Tensor, Tensor]:
    """MXFP4: (q uint8 [M, K/2] e2m1 pairs, e8m0 scale bytes uint8 [ceil32(M), K/32]).  quant_utils.py:2107-2135."""
    x, _ = _as_2d(tensor)
    M, K = x.shape
    q = torch.empty((M, K // 2), dtype=torch.uint8, device=x.device)
    scales = _scale_buffer(M, K // 32, 32, scale_layout, torch.uint8, x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().gl_scale_activations_mxfp4(x.data_ptr(), q.data_ptr(), scales.data_ptr(), M, K,
                                                        TORCH_TO_DTYPE[x.dtype].value, scale_layout, _lib.current_stream_ptr(x.device)))
    return q, scales


# ---- the block-scaled quantisers in plain torch ops (any device): the comparison points the reference keeps beside its
# kernels (gemlite/quant_utils.py:712-747, 1131-1175, 1177-1224), here with the arithmetic of the active kernels so that
# codes and scale bytes agree bit for bit with `scale_activations_mx*` / `_nvfp4` above (row layout of the scales).
_E2M1_MIDPOINTS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)


def _pow2_ceil_exponent(v: Tensor) -> Tensor:
    """Biased exponent of 2^ceil(log2 v), clamped to [2^-30, 2^127], from the fp32 bit pattern (quant_utils.py:697-705)."""
    bits = v.to(torch.float32).contiguous().view(torch.int32)
    e = ((bits >> 23) & 0xFF) + ((bits & 0x7FFFFF) != 0).to(torch.int32)
    return e.clamp(127 - 30, 254)


def _e2m1_codes(v: Tensor) -> Tensor:
    """e2m1 code of every value: the number of midpoints it exceeds, sign in bit 3 (quant_utils.py:66-73, 2081-2090)."""
    a = v.abs()
    idx = torch.zeros_like(v, dtype=torch.int32)
    for t in _E2M1_MIDPOINTS:
        idx += (a > t).to(torch.int32)
    return torch.where(v >= 0, idx, idx + 8).to(torch.uint8)


def _pad_rows(rows: int, pad: int) -> int:
    return (rows + pad - 1) // pad * pad


def scale_activations_mxfp8_torch(tensor: Tensor, w_dtype: torch.dtype = torch.float8_e4m3fn) -> Tuple[Tensor, Tensor]:
    x = tensor.reshape(-1, tensor.shape[-1]).to(torch.float32)
    M, K = x.shape
    g = x.view(M, K // 32, 32)
    e = _pow2_ceil_exponent(g.abs().amax(-1) / 448.0)
    scale = (e << 23).view(torch.float32)
    q = (g / scale.unsqueeze(-1)).clamp(-448.0, 448.0).to(w_dtype).view(tensor.shape)
    scales = torch.full((_pad_rows(M, 32), K // 32), 127, dtype=torch.uint8, device=x.device)
    scales[:M] = e.to(torch.uint8)
    return q, scales


def scale_activations_mxfp4_torch(tensor: Tensor) -> Tuple[Tensor, Tensor]:
    x = tensor.reshape(-1, tensor.shape[-1]).to(torch.float32)
    M, K = x.shape
    g = x.view(M, K // 32, 32)
    e = _pow2_ceil_exponent(g.abs().amax(-1) / 6.0)
    scale = (e << 23).view(torch.float32)
    codes = _e2m1_codes(g / scale.unsqueeze(-1)).view(M, K)
    q = codes[:, 0::2] | (codes[:, 1::2] << 4)
    scales = torch.full((_pad_rows(M, 32), K // 32), 127, dtype=torch.uint8, device=x.device)
    scales[:M] = e.to(torch.uint8)
    return q, scales


def scale_activations_nvfp4_torch(tensor: Tensor, meta_scale=None) -> Tuple[Tensor, Tensor, Tensor]:
    x = tensor.reshape(-1, tensor.shape[-1]).to(torch.float32)
    M, K = x.shape
    if meta_scale is None:
        meta = torch.tensor(448.0 * 6.0, dtype=torch.float32, device=x.device) / x.abs().amax().clamp(min=1e-6)
    else:
        meta = torch.as_tensor(meta_scale, dtype=torch.float32, device=x.device).reshape(())
    g = x.view(M, K // 16, 16)
    s8 = ((g.abs().amax(-1) * meta) / 6.0).clamp(max=448.0).to(torch.float8_e4m3fn)
    full = (s8.to(torch.float32) / meta).clamp(min=1e-6)
    codes = _e2m1_codes(g / full.unsqueeze(-1)).view(M, K)
    q = codes[:, 0::2] | (codes[:, 1::2] << 4)
    scales = torch.full((_pad_rows(M, 16), K // 16), 1.0, dtype=torch.float32, device=x.device).to(torch.float8_e4m3fn)
    scales[:M] = s8
    return q, scales, meta.reshape(1)


_NVFP4_SCRATCH = {}


def _nvfp4_scratch(device):
    """4 bytes per (device, stream) for the tensor-wide amax (allocated on first use, outside any graph capture): two
    layers quantising on different streams of one GPU must not share the cell."""
    key = (device.type, device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _NVFP4_SCRATCH.get(key)
    if buf is None:
        buf = torch.zeros(1, dtype=torch.int32, device=device)
        _NVFP4_SCRATCH[key] = buf
    return buf


def scale_activations_nvfp4(tensor: Tensor, meta_scale=None, scale_layout: int = 0) -> Tuple[Tensor, Tensor, Tensor]:
    """NVFP4: (q uint8 [M, K/2], e4m3 scales [ceil16(M), K/16], fp32 tensor scale [1]).

    ``meta_scale`` (device fp32 tensor) switches to the static-scale path.  quant_utils.py:2434-2493."""
    x, _ = _as_2d(tensor)
    M, K = x.shape
    q = torch.empty((M, K // 2), dtype=torch.uint8, device=x.device)
    scales = _scale_buffer(M, K // 16, 16, scale_layout, torch.float8_e4m3fn, x.device)
    meta_out = torch.empty(1, dtype=torch.float32, device=x.device)
    meta_in = None
    if meta_scale is not None:
        meta_in = meta_scale.to(device=x.device, dtype=torch.float32).reshape(-1)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().gl_scale_activations_nvfp4(
            x.data_ptr(), q.data_ptr(), scales.data_ptr(), meta_out.data_ptr(),
            None if meta_in is None else meta_in.data_ptr(), _nvfp4_scratch(x.device).data_ptr(),
            M, K, TORCH_TO_DTYPE[x.dtype].value, scale_layout, _lib.current_stream_ptr(x.device)))
    return q, scales, meta_out


BLOCK_QUANT_SIZE = 128   # gemlite/triton_kernels/config.py


def scale_activations_per_block(tensor: Tensor, w_dtype: torch.dtype, block_size: int = BLOCK_QUANT_SIZE) -> Tuple[Tensor, Tensor]:
    """One scale per row and per 128 consecutive k (the activation side of 128 x 128 block quantisation): returns
    (q like tensor, scales fp32 [M, K / 128]).  Replaces scale_activations_per_block (gemlite/quant_utils.py:2504-2590)."""
    if w_dtype not in (torch.float8_e4m3fn, torch.int8):
        raise NotImplementedError("per-block activation quantisation supports float8_e4m3fn and int8, got %s" % w_dtype)
    if block_size != BLOCK_QUANT_SIZE:
        raise NotImplementedError("per-block activation quantisation uses blocks of %d" % BLOCK_QUANT_SIZE)
    x, shape = _as_2d(tensor)
    M, K = x.shape
    assert K % block_size == 0, "K must be divisible by block_size for per-block activation quantization."
    q = torch.empty((M, K), dtype=w_dtype, device=x.device)
    scales = torch.empty((M, K // block_size), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().gl_scale_activations_per_block(
            x.data_ptr(), q.data_ptr(), scales.data_ptr(), M, K, TORCH_TO_DTYPE[x.dtype].value,
            DType.INT8.value if w_dtype == torch.int8 else DType.FP8.value, _lib.current_stream_ptr(x.device)))
    return q.view(shape), scales


def scale_activations_per_block_torch(tensor: Tensor, w_dtype: torch.dtype, block_size: int = BLOCK_QUANT_SIZE) -> Tuple[Tensor, Tensor]:
    """The same quantiser in plain torch ops (gemlite/quant_utils.py:2504-2522), the comparison point of the kernel."""
    lo, hi = get_dtype_range(w_dtype)
    rows = tensor.to(torch.float32).reshape(-1, tensor.shape[-1])
    M, K = rows.shape
    assert K % block_size == 0, "K must be divisible by block_size for per-block activation quantization."
    t = rows.view(M, K // block_size, block_size)
    scales = (t.abs().amax(dim=-1) / hi).clamp_(min=1e-6)
    q = (t / scales.unsqueeze(-1)).clamp_(lo, hi)
    if not w_dtype.is_floating_point:
        q = q.round_()
    return q.to(w_dtype).view(tensor.shape), scales.contiguous()
