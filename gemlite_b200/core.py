"""``GemLiteLinear``: the module-level API of the reference (gemlite/core.py) over the sm_100a
CUDA library.

What is kept from the reference, because callers and checkpoints depend on it:
constructor arguments and validation (core.py:310-389), ``pack()`` and the
``W_group_mode`` / ``channel_scale_mode`` it selects (core.py:559-795), the serialized schema
``W_q, scales, zeros, metadata, orig_shape, meta_scale[, bias]`` (core.py:379-554), the
12-integer ``get_meta_args()`` list (core.py:804-817), the custom op
``gemlite::forward_functional`` (core.py:193-285), the kernel-family names for
``forward_manual`` (core.py:57-67) and the global setters exported by ``gemlite/__init__.py``.

What is different: every device computation is one call into ``libgemlite_b200.so``; there is
no Triton, no autotuner and no CPU path (a CPU tensor raises).  Bias is fused into the matmul
kernel.
"""
import ctypes
import json
import logging
import os
import threading
from typing import List, Union

import torch
from torch import Tensor

from . import _lib
from .bitpack import pack_weights_over_cols
from .dtypes import (DType, DTYPE_TO_TORCH, TORCH_TO_DTYPE, FP8_INT8_DTYPES, is_mx_dtype)
from .quant_utils import (scale_activations_per_token, scale_activations_per_block, scale_activations_mxfp8,
                          scale_activations_mxfp4, scale_activations_nvfp4)

logger = logging.getLogger(__name__)
FILE_LOCK = threading.Lock()

# Accumulator dtype per input dtype (core.py:40-55); reported in the metadata only: the CUDA
# kernels always accumulate in fp32 (int32 for INT8 x INT8).
GEMLITE_ACC_DTYPE = {
    DType.FP16: DType.FP32, DType.BF16: DType.FP32, DType.FP32: DType.FP32, DType.FP8: DType.FP32,
    DType.FP8e4: DType.FP32, DType.FP8e4nuz: DType.FP32, DType.FP8e5: DType.FP32, DType.FP8e5nuz: DType.FP32,
    DType.INT8: DType.INT32, DType.MXFP16: DType.FP32, DType.MXBF16: DType.FP32, DType.MXFP8: DType.FP32,
    DType.MXFP4: DType.FP32, DType.NVFP4: DType.FP32,
}

GEMLITE_MATMUL_TYPES = ["GEMV", "GEMV_REVSPLITK", "GEMV_SPLITK", "GEMM_SPLITK", "GEMM"]
GEMLITE_MATMUL_TYPES_MAPPING = {name: i for i, name in enumerate(GEMLITE_MATMUL_TYPES)}
GEMLITE_USE_TMA = False              # the 5-D pre-shuffled MX scale layout of the reference is never produced
GEMLITE_ENABLE_PTX_FP4_PACK = False
GEMLITE_FAST_NVFP4 = False
GEMLITE_NVFP4_META_SCALES = []       # per-GPU static activation tensor scales (set_fast_nvfp4)
GEMLITE_NVFP4_INPUT_SCALES = {}      # per-layer calibrated scale, keyed by W_q.data_ptr()


# ---------------------------------------------------------------------------------------------
# Global setters (gemlite/core.py:91-160, triton_kernels/config.py:49-68).  The knobs that steered
# Triton code generation have nothing to steer here; they are accepted and recorded.
# ---------------------------------------------------------------------------------------------
_SETTINGS = {"autotune": "fast", "kernel_caching": False, "acc_dtype": DType.FP32, "warp_specialize": False,
             "native_atomic_bf16": True, "fast_gemv_acc": False}


def set_autotune(mode="fast", **kwargs):
    """Recorded only: tile parameters come from the config cache / built-in heuristics."""
    _SETTINGS["autotune"] = mode


def set_autotune_setting(fct):
    """Override the M-bucket function used in config-cache signatures (core.py:92-93)."""
    global _closest_m_override
    _closest_m_override = fct


def set_packing_bitwidth(packing_bitwidth: int):
    GemLiteLinear.PACKING_BITWIDTH = packing_bitwidth


def set_acc_dtype(dtype):
    assert dtype in [DType.FP16, DType.FP32], "Invalid dtype (should be DType.FP16 or DType.FP32)."
    _SETTINGS["acc_dtype"] = dtype   # fp16 accumulation is not offered on sm_100a; metadata keeps fp32


def enable_tma(enabled: bool = True):
    _SETTINGS["tma"] = enabled       # tensor-core kernels always use TMA; scale layout stays 2-D


def enable_warp_specialize(enabled: bool = True):
    _SETTINGS["warp_specialize"] = enabled


def set_native_atomic_bfp16(enabled: bool = True):
    _SETTINGS["native_atomic_bf16"] = enabled   # no atomics in the CUDA kernels


def set_fast_gemv_acc(enabled: bool = True):
    _SETTINGS["fast_gemv_acc"] = enabled


def set_ptx_fp4_pack(enabled: bool = True):
    global GEMLITE_ENABLE_PTX_FP4_PACK
    GEMLITE_ENABLE_PTX_FP4_PACK = enabled       # threshold rounding is always used (ties to the smaller magnitude)


def set_kernel_caching(enabled: bool = True):
    _SETTINGS["kernel_caching"] = enabled       # the output ring existed for atomics; outputs are written once here


def enable_cudagraph_autotune(enabled: bool = True):
    set_autotune("fast", use_cuda_graph=enabled)


def set_fast_nvfp4(enabled: bool = True, default_value: float = 448.0):
    """Static activation tensor scale for NVFP4 (skips the dynamic amax pass), core.py:149-157."""
    global GEMLITE_FAST_NVFP4, GEMLITE_NVFP4_META_SCALES
    GEMLITE_FAST_NVFP4 = enabled
    if enabled and len(GEMLITE_NVFP4_META_SCALES) == 0:
        GEMLITE_NVFP4_META_SCALES = [
            torch.full((1,), fill_value=default_value, device="cuda:%d" % i, dtype=torch.float32)
            for i in range(torch.cuda.device_count())
        ]


_closest_m_override = None


def get_closest_m(M: int) -> int:
    if _closest_m_override is not None:
        return _closest_m_override(M)
    return int(_lib.lib().gl_get_closest_m(int(M)))


def get_default_gemv(W_nbits: int, mx_dtype: bool = False) -> str:
    if mx_dtype:
        return "GEMM_SPLITK"
    return "GEMV_REVSPLITK" if (W_nbits < 8) else "GEMV_SPLITK"


def get_matmul_type(batch_size: int, W_nbits: int, mx_dtype: bool = False) -> str:
    """Kernel family for a batch size (core.py:171-179); evaluated by the C library."""
    return GEMLITE_MATMUL_TYPES[_lib.lib().gl_get_matmul_type(int(batch_size), int(W_nbits), int(bool(mx_dtype)))]


def enable_activation_scaling(batch_size):
    return True


# ---------------------------------------------------------------------------------------------
# Workspace (split-K partial sums + arrival counters).  Allocated once per (device, stream) and
# grown on demand, never inside the C library.  Its counter head must be zero on first use.
# ---------------------------------------------------------------------------------------------
_WORKSPACES = {}
# 1 routes every matmul to the general CUDA-core kernel (tests compare kernels with it), 2 to the tensor-core kernel
# wherever it covers the problem (decode sizes included)
_KERNEL_OVERRIDE = int(os.environ.get("GEMLITE_B200_KERNEL_OVERRIDE", "0"))


def set_kernel_override(value: int):
    global _KERNEL_OVERRIDE
    _KERNEL_OVERRIDE = int(value)



def _workspace(device, nbytes, stream_ptr=None):
    if nbytes == 0:
        return None
    key = (device.index, _lib.current_stream_ptr(device) if stream_ptr is None else stream_ptr)
    ws = _WORKSPACES.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(int(nbytes), 8 << 20), dtype=torch.uint8, device=device)
        _WORKSPACES[key] = ws
    return ws


def matmul_status(device=None, clear: bool = True) -> int:
    """Status word of the tensor-core kernels for the current stream's workspace on `device`: 0 after clean launches,
    else the code of the bounded wait that gave up (the outputs of that launch are undefined).  Synchronises the
    stream.  With `clear`, a non-zero status re-zeroes the workspace's counter block so that it can be used again."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    L = _lib.lib()
    ws = _WORKSPACES.get((device.index, torch.cuda.current_stream(device).cuda_stream))
    if ws is None:
        return 0
    torch.cuda.current_stream(device).synchronize()
    off = int(L.gl_matmul_status_offset())
    code = int(ws[off:off + 4].view(torch.int32).item())
    if code != 0 and clear:
        ws[: int(L.gl_matmul_counter_bytes())].zero_()
    return code


def _make_scale_atoms(scales):
    """MX / NV weight scales [N, G] as 128x4 scale atoms (the reference's 5-D pre-shuffle,
    gemlite/core.py:748-752): [N/128, G/4, 32, 4, 4] bytes.  None when the shape does not tile."""
    if scales is None or scales.dim() != 2:
        return None
    N, G = scales.shape
    if N % 128 != 0 or G % 4 != 0:
        return None
    s2d = scales.view(torch.uint8) if scales.dtype != torch.uint8 else scales
    return s2d.contiguous().view(N // 128, 4, 32, G // 4, 4).permute(0, 3, 2, 1, 4).contiguous()


def _scale_atoms_of(scales):
    """The 128x4-atom copy of MX / NV weight scales, kept as an attribute of the scales tensor itself (so that it lives
    and dies with it and `get_tensor_args()` stays the reference's four tensors); rebuilt when the tensor was
    modified in place or the attribute is missing (a tensor that did not come from `get_tensor_args()`)."""
    if scales is None or scales.dim() != 2:
        return None
    key = (scales.data_ptr(), scales._version, tuple(scales.shape), tuple(scales.stride()))
    cached = getattr(scales, "_gl_scale_atoms", None)
    if cached is None or cached[0] != key:
        cached = (key, _make_scale_atoms(scales))
        try:
            scales._gl_scale_atoms = cached
        except Exception:       # a tensor subclass that refuses attributes: recomputed per call
            pass
    return cached[1]


def _fill_args(x2d, bias, W_q, scales, zeros, scales_x, meta_scale, out, meta_args, matmul_type, w_atoms=None, sx_layout=0):
    (_, W_nbits, group_size, _, eps, input_dtype, output_dtype, _, meta_dtype, channel_scale_mode,
     W_group_mode, _) = meta_args
    a = _lib.GLMatmulArgs()
    mx = is_mx_dtype(input_dtype)
    K_words, N = W_q.shape
    M = x2d.shape[0]
    a.x = x2d.data_ptr()
    a.w = W_q.data_ptr()
    has_scales = scales is not None and scales.numel() > 0
    has_zeros = zeros is not None and zeros.numel() > 0
    a.scales = scales.data_ptr() if has_scales else None
    a.zeros = zeros.data_ptr() if has_zeros else None
    a.scales_x = None if scales_x is None else scales_x.data_ptr()
    a.bias = None if bias is None else bias.data_ptr()
    a.meta_scale = None if meta_scale is None else meta_scale.data_ptr()
    a.out = out.data_ptr()
    a.M, a.N, a.K = M, N, K_words * eps
    a.W_nbits, a.group_size, a.elements_per_sample = W_nbits, group_size, eps
    a.input_dtype = input_dtype
    a.x_dtype = _lib.dtype_code(x2d)
    a.w_dtype = _lib.dtype_code(W_q)
    a.out_dtype = output_dtype
    a.meta_dtype = _lib.dtype_code(scales) if has_scales else meta_dtype
    a.zeros_dtype = _lib.dtype_code(zeros) if has_zeros else DType.INT32.value
    a.channel_scale_mode, a.W_group_mode = channel_scale_mode, W_group_mode
    a.zero_is_scalar = int(has_zeros and zeros.numel() == 1)
    a.matmul_type = matmul_type
    a.kernel_override = _KERNEL_OVERRIDE
    a.sx_layout = sx_layout
    a.w_scales_atoms = None if w_atoms is None else w_atoms.data_ptr()
    a.w_stride_k, a.w_stride_n = W_q.stride(0), W_q.stride(1)
    if has_scales and scales.dim() == 2:
        if mx:   # logical [N, G]
            a.s_stride_n, a.s_stride_g = scales.stride(0), scales.stride(1)
        else:    # logical [G, N]
            a.s_stride_g, a.s_stride_n = scales.stride(0), scales.stride(1)
    elif has_scales and scales.dim() > 2:
        raise NotImplementedError("pre-shuffled 5-D MX scales are not supported; store them as [N, K/group]")
    else:
        a.s_stride_g, a.s_stride_n = N, 1
    return a


# ---------------------------------------------------------------------------------------------
# Functional forward (custom op so that torch.compile / CUDA-graph capture see one opaque node)
# ---------------------------------------------------------------------------------------------
def _forward_impl(
    x: Tensor,
    bias: Union[None, Tensor],
    tensor_args: List[Tensor],
    meta_args: List[int],
    matmul_type: int = -1,  # -1: auto, >= 0: index into GEMLITE_MATMUL_TYPES
) -> Tensor:
    _lib.require_cuda(x, "x")
    W_q, scales, zeros, layer_meta_scale = tensor_args[0], tensor_args[1], tensor_args[2], tensor_args[3]
    out_features = W_q.shape[1]
    if not x.is_contiguous():
        x = x.contiguous()
    out_shape = x.shape[:-1] + (out_features,)
    input_dtype = DType(meta_args[5])
    channel_scale_mode = meta_args[9]

    scales_x, meta_scale = None, None
    # block-scaled fp4 layers: the derived copy of the weight scales as 128x4 scale atoms rides on the scales tensor
    w_atoms = None
    if _KERNEL_OVERRIDE != 1 and channel_scale_mode == 4 and input_dtype in (DType.MXFP4, DType.NVFP4, DType.MXFP8):
        w_atoms = _scale_atoms_of(scales)
    sx_layout = 0 if w_atoms is None else 1
    if _KERNEL_OVERRIDE != 1 and channel_scale_mode == 2 and input_dtype == DType.MXFP8 and meta_args[1] == 8:
        w_atoms = _scale_atoms_of(scales)      # MXFP8 weights, activations scaled per token: weight atoms only
    if bool(meta_args[0]) and enable_activation_scaling(x.numel() // x.shape[-1]):
        if input_dtype in FP8_INT8_DTYPES and channel_scale_mode == 5:
            x, scales_x = scale_activations_per_block(x, w_dtype=DTYPE_TO_TORCH[input_dtype.value])
        elif input_dtype in FP8_INT8_DTYPES:
            x, scales_x = scale_activations_per_token(x, w_dtype=DTYPE_TO_TORCH[input_dtype.value])
        elif input_dtype == DType.MXFP8 and channel_scale_mode == 4:
            x, scales_x = scale_activations_mxfp8(x, w_dtype=torch.float8_e4m3fn, scale_layout=sx_layout)
        elif input_dtype == DType.MXFP8 and channel_scale_mode == 2:
            x, scales_x = scale_activations_per_token(x, w_dtype=torch.float8_e4m3fn)
        elif input_dtype == DType.MXFP4 and channel_scale_mode == 4:
            x, scales_x = scale_activations_mxfp4(x, scale_layout=sx_layout)
        elif input_dtype == DType.NVFP4 and channel_scale_mode == 4:
            static_meta = GEMLITE_NVFP4_INPUT_SCALES.get(W_q.data_ptr()) if GEMLITE_NVFP4_INPUT_SCALES else None
            if static_meta is None and GEMLITE_FAST_NVFP4:
                static_meta = GEMLITE_NVFP4_META_SCALES[x.device.index]
            x, scales_x, meta_a = scale_activations_nvfp4(x, meta_scale=static_meta, scale_layout=sx_layout)
            meta_scale = (1.0 / (layer_meta_scale * meta_a)).reshape(1)   # stays on the device (graph-safe)
    if meta_scale is None and meta_args[2] == 16 and is_mx_dtype(input_dtype):
        meta_scale = layer_meta_scale.reshape(1)   # weight-only NVFP4: stored tensor scale

    x2d = x.view(-1, x.shape[-1])
    out = torch.empty((x2d.shape[0], out_features), dtype=DTYPE_TO_TORCH[meta_args[6]], device=x.device)
    if x2d.shape[0] == 0:
        return out.view(out_shape)
    if bias is not None and bias.dtype != out.dtype:
        bias = bias.to(out.dtype)
    a = _fill_args(x2d, bias, W_q, scales, zeros, scales_x, meta_scale, out, meta_args, matmul_type, w_atoms, sx_layout)
    L = _lib.lib()
    with torch.cuda.device(x.device):
        ws = _workspace(x.device, int(L.gl_matmul_workspace_bytes(ctypes.byref(a))))
        if ws is not None:
            a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        status = L.gl_matmul(ctypes.byref(a), _lib.current_stream_ptr(x.device))
    if status != 0:
        msg = L.gl_last_error().decode("utf-8", "replace")
        if status == _lib.GL_E_UNSUPPORTED:
            raise Exception(msg)
        _lib.check(status)
    return out.view(out_shape)


# the operator the reference registers (gemlite/core.py:193); eager module calls go to _forward_impl directly
forward_functional = torch.library.custom_op("gemlite::forward_functional", mutates_args=())(_forward_impl)


@torch.library.register_fake("gemlite::forward_functional")
def forward_functional_fake(x, bias, tensor_args, meta_args, matmul_type=-1):
    out_features = tensor_args[0].shape[1]
    return torch.empty(x.shape[:-1] + (out_features,), device=x.device, dtype=DTYPE_TO_TORCH[meta_args[6]])


# ---------------------------------------------------------------------------------------------
# Module
# ---------------------------------------------------------------------------------------------
class GemLiteLinear(torch.nn.Module):
    SUPPORTED_BITS_TRITON = [1, 2, 4, 8, 16]   # name kept for callers that read it
    SUPPORTED_DTYPES = [DType.FP16, DType.BF16, DType.FP32, DType.FP8, DType.FP8e4, DType.FP8e4nuz, DType.FP8e5,
                        DType.FP8e5nuz, DType.INT8, DType.MXFP16, DType.MXBF16, DType.MXFP8, DType.MXFP4, DType.NVFP4]
    MIN_SIZE = 32
    PACKING_BITWIDTH = 32
    _SCHEMA = ("W_q", "bias", "scales", "zeros", "metadata", "orig_shape", "meta_scale")
    _PACK_MUTATED_NAMES = ("W_q", "scales", "zeros", "bias")

    def __init__(self, W_nbits=4, group_size=64, in_features=None, out_features=None, input_dtype=DType.FP16,
                 output_dtype=DType.FP16, acc_dtype=None, scaled_activations=False):
        super().__init__()
        if W_nbits not in GemLiteLinear.SUPPORTED_BITS_TRITON:
            raise NotImplementedError("Only " + str(GemLiteLinear.SUPPORTED_BITS_TRITON) + " W_nbits are supported.")
        if in_features is not None and out_features is not None:
            bad_group = (in_features % group_size != 0) if (group_size is not None and W_nbits < 16) else False
            if (in_features % GemLiteLinear.MIN_SIZE != 0) or bad_group:
                raise NotImplementedError(
                    "Invalid input shapes: " + str(in_features) + " , " + str(out_features)
                    + ". in_features should be divisible by 32 or the group_size")
        if input_dtype not in GemLiteLinear.SUPPORTED_DTYPES:
            raise NotImplementedError("Unsupport input dtype: " + str(input_dtype))
        if group_size is not None and group_size < 16:
            raise NotImplementedError("Only group_size >= 16 is supported.")
        group_size = 1 if (group_size is None) else group_size

        self.in_features, self.out_features = in_features, out_features
        self.W_nbits, self.group_size = W_nbits, group_size
        self.unpack_mask = 2 ** W_nbits - 1
        self.elements_per_sample = None
        self.signature = (in_features, out_features, W_nbits, group_size)
        self.input_dtype, self.output_dtype = input_dtype, output_dtype
        self.compute_dtype = DTYPE_TO_TORCH[input_dtype.value]
        self.meta_dtype = input_dtype
        self.acc_dtype = GEMLITE_ACC_DTYPE[input_dtype] if (acc_dtype is None) else acc_dtype
        # 16/32-bit float inputs are never re-quantised (core.py:371-374)
        self.scaled_activations = False if self.compute_dtype in (torch.float16, torch.bfloat16, torch.float32) else scaled_activations
        self.forward = self.forward_auto_no_warmup

        # checkpoint schema is visible on a fresh module (empty placeholders), core.py:379-389
        self.register_buffer("W_q", torch.empty(0, dtype=torch.uint8))
        self.register_buffer("scales", torch.empty(0, dtype=torch.uint8))
        self.register_buffer("zeros", torch.empty(0, dtype=torch.int32))
        self.register_buffer("metadata", torch.empty(0, dtype=torch.int32))
        self.register_buffer("orig_shape", torch.empty(0, dtype=torch.int32))
        self.register_buffer("meta_scale", torch.tensor(0.0, dtype=torch.float32))
        self.register_parameter("bias", None)

    # -- slot helpers: nn.Module types its attributes, pack() needs to stash plain values ----
    def _clear_slot(self, name):
        self._buffers.pop(name, None)
        self._parameters.pop(name, None)
        self.__dict__.pop(name, None)

    def _clear_pack_slots(self):
        self.__dict__.pop("_atoms_cache", None)
        self.__dict__.pop("_arg_cache", None)
        for name in self._PACK_MUTATED_NAMES:
            self._clear_slot(name)

    def _promote_to_parameter(self, name, tensor):
        self._clear_slot(name)
        self.register_parameter(name, torch.nn.Parameter(tensor, requires_grad=False))

    def _register_none_param(self, name):
        self._clear_slot(name)
        self.register_parameter(name, None)

    # -- (de)serialisation ------------------------------------------------------------------
    def _save_to_state_dict(self, destination, prefix, keep_vars):
        # metadata is rebuilt from the live attributes: helpers change the modes after pack()
        if isinstance(self.W_q, torch.Tensor) and self.W_q.numel() > 0 and hasattr(self, "W_nbits"):
            self._promote_to_parameter("metadata", torch.tensor(self.get_meta_args(), device=self.W_q.device, dtype=torch.int32))
        super()._save_to_state_dict(destination, prefix, keep_vars)

    def _apply_state_dict(self, sd):
        W_q, bias, scales, zeros = sd.get("W_q"), sd.get("bias"), sd.get("scales"), sd.get("zeros")
        metadata, orig_shape, meta_scale = sd.get("metadata"), sd.get("orig_shape"), sd.get("meta_scale")
        if metadata is None or orig_shape is None or W_q is None:
            raise RuntimeError("GemLite checkpoint is missing required keys (W_q / metadata / orig_shape). "
                               "Got keys: %s" % sorted(k for k, v in sd.items() if v is not None))
        md = [int(v) for v in metadata.tolist()]
        (sa, self.W_nbits, self.group_size, self.unpack_mask, self.elements_per_sample, idt, odt, adt, mdt,
         self.channel_scale_mode, self.W_group_mode, dc) = md
        self.input_dtype, self.output_dtype = DType(idt), DType(odt)
        self.acc_dtype, self.meta_dtype = DType(adt), DType(mdt)
        self.scaled_activations, self.data_contiguous = bool(sa), bool(dc)
        self.out_features, self.in_features = (int(v) for v in orig_shape.tolist())
        self.compute_dtype = DTYPE_TO_TORCH[self.input_dtype.value]
        if meta_scale is not None:
            ms = float(meta_scale.float().item()) if isinstance(meta_scale, torch.Tensor) else float(meta_scale)
        else:   # checkpoints older than the meta_scale key
            ms = 0.05 if self.input_dtype == DType.NVFP4 else 0.0
        if is_mx_dtype(self.input_dtype) and scales is not None and scales.dim() == 5:
            # undo the reference's 5-D TMA pre-shuffle [1, N/128, G/4, 2, 256] -> [N, G] (core.py:748-752)
            _, n128, g4, _, _ = scales.shape
            scales = scales.reshape(n128, g4, 32, 4, 4).permute(0, 3, 2, 1, 4).reshape(n128 * 128, g4 * 4)
        dev = W_q.device
        self.__dict__.pop("_atoms_cache", None)
        self._promote_to_parameter("W_q", W_q)
        if bias is not None:
            self._promote_to_parameter("bias", bias)
        else:
            self._register_none_param("bias")
        self._promote_to_parameter("scales", scales)
        self._promote_to_parameter("zeros", zeros)
        self._promote_to_parameter("metadata", torch.tensor(self.get_meta_args(), device=dev, dtype=torch.int32))
        self._promote_to_parameter("orig_shape", torch.tensor([self.out_features, self.in_features], device=dev, dtype=torch.int32))
        self._promote_to_parameter("meta_scale", torch.tensor(ms, device=dev, dtype=torch.float32))

    def load_state_dict(self, state_dict, strict=True, assign=False):
        sd = {k: state_dict.pop(k, None) for k in self._SCHEMA}
        state_dict.pop("scales_5d", None)
        self._apply_state_dict(sd)

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
        sd = {}
        for k in self._SCHEMA:
            if prefix + k in state_dict:
                sd[k] = state_dict.pop(prefix + k)
        state_dict.pop(prefix + "scales_5d", None)
        if "W_q" not in sd:
            super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs)
            return
        try:
            self._apply_state_dict(sd)
        except Exception as e:  # reported the way nn.Module reports loader errors
            error_msgs.append("GemLite load error at prefix '%s': %s" % (prefix, e))

    # -- packing ----------------------------------------------------------------------------
    def pack(self, W_q: Tensor, scales: Tensor, zeros: Union[Tensor, int], bias: Union[Tensor, None] = None,
             fma_mode: bool = True, contiguous: Union[int, None] = None, packing_bitwidth: Union[int, None] = None,
             packed: bool = False):
        """Store quantised weights in the kernel layout and resolve the dequantisation modes.

        ``W_q``: uint8 codes [N, K] (packed here), or int8 / fp8 / fp16 / bf16 / fp32 weights kept as
        they are, or, with ``packed=True``, uint8 bytes that already hold the packed codes."""
        self._clear_pack_slots()
        mx = is_mx_dtype(self.input_dtype)
        if zeros is not None and self.input_dtype == DType.INT8:
            if (isinstance(zeros, Tensor) and zeros.mean() != zeros.int().float().mean()) or isinstance(zeros, float):
                raise Exception("INT8 inputs is not compatible with floating-point zeros.")
        if packing_bitwidth is None:
            packing_bitwidth = GemLiteLinear.PACKING_BITWIDTH
        if mx:
            packing_bitwidth = 8   # block-scaled formats are byte-packed (core.py:593-594)

        N, K = self.out_features, self.in_features
        W_store = None
        if W_q.dtype == torch.int8 or W_q.is_floating_point():
            if W_q.dtype == torch.float32:
                assert self.W_nbits == 32, "Invalid fp32 weights."
            elif W_q.dtype in (torch.float16, torch.bfloat16):
                assert self.W_nbits == 16, "Invalid fp16 weights."
            else:
                assert self.W_nbits == 8, "Invalid 8-bit weights."
            W_store, self.elements_per_sample = W_q.t(), 1
            if contiguous is None:
                contiguous = False
        if packed and W_q.dtype == torch.uint8:
            self.elements_per_sample = packing_bitwidth // self.W_nbits
            W_store = W_q.view(N, K // self.elements_per_sample).t()
            if contiguous is None:
                contiguous = not mx
        elif W_q.dtype == torch.uint8:
            W_store, self.elements_per_sample = pack_weights_over_cols(
                W_q.view((N, K)), W_nbits=self.W_nbits, packing_bitwidth=packing_bitwidth, transpose=True)
            if contiguous is None:
                contiguous = not mx
        if W_store is None:
            raise Exception("Weights were not packed, please check your W_q.dtype")
        _lib.require_cuda(W_store, "W_q")

        self.device = W_store.device
        bias_t = None if bias is None else bias.to(device=self.device)

        # ---- dequantisation mode (core.py:646-703) ----
        scales_t = None if scales is None else scales.view((N, -1)).t()
        self.meta_is_channelwise = False if scales_t is None else scales_t.numel() == N
        self.W_group_mode, self.channel_scale_mode = -1, 0
        if scales is None and zeros is None:
            self.W_group_mode = 0
            self.channel_scale_mode = 2 if self.scaled_activations else 0
        zeros_t = None
        if zeros is None:
            self.W_group_mode = 2 if scales_t is not None else 0
        elif isinstance(zeros, torch.Tensor):
            if fma_mode and not self.meta_is_channelwise:      # W ~ W_q * s + (-z * s)
                zeros_t = (-zeros.float() * scales.float()).to(zeros.dtype).view((N, -1)).t()
                self.W_group_mode = 4
            else:                                              # W ~ (W_q - z) * s
                zeros_t = zeros.view((N, -1)).t()
                self.W_group_mode = 3
        else:
            zeros_t = int(zeros)
            self.W_group_mode = 3 if scales_t is not None else 1
        assert self.W_group_mode > -1, "Invalid scales/zeros settings."
        if (not self.scaled_activations) and self.meta_is_channelwise:
            self.channel_scale_mode = 1
            self.W_group_mode = 1 if zeros_t is not None else 0
        if self.scaled_activations and not self.meta_is_channelwise:
            self.channel_scale_mode = 2
        if self.scaled_activations and self.meta_is_channelwise:
            self.channel_scale_mode = 3
            self.W_group_mode = 1 if zeros_t is not None else 0
        if self.channel_scale_mode in [1, 3]:
            assert self.W_group_mode not in [3, 4], "Can't use channel_scale_mode with W_group_mode == 3 or 4."

        if isinstance(zeros_t, int):
            zeros_t = torch.tensor(zeros_t, dtype=torch.int32, device=self.device)
        if zeros_t is None:
            zeros_t = torch.tensor([[]], dtype=torch.int32, device=self.device)
        if scales_t is None:
            scales_t = torch.tensor([[]], dtype=torch.int32, device=self.device)

        self.data_contiguous = bool(contiguous)
        if contiguous:
            W_store = W_store.contiguous()
        scales_t, zeros_t = scales_t.contiguous(), zeros_t.contiguous()

        if self.input_dtype in (DType.MXFP16, DType.MXBF16, DType.MXFP8, DType.MXFP4):
            scales_t = scales_t.to(torch.float8_e8m0fnu).view(torch.uint8)
        if self.input_dtype == DType.NVFP4:
            scales_t = scales_t.to(torch.float8_e4m3fn)
        if mx:
            self.W_group_mode, self.channel_scale_mode = 2, 0
            scales_t = scales_t.T     # logical [N, G], memory stays [G, N] (core.py:753-755)
        if scales_t is not None:
            self.meta_dtype = TORCH_TO_DTYPE[scales_t.dtype]

        self._promote_to_parameter("W_q", W_store)
        self._promote_to_parameter("scales", scales_t)
        self._promote_to_parameter("zeros", zeros_t)
        if bias_t is not None:
            self._promote_to_parameter("bias", bias_t)
        else:
            self._register_none_param("bias")
        self._promote_to_parameter("metadata", torch.tensor(self.get_meta_args(), device=self.device, dtype=torch.int32))
        self._promote_to_parameter("orig_shape", torch.tensor([N, K], device=self.device, dtype=torch.int32))
        ms = self.meta_scale
        ms = float(ms.item()) if isinstance(ms, torch.Tensor) else float(ms)
        self._promote_to_parameter("meta_scale", torch.tensor(ms, device=self.device, dtype=torch.float32))
        return self

    # -- forward ----------------------------------------------------------------------------
    def get_tensor_args(self):
        meta_scale = self.meta_scale
        if not isinstance(meta_scale, torch.Tensor):
            meta_scale = torch.tensor(meta_scale, dtype=torch.float32, device=self.W_q.device)
        if self.channel_scale_mode == 4 and self.input_dtype in (DType.MXFP4, DType.NVFP4):
            _scale_atoms_of(self.scales)      # derived layout for the block-scaled tensor-core kernel, built once
        return [self.W_q, self.scales, self.zeros, meta_scale]

    def _scale_atoms(self):
        """Derived, non-serialised copy of the MX / NV weight scales in the layout the block-scaled tensor-core
        kernel reads; rebuilt when the stored scales change."""
        return _scale_atoms_of(self.scales)

    def get_meta_args(self):
        return [int(self.scaled_activations), self.W_nbits, self.group_size, self.unpack_mask, self.elements_per_sample,
                self.input_dtype.value, self.output_dtype.value, self.acc_dtype.value, self.meta_dtype.value,
                self.channel_scale_mode, self.W_group_mode, int(self.data_contiguous)]

    def forward_manual(self, x: Tensor, matmul_type: str = "GEMM") -> Tensor:
        return self._forward(x, GEMLITE_MATMUL_TYPES_MAPPING[matmul_type])

    def forward_auto_no_warmup(self, x: Tensor) -> Tensor:
        return self._forward(x, -1)

    def _forward(self, x: Tensor, matmul_type: int) -> Tensor:
        """Module call.  Under torch.compile the registered operator is used (one opaque node); in eager mode the
        dispatcher is skipped, and layers without activation quantisation re-use a filled argument struct per
        (batch rows, dtype, family): only the x / out / workspace pointers change between calls."""
        if torch.compiler.is_compiling():
            return forward_functional(x, self.bias, self.get_tensor_args(), self.get_meta_args(), matmul_type)
        if self.scaled_activations or is_mx_dtype(self.input_dtype) or _KERNEL_OVERRIDE != 0 or x.device.type != "cuda":
            return _forward_impl(x, self.bias, self.get_tensor_args(), self.get_meta_args(), matmul_type)
        if not x.is_contiguous():
            x = x.contiguous()
        x2d = x.view(-1, x.shape[-1])
        M = x2d.shape[0]
        W_q, scales, zeros, bias = self.W_q, self.scales, self.zeros, self.bias
        out_dtype = DTYPE_TO_TORCH[self.output_dtype.value]
        if bias is not None and bias.dtype != out_dtype:
            return _forward_impl(x, bias, self.get_tensor_args(), self.get_meta_args(), matmul_type)
        out = torch.empty((M, W_q.shape[1]), dtype=out_dtype, device=x.device)
        if M == 0:
            return out.view(x.shape[:-1] + (W_q.shape[1],))
        sig = (W_q.data_ptr(), scales.data_ptr(), zeros.data_ptr(), 0 if bias is None else bias.data_ptr(),
               self.W_group_mode, self.channel_scale_mode, self.output_dtype)
        cache = self.__dict__.setdefault("_arg_cache", {})
        key = (M, x2d.dtype, matmul_type, x.device.index)
        ent = cache.get(key)
        L = _lib.lib()
        if ent is None or ent[0] != sig:
            a = _fill_args(x2d, bias, W_q, scales, zeros, None, None, out, self.get_meta_args(), matmul_type)
            with torch.cuda.device(x.device):
                need = int(L.gl_matmul_workspace_bytes(ctypes.byref(a)))
            if len(cache) > 64:
                cache.clear()
            ent = (sig, a, need)
            cache[key] = ent
        a, need = ent[1], ent[2]
        a.x, a.out = x2d.data_ptr(), out.data_ptr()
        sp = _lib.current_stream_ptr(x.device)
        if torch.cuda.current_device() == x.device.index:      # the usual case: no device switch around the launch
            ws = _workspace(x.device, need, sp)
            if ws is not None:
                a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
            status = L.gl_matmul(ctypes.byref(a), sp)
        else:
            with torch.cuda.device(x.device):
                ws = _workspace(x.device, need, sp)
                if ws is not None:
                    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
                status = L.gl_matmul(ctypes.byref(a), sp)
        if status != 0:
            msg = L.gl_last_error().decode("utf-8", "replace")
            if status == _lib.GL_E_UNSUPPORTED:
                raise Exception(msg)
            _lib.check(status)
        return out.view(x.shape[:-1] + (W_q.shape[1],))

    # -- tile-config cache (core.py:838-906), kept in the C library --------------------------
    @staticmethod
    def cache_config(filename: str):
        with FILE_LOCK:
            _lib.check(_lib.lib().gl_cfg_save(os.fsencode(filename)))

    @staticmethod
    def load_config(filename: str, print_error: bool = True, overwrite: bool = False):
        if filename is None:
            return False
        with FILE_LOCK:
            status = _lib.lib().gl_cfg_load(os.fsencode(filename), int(bool(overwrite)))
        if status != 0:
            if print_error:
                logger.error(_lib.lib().gl_last_error().decode("utf-8", "replace"))
            return False
        return True

    @staticmethod
    def reset_config():
        _lib.lib().gl_cfg_reset()


GemLiteLinearTriton = GemLiteLinear   # the reference's class name (core.py:289, 910)


def get_default_cache_config():
    """Shipped config whose tag is contained in the GPU name (longest tag wins), core.py:913-929."""
    root = os.path.join(os.path.dirname(os.path.abspath(__file__)), "configs")
    if not os.path.isdir(root) or not torch.cuda.is_available():
        return None
    name = torch.cuda.get_device_properties(0).name.lower().replace(" ", "_")
    tags = sorted((f.split(".")[0] for f in os.listdir(root) if f.endswith(".json")), key=len, reverse=True)
    for tag in tags:
        if tag in name:
            return os.path.join(root, tag + ".json")
    return None
