"""ctypes binding of ``libgemlite_b200.so`` (the C ABI declared in ``include/gemlite_b200.h``).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
import ctypes
import os

import torch

from .dtypes import TORCH_TO_DTYPE

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libgemlite_b200.so")

GL_OK, GL_E_INVALID, GL_E_UNSUPPORTED, GL_E_WORKSPACE, GL_E_CUDA, GL_E_IO, GL_E_NOTFOUND = 0, -1, -2, -3, -4, -5, -6

c_void_p, c_int32, c_int64, c_uint64, c_char_p = (
    ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_uint64, ctypes.c_char_p)


class GLMatmulArgs(ctypes.Structure):
    """Mirror of ``struct gl_matmul_args``."""
    _fields_ = [
        ("x", c_void_p), ("w", c_void_p), ("scales", c_void_p), ("zeros", c_void_p),
        ("scales_x", c_void_p), ("bias", c_void_p), ("meta_scale", c_void_p), ("out", c_void_p),
        ("workspace", c_void_p), ("workspace_bytes", c_uint64),
        ("M", c_int32), ("N", c_int32), ("K", c_int32),
        ("W_nbits", c_int32), ("group_size", c_int32), ("elements_per_sample", c_int32),
        ("input_dtype", c_int32), ("x_dtype", c_int32), ("w_dtype", c_int32), ("out_dtype", c_int32),
        ("meta_dtype", c_int32), ("zeros_dtype", c_int32),
        ("channel_scale_mode", c_int32), ("W_group_mode", c_int32), ("zero_is_scalar", c_int32),
        ("matmul_type", c_int32),
        ("w_stride_k", c_int64), ("w_stride_n", c_int64), ("s_stride_g", c_int64), ("s_stride_n", c_int64),
        ("kernel_override", c_int32), ("sx_layout", c_int32), ("reserved", c_int32 * 2),
        ("w_scales_atoms", c_void_p),
    ]


class GLTpComm(ctypes.Structure):
    """Mirror of ``struct gl_tp_comm``."""
    _fields_ = [("rank", c_int32), ("world", c_int32), ("slot_bytes", c_uint64), ("wait_cycles", c_uint64),
                ("buffers", c_void_p * 8)]


# name -> (restype, argtypes); every symbol include/gemlite_b200.h declares
SIGNATURES = {
    "gl_abi_version": (c_int32, []),
    "gl_last_error": (c_char_p, []),
    "gl_build_info": (c_char_p, []),
    "gl_get_matmul_type": (c_int32, [c_int32, c_int32, c_int32]),
    "gl_matmul_workspace_bytes": (c_uint64, [ctypes.POINTER(GLMatmulArgs)]),
    "gl_matmul_counter_bytes": (c_uint64, []),
    "gl_matmul_status_offset": (c_uint64, []),
    "gl_matmul": (c_int32, [ctypes.POINTER(GLMatmulArgs), c_void_p]),
    "gl_matmul_kernel_name": (c_char_p, [ctypes.POINTER(GLMatmulArgs)]),
    "gl_matmul_noalloc": (c_int32, [ctypes.POINTER(GLMatmulArgs), c_void_p]),
    "gl_pack_over_cols": (c_int32, [c_void_p, c_void_p, c_int64, c_int64, c_int32, c_int32, c_void_p]),
    "gl_pack_over_rows": (c_int32, [c_void_p, c_void_p, c_int64, c_int64, c_int32, c_int32, c_void_p]),
    "gl_unpack_over_cols": (c_int32, [c_void_p, c_void_p, c_int64, c_int64, c_int32, c_int32, c_int32, c_int32, c_void_p]),
    "gl_unpack_over_rows": (c_int32, [c_void_p, c_void_p, c_int64, c_int64, c_int32, c_int32, c_int32, c_int32, c_void_p]),
    "gl_scale_activations_per_token": (c_int32, [c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32, c_void_p]),
    "gl_scale_activations_per_block": (c_int32, [c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32, c_void_p]),
    "gl_scale_activations_mxfp4": (c_int32, [c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32, c_void_p]),
    "gl_scale_activations_mxfp8": (c_int32, [c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32, c_void_p]),
    "gl_scale_activations_nvfp4": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32, c_void_p]),
    "gl_cfg_load": (c_int32, [c_char_p, c_int32]),
    "gl_cfg_save": (c_int32, [c_char_p]),
    "gl_cfg_reset": (None, []),
    "gl_cfg_set": (c_int32, [c_char_p, c_char_p, c_char_p]),
    "gl_cfg_get": (c_char_p, [c_char_p, c_char_p]),
    "gl_cfg_size": (c_int64, [c_char_p]),
    "gl_get_closest_m": (c_int32, [c_int32]),
    "gl_tp_buffer_bytes": (c_uint64, [c_int32, c_uint64]),
    "gl_tp_buffer_create": (c_int32, [c_uint64, ctypes.POINTER(c_void_p), c_void_p]),
    "gl_tp_buffer_open": (c_int32, [c_void_p, ctypes.POINTER(c_void_p)]),
    "gl_tp_buffer_close": (c_int32, [c_void_p]),
    "gl_tp_buffer_destroy": (c_int32, [c_void_p]),
    "gl_tp_allreduce": (c_int32, [ctypes.POINTER(GLTpComm), c_void_p, c_void_p, c_int64, c_int32, c_int32, c_void_p]),
    "gl_tp_status": (c_int32, [ctypes.POINTER(GLTpComm), ctypes.POINTER(c_int32), ctypes.POINTER(ctypes.c_uint32)]),
    "gl_silu_mul": (c_int32, [c_void_p, c_void_p, c_int32, c_int32, c_int32, c_void_p]),
    "gl_mma_peak": (c_int32, [c_int32, c_int32, c_void_p, ctypes.POINTER(ctypes.c_double), c_void_p]),
}

_lib = None


class GemliteB200Error(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, code, message):
        super().__init__("gemlite_b200 error %d: %s" % (code, message))
        self.code = code


def lib():
    """The loaded library; raises if it has not been built (``python -m gemlite_b200.build``)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                "gemlite_b200: %s not found. Build it with `python -m gemlite_b200.build` "
                "(nvcc, sm_100a). There is no fallback implementation." % LIB_PATH)
        handle = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
        _load_shipped_config(handle)
    return _lib


def _load_shipped_config(handle):
    """Tile-config table shipped for this GPU (configs/<tag>.json, the tag contained in the device name, longest tag
    first), loaded once when the library is first used: what the reference does at import (gemlite/core.py:913-933).
    GEMLITE_B200_NO_SHIPPED_CONFIG=1 skips it."""
    if os.environ.get("GEMLITE_B200_NO_SHIPPED_CONFIG") or not torch.cuda.is_available():
        return
    root = os.path.join(_HERE, "configs")
    if not os.path.isdir(root):
        return
    try:
        name = torch.cuda.get_device_properties(torch.cuda.current_device()).name.lower().replace(" ", "_")
    except Exception:
        return
    for tag in sorted((f[:-5] for f in os.listdir(root) if f.endswith(".json")), key=len, reverse=True):
        if tag in name:
            handle.gl_cfg_load(os.fsencode(os.path.join(root, tag + ".json")), 0)
            return


def check(status):
    """Turn a C status into an exception of the type the reference raises for that case."""
    if status == GL_OK:
        return
    msg = lib().gl_last_error().decode("utf-8", "replace")
    if status == GL_E_UNSUPPORTED:
        raise NotImplementedError(msg)
    if status == GL_E_INVALID:
        raise ValueError(msg)
    raise GemliteB200Error(status, msg)


def require_cuda(t, what):
    if not isinstance(t, torch.Tensor) or t.device.type != "cuda":
        raise RuntimeError(
            "gemlite_b200: %s must be a CUDA tensor; the kernels are CUDA-only and there is no CPU path." % what)


_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def current_stream_ptr(device):
    """cudaStream_t of torch's current stream on `device` (the raw getter skips building a Stream object per call)."""
    if _RAW_STREAM is not None and device.index is not None:
        return _RAW_STREAM(device.index)
    return torch.cuda.current_stream(device).cuda_stream


def dtype_code(t):
    """DType integer of a tensor's dtype."""
    return TORCH_TO_DTYPE[t.dtype].value


def ptr(t):
    return None if t is None else t.data_ptr()
