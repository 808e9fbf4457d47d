"""gemlite_b200: sm_100a CUDA implementation of GemLite's low-bit matmul path behind the
GemLite Python API (``GemLiteLinear``, ``DType``, ``helper`` processors)."""
__version__ = "0.1.0"

from .dtypes import DType
from .core import (
    GemLiteLinearTriton,
    GemLiteLinear,
    GEMLITE_ACC_DTYPE,
    GEMLITE_MATMUL_TYPES,
    set_autotune_setting,
    set_packing_bitwidth,
    set_acc_dtype,
    set_autotune,
    set_kernel_caching,
    enable_tma,
    enable_warp_specialize,
    set_native_atomic_bfp16,
    set_fast_gemv_acc,
    set_ptx_fp4_pack,
    enable_cudagraph_autotune,
    set_fast_nvfp4,
    forward_functional,
    get_matmul_type,
    get_closest_m,
    get_default_cache_config,
)
from . import helper


def auto_detect_ptx_fp4_pack():
    """The reference probes its ptxas for the e2m1x2 cvt; the CUDA kernels here always round by
    thresholds, so there is nothing to detect."""
    return False


load_config = GemLiteLinear.load_config
cache_config = GemLiteLinear.cache_config
reset_config = GemLiteLinear.reset_config
