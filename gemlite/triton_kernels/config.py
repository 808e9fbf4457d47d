"""The two knobs of gemlite/triton_kernels/config.py that callers of the reference touch.

`KERNEL_CACHE` steered the reference's ring of pre-zeroed outputs for its atomics-based GEMV
(gemlite/triton_kernels/gemv_kernels.py:622-647); the CUDA kernels write every output once, so the switch is
recorded and has no effect.  `set_autotune` / `set_kernel_caching` forward to the package-level setters."""
from gemlite_b200.core import set_autotune, set_kernel_caching as _set_kernel_caching


class KERNEL_CACHE:
    ENABLE = False
    CACHE_SIZE = 256
    CACHE = {}


def set_kernel_caching(enable: bool):
    KERNEL_CACHE.ENABLE = bool(enable)
    _set_kernel_caching(enable)
