"""Placeholder for the reference's kernel package: the kernels are CUDA (libgemlite_b200.so), there is no Triton
here.  Only `config` exists, for callers that set `KERNEL_CACHE.ENABLE` or call `set_autotune` through it."""
from . import config  # noqa: F401
