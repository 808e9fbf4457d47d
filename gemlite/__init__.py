"""`gemlite`: the reference's import name, served by the sm_100a implementation in `gemlite_b200`.

Callers of the reference (`import gemlite`, `from gemlite.core import GemLiteLinearTriton`,
`from gemlite.helper import A16W4_HQQ_INT`, external packages such as hqq) bind here without a change;
`gemlite.core`, `.helper`, `.bitpack`, `.dtypes` and `.quant_utils` are the modules of `gemlite_b200` themselves,
not copies, so state such as the config cache is shared whichever name was imported.  The export list is the
reference's (gemlite/__init__.py:5-32).  There is no Triton code behind it: `gemlite.triton_kernels.config` only
keeps the two objects that callers of the reference poke (`KERNEL_CACHE`, `set_autotune`)."""
import importlib
import sys

import gemlite_b200 as _impl
from gemlite_b200 import *          # noqa: F401,F403
from gemlite_b200 import (DType, GemLiteLinear, GemLiteLinearTriton, GEMLITE_ACC_DTYPE, GEMLITE_MATMUL_TYPES, helper,
                          load_config, cache_config, reset_config, forward_functional, get_matmul_type, get_closest_m,
                          get_default_cache_config, auto_detect_ptx_fp4_pack, set_autotune_setting, set_packing_bitwidth,
                          set_acc_dtype, set_autotune, set_kernel_caching, enable_tma, enable_warp_specialize,
                          set_native_atomic_bfp16, set_fast_gemv_acc, set_ptx_fp4_pack, enable_cudagraph_autotune,
                          set_fast_nvfp4)

__version__ = _impl.__version__

for _name in ("core", "helper", "bitpack", "dtypes", "quant_utils"):
    _mod = importlib.import_module("gemlite_b200." + _name)
    sys.modules[__name__ + "." + _name] = _mod
    globals()[_name] = _mod
del _name, _mod
