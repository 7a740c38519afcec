"""worldattention_b200: the HSA / HKV inference hot path of WorldAttention as sm_100a CUDA.

`hsa` mirrors the reference's `wan.modules.hsa`, `hkv` mirrors `pipeline.hkv`, `hsa_stage` the
helpers of `trainer.hsa_stage` that inference users need.  `install_reference_aliases()` registers
those reference module paths so existing imports resolve to this package.
"""
from . import _lib, hkv, hsa, hsa_stage  # noqa: F401
from .compat import install_reference_aliases  # noqa: F401

__version__ = "0.1.0"
