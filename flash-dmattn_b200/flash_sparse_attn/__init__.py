"""B200-native dynamic-mask attention behind the reference's `flash_sparse_attn` import paths.

`from flash_sparse_attn import flash_sparse_attn_func` and
`from flash_sparse_attn.utils.mask import create_mask` work as with the reference package
(flash_sparse_attn/__init__.py:9-14); the Triton / Flex backends and the `_auto` selector are not part of
this build.
"""
__version__ = "1.0.0"

from .flash_sparse_attn_interface import (FlashDMAttnFunc, flash_sparse_attn_func,  # noqa: F401
                                          flash_sparse_attn_varlen_func)
from .compaction import compact_keys, flash_sparse_attn_compact_func  # noqa: F401
from .packed import PackedMask, pack_mask  # noqa: F401

CUDA_AVAILABLE = True
TRITON_AVAILABLE = False
FLEX_AVAILABLE = False
