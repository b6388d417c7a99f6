"""flash_moba_b200 — B200-native MoBA sparse attention with the FlashMoBA Python API.

    from flash_moba_b200 import (flash_moba_varlen_func, flash_topk_varlen_func,
                                 flash_moba_attn_varlen_func)

Importing the package loads libflashmoba_b200.so (built by `python flash_moba_b200/build.py`)
and fails loudly if it is missing: there is no CPU or PyTorch fallback.
"""
__version__ = "0.1.0"

from .interface import (  # noqa: F401
    FlashMobaAttnVarlenFunc,
    decide_lg_block_m,
    flash_moba_attn_varlen_func,
    flash_moba_varlen_func,
    flash_topk_mean_pool,
    flash_topk_varlen_func,
)
from .modules import CentroidCache, MobaAttention  # noqa: F401

__all__ = [
    "flash_moba_varlen_func",
    "flash_topk_varlen_func",
    "flash_moba_attn_varlen_func",
    "flash_topk_mean_pool",
    "decide_lg_block_m",
    "FlashMobaAttnVarlenFunc",
    "MobaAttention",
    "CentroidCache",
]
