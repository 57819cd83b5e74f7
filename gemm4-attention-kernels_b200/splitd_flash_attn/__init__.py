"""B200 (sm_100a) SplitD FlashAttention for head_dim 512; same import surface as the reference's
``splitd_flash_attn`` package (splitd-flash-attn/src/__init__.py:3-10)."""

from .interface import split_flash_attn_func, split_flash_attn_varlen_func

__version__ = "0.1.0"

__all__ = ["split_flash_attn_func", "split_flash_attn_varlen_func"]
