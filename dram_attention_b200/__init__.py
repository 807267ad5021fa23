"""B200-native implementation of the generate stage of DRAM Attention.

Exports the same names as the reference package (dram_attention/__init__.py:3-13)."""

__version__ = "0.1.0"

from .dram_attention import DRAMAttention
from .lru_cache import CacheOutput, LRUCache
from .max_ip import max_inner_product, max_ip_ref

__all__ = (
    "CacheOutput",
    "DRAMAttention",
    "LRUCache",
    "max_inner_product",
    "max_ip_ref",
)
