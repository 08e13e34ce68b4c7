"""diffcache_b200 — B200-native retrieval-attention engine for DiffCache's decode hot path.

Drop-in for the reference's Rust offload engine ``diffcache._cpu``
(diffcache_cpu/src/lib.rs:523-672): ``DiffCacheGPU`` has the methods of
``DiffCacheCPU`` and ``DiffCache`` the API of src/diffcache/kvcache/diffcache.py,
both backed by hand-written sm_100a CUDA kernels behind a C ABI
(include/diffcache_b200.h).  There is no CPU fallback.
"""
from ._lib import DiffCacheError, load as load_library
from .engine import BF16, FP16, DiffCacheGPU, init_metrics
from .kvcache import DiffCache

__all__ = ["DiffCacheGPU", "DiffCache", "DiffCacheError", "init_metrics", "load_library", "BF16", "FP16"]
