"""Inference engine: paged KV per iteration depth, iteration-level scheduling, CUDA-graph ticks."""
from tah_b200.engine.engine import GenerationResult, TaHEngine, get_engine
from tah_b200.engine.kv_cache import CacheGeometry, PagedKVCache

__all__ = ["TaHEngine", "GenerationResult", "get_engine", "PagedKVCache", "CacheGeometry"]
